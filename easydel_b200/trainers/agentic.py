"""Agentic MoshPit: multi-turn, tool-using rollouts in text environments scored at episode end and trained with
the group-relative objective (easydel/trainers/agentic_moshpit).

Pieces: :class:`TextEnvironment` (protocol: ``reset() -> observation``, ``step(action) -> (observation, reward,
done, info)``), :class:`ToolEnvironment` (parses ``<tool>name(args)</tool>`` calls and answers with the tool's
output), :class:`EnvironmentManager` (a pit of environment instances stepped in lock step, with optional
self-play pairing) and :class:`AgenticMoshPitTrainer`, whose rollouts interleave model turns (trained, mask 1) and
environment turns (context only, mask 0).
"""

from __future__ import annotations

import re
import typing as tp
from dataclasses import dataclass

import torch

from .rl import GRPOConfig, GRPOTrainer, first_eos_mask, group_advantages
from .training_configurations import register_trainer, register_trainer_arguments
from .utils import pad_to_length


class TextEnvironment:
    """Base class of the environments; override :meth:`reset` and :meth:`step`."""

    def reset(self, task: tp.Any = None) -> str:
        raise NotImplementedError

    def step(self, action: str) -> tuple[str, float, bool, dict]:
        raise NotImplementedError


class ToolEnvironment(TextEnvironment):
    """Answers tool calls of the form ``<tool>name(arg text)</tool>``; ``<answer>..</answer>`` ends the episode and
    is scored by ``scorer(task, answer)``."""

    CALL = re.compile(r"<tool>\s*(\w+)\((.*?)\)\s*</tool>", re.S)
    ANSWER = re.compile(r"<answer>(.*?)</answer>", re.S)

    def __init__(self, tools: dict[str, tp.Callable[[str], str]], scorer: tp.Callable[[tp.Any, str], float],
                 max_turns: int = 4, prompt_key: str = "prompt"):
        self.tools, self.scorer, self.max_turns, self.prompt_key = tools, scorer, max_turns, prompt_key
        self.task, self.turn = None, 0

    def reset(self, task=None) -> str:
        self.task, self.turn = task, 0
        return task[self.prompt_key] if isinstance(task, dict) else str(task)

    def step(self, action: str):
        self.turn += 1
        ans = self.ANSWER.search(action)
        if ans:
            return "", float(self.scorer(self.task, ans.group(1).strip())), True, {"answered": True}
        call = self.CALL.search(action)
        if call and call.group(1) in self.tools:
            try:
                obs = f"<result>{self.tools[call.group(1)](call.group(2))}</result>"
            except Exception as e:  # noqa: BLE001
                obs = f"<result>error: {e}</result>"
        else:
            obs = "<result>no valid tool call or answer found</result>"
        done = self.turn >= self.max_turns
        return obs, 0.0, done, {"answered": False}


class EnvironmentManager:
    """Keeps ``n`` environment instances, resets them on tasks and steps the live ones together."""

    def __init__(self, factory: tp.Callable[[], TextEnvironment], n: int):
        self.envs = [factory() for _ in range(n)]

    def reset(self, tasks: list) -> list[str]:
        if len(tasks) != len(self.envs):
            raise ValueError(f"{len(tasks)} tasks for {len(self.envs)} environments")
        self.done = [False] * len(self.envs)
        self.returns = [0.0] * len(self.envs)
        return [e.reset(t) for e, t in zip(self.envs, tasks)]

    def step(self, actions: list[str]) -> list[str]:
        obs = []
        for i, (e, a) in enumerate(zip(self.envs, actions)):
            if self.done[i]:
                obs.append("")
                continue
            o, r, d, _ = e.step(a)
            self.returns[i] += r
            self.done[i] = d
            obs.append(o)
        return obs


@register_trainer_arguments("agentic-moshpit")
@dataclass
class AgenticMoshPitConfig(GRPOConfig):
    trainer_prefix: str | None = "agenticmoshpit"
    max_turns: int = 4
    max_turn_tokens: int = 64
    max_episode_tokens: int = 512
    task_key: str = "task"


@register_trainer("agentic-moshpit")
class AgenticMoshPitTrainer(GRPOTrainer):
    trainer_type = "agentic-moshpit"
    arguments_class = AgenticMoshPitConfig

    def __init__(self, arguments=None, model=None, env_factory: tp.Callable[[], TextEnvironment] | None = None,
                 processing_class=None, **kw):
        if env_factory is None:
            raise ValueError("`env_factory` is required")
        if processing_class is None or not hasattr(processing_class, "decode"):
            raise ValueError("the agentic trainer needs a tokenizer (`processing_class`) to talk to environments")
        self.env_factory = env_factory
        self._managers: dict[int, EnvironmentManager] = {}
        arguments = arguments or AgenticMoshPitConfig()
        super().__init__(arguments=arguments, model=model, reward_funcs=[lambda **k: [0.0]],
                         processing_class=processing_class, **kw)

    def _manager(self, n: int) -> EnvironmentManager:
        if n not in self._managers:
            self._managers[n] = EnvironmentManager(self.env_factory, n)
        return self._managers[n]

    def _encode(self, text: str) -> list[int]:
        return self.processing_class(text, add_special_tokens=False)["input_ids"] if text else []

    def _preprocess_batch_input(self, state, batch, is_train):
        a = self.arguments
        n = a.num_return_sequences
        tasks = batch.get(a.task_key)
        if tasks is None:
            tasks = self._decode(batch["input_ids"], batch["attention_mask"])
        tasks = [t for t in tasks for _ in range(n)]
        mgr = self._manager(len(tasks))
        obs = mgr.reset(tasks)
        ctx = [self._encode(o) for o in obs]            # token context per episode
        mask = [[0] * len(c) for c in ctx]              # 1 on model-generated tokens
        saved = a.max_completion_length
        a.max_completion_length = a.max_turn_tokens
        try:
            for _ in range(a.max_turns):
                live = [i for i, d in enumerate(mgr.done) if not d and len(ctx[i]) < a.max_episode_tokens]
                if not live:
                    break
                L = max(len(ctx[i]) for i in live)
                ids = torch.stack([pad_to_length(torch.tensor(ctx[i]), L, self.pad_token_id, left=True) for i in live])
                att = torch.stack([pad_to_length(torch.ones(len(ctx[i]), dtype=torch.long), L, 0, left=True)
                                   for i in live])
                comp, cm = self.sample_completions(ids, att, 1)
                actions = [""] * len(tasks)
                for j, i in enumerate(live):
                    toks = comp[j][cm[j].bool()].tolist()
                    ctx[i] += toks
                    mask[i] += [1] * len(toks)
                    actions[i] = self.processing_class.decode(toks, skip_special_tokens=True)
                for i, o in enumerate(mgr.step(actions)):
                    t = self._encode(o)
                    ctx[i] += t
                    mask[i] += [0] * len(t)
        finally:
            a.max_completion_length = saved
        rewards = torch.tensor(mgr.returns, dtype=torch.float32, device=self.device)
        L = min(max(len(c) for c in ctx), a.max_episode_tokens)
        ids = torch.stack([pad_to_length(torch.tensor(c[:L]), L, self.pad_token_id) for c in ctx]).to(self.device)
        att = torch.stack([pad_to_length(torch.ones(min(len(c), L), dtype=torch.long), L, 0) for c in ctx]).to(
            self.device)
        lm = torch.stack([pad_to_length(torch.tensor(m[:L]), L, 0) for m in mask]).to(self.device)
        new = {"input_ids": ids, "attention_mask": att, "loss_mask": lm,
               "advantages": group_advantages(rewards, n, a.scale_rewards, a.advantage_epsilon)}
        with torch.no_grad():
            was = self.model.training
            self.model.eval()
            new["old_logps"] = self._chunked_logps(self.model, ids, att, lm)
            if self.reference_model is not None and a.beta:
                new["ref_logps"] = self._chunked_logps(self.reference_model, ids, att, lm)
            self.model.train(was)
        return new, {"rewards/mean": float(rewards.mean()), "episodes/finished": float(sum(mgr.done)) / len(tasks),
                     "episodes/mean_tokens": float(att.sum(1).float().mean())}
