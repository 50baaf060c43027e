"""Every registered trainer runs optimizer steps on a tiny Llama on CPU; loss formulas are checked by hand."""

import math

import pytest
import torch
import torch.nn.functional as tF

from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM, LlamaForSequenceClassification
from easydel_b200 import trainers as T
from easydel_b200.trainers.packer import pack_sequences
from easydel_b200.trainers.preference import cpo_loss, kto_loss, orpo_loss
from easydel_b200.trainers.rl import first_eos_mask, group_advantages, grpo_objective, extract_final_answer
from easydel_b200.trainers.rl_online import gae

V = 96


class CharTok:
    """Byte-level stand-in for a tokenizer (ids 3.. are characters; 0 pad, 1 bos, 2 eos)."""

    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2

    def __call__(self, text, add_special_tokens=False, truncation=False, max_length=None, **_):
        ids = [3 + (ord(c) % (V - 3)) for c in text]
        if max_length:
            ids = ids[:max_length]
        return {"input_ids": ids}

    def encode(self, text, add_special_tokens=False):
        return self(text)["input_ids"]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(32 + ((i - 3) % 90)) for i in ids if i >= 3)


def _model(cls=LlamaForCausalLM, seed=0, **kw):
    cfg = LlamaConfig(vocab_size=V, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128, eos_token_id=2, pad_token_id=0, **kw)
    torch.manual_seed(seed)
    return cls(cfg, dtype=torch.float32, param_dtype=torch.float32)


def _args(cls, tmp_path, **kw):
    base = dict(model_name="t", save_directory=str(tmp_path), total_batch_size=4, max_training_steps=2,
                learning_rate=1e-3, do_last_save=False, use_wandb=False, progress_bar_type="none", report_steps=1,
                shuffle_train_dataset=False)
    base.update(kw)
    return cls(**base)


def _rand(n, lo=3, hi=V, g=None):
    return torch.randint(lo, hi, (n,), generator=g).tolist()


def _pairs(n=8):
    g = torch.Generator().manual_seed(0)
    return [{"prompt_input_ids": _rand(6, g=g), "chosen_input_ids": _rand(5, g=g) + [2],
             "rejected_input_ids": _rand(7, g=g) + [2]} for _ in range(n)]


def _prompts(n=8):
    g = torch.Generator().manual_seed(1)
    return [{"input_ids": _rand(5 + i % 3, g=g), "answer": str(i)} for i in range(n)]


def _run(trainer):
    before = [p.detach().clone() for p in trainer.model.parameters()]
    out = trainer.train()
    assert out.state.step == 2
    for h in out.metrics_history:
        assert math.isfinite(h["train/loss"]), h
    assert any(not torch.equal(a, b) for a, b in zip(before, trainer.model.parameters()))
    return out


# ------------------------------------------------------------------------------------------- loss algebra
def test_dpo_loss_variants_by_hand():
    pc, pr = torch.tensor([-10.0, -12.0]), torch.tensor([-11.0, -11.5])
    rc, rr = torch.tensor([-10.5, -12.5]), torch.tensor([-10.8, -11.0])
    logits = (pc - pr) - (rc - rr)
    l, cr, rw = T.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type="sigmoid")
    assert torch.allclose(l, -tF.logsigmoid(0.5 * logits)) and torch.allclose(cr, 0.5 * (pc - rc))
    l, _, _ = T.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type="ipo")
    assert torch.allclose(l, (logits - 1.0) ** 2)
    l, _, _ = T.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type="hinge")
    assert torch.allclose(l, torch.relu(1 - 0.5 * logits))
    l, _, _ = T.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type="sigmoid", label_smoothing=0.1)
    assert torch.allclose(l, -0.9 * tF.logsigmoid(0.5 * logits) - 0.1 * tF.logsigmoid(-0.5 * logits))
    for name in ("robust", "exo_pair", "nca_pair", "bco_pair", "sppo_hard", "aot", "aot_pair", "apo_zero",
                 "apo_down", "discopop", "kto"):
        l, _, _ = T.dpo_loss(pc, pr, rc, rr, beta=0.5, loss_type=name, label_smoothing=0.05)
        assert torch.isfinite(l).all(), name
    with pytest.raises(ValueError):
        T.dpo_loss(pc, pr, rc, rr, loss_type="nope")


def test_other_preference_losses():
    ca, ra, nll = torch.tensor([-0.5, -0.7]), torch.tensor([-0.9, -0.6]), torch.tensor(0.6)
    loss, log_odds, _ = orpo_loss(ca, ra, nll, beta=0.2)
    ref = (ca - ra) - (torch.log1p(-ca.exp()) - torch.log1p(-ra.exp()))
    assert torch.allclose(log_odds, ref) and torch.allclose(loss, nll - 0.2 * tF.logsigmoid(ref).mean())
    l, _, _ = cpo_loss(ca, ra, beta=2.0, loss_type="simpo", simpo_gamma=1.0)
    assert torch.allclose(l, -tF.logsigmoid(2.0 * ((ca - ra) - 0.5)))
    lab = torch.tensor([True, False])
    l, rew, kl = kto_loss(ca, ra, torch.tensor([-1.0, -1.0]), torch.tensor([-1.2, -1.1]), lab, beta=0.5)
    assert abs(float(kl) - 0.15) < 1e-6
    assert torch.allclose(l[0], 1 - torch.sigmoid(0.5 * ((ca - ra)[0] - kl)))
    assert torch.allclose(l[1], 1 - torch.sigmoid(0.5 * (kl - (ca - ra)[1])))


def test_rl_algebra():
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0])
    adv = group_advantages(r, 4, scale=True, eps=1e-4)
    assert torch.allclose(adv[:4], torch.tensor([0.5, -0.5, -0.5, 0.5]) / (0.5 + 1e-4)) and adv[4:].abs().max() == 0
    keep = torch.tensor([1, 1, 0, 0, 1, 1, 1, 1]).bool()
    adv = group_advantages(r, 4, scale=False, keep=keep)
    assert torch.allclose(adv[:4], torch.tensor([0.5, -0.5, 0.0, 0.0]))
    m = first_eos_mask(torch.tensor([[5, 2, 7, 2], [5, 6, 7, 8]]), [2])
    assert m.tolist() == [[1, 1, 0, 0], [1, 1, 1, 1]]
    lp = torch.log(torch.tensor([[0.5, 0.25]]))
    old = torch.log(torch.tensor([[0.25, 0.25]]))
    loss, st = grpo_objective(lp, old, None, torch.tensor([1.0]), torch.ones(1, 2), epsilon=0.2)
    assert abs(float(loss) + (1.2 + 1.0) / 2) < 1e-6 and abs(float(st["clip_ratio"]) - 0.5) < 1e-6
    loss_seq, _ = grpo_objective(lp, old, None, torch.tensor([1.0]), torch.ones(1, 2), epsilon=0.5, level="sequence")
    assert abs(float(loss_seq) + math.sqrt(2.0)) < 1e-5
    adv, ret = gae(torch.tensor([[0.0, 0.0, 1.0]]), torch.tensor([[0.5, 0.5, 0.5]]),
                   torch.tensor([[1.0, 1.0, 1.0, 0.0]]), gamma=1.0, lam=1.0)
    assert torch.allclose(adv, torch.tensor([[0.5, 0.5, 0.5]])) and torch.allclose(ret, torch.ones(1, 3))
    assert extract_final_answer("so \\boxed{42}.") == "42" and extract_final_answer("x\n#### 7") == "7"


def test_packing_strategies():
    rows = [{"input_ids": list(range(1, n + 1))} for n in (5, 3, 7, 2, 4)]
    packed = pack_sequences(rows, 8, "bfd")
    assert all(len(r["input_ids"]) == 8 for r in packed) and len(packed) == 3
    tot = sum(sum(m) for m in (r["attention_mask"] for r in packed))
    assert tot == 21
    for r in packed:
        seg = r["segment_ids"]
        firsts = [i for i in range(8) if seg[i] and (i == 0 or seg[i] != seg[i - 1])]
        assert all(r["labels"][i] == -100 for i in firsts)
    wrapped = pack_sequences(rows, 8, "wrapped")
    assert len(wrapped) == 2 and wrapped[0]["input_ids"][:5] == [1, 2, 3, 4, 5]


# ------------------------------------------------------------------------------------------- trainers end to end
def test_sft_text_completion_masks_and_packing(tmp_path):
    tok = CharTok()
    data = [{"prompt": "question %d?" % i, "completion": " answer %d" % i} for i in range(8)]
    tr = T.SFTTrainer(_args(T.SFTConfig, tmp_path, max_length=32, packing=True), model=_model(), processing_class=tok,
                      train_dataset=data)
    row = tr.dataset_train[0]
    assert len(row["input_ids"]) == 32 and "segment_ids" in row and -100 in row["labels"]
    _run(tr)


@pytest.mark.parametrize("name,cfg", [("dpo", dict(loss_type="sigmoid")), ("dpo", dict(loss_type="ipo", rpo_alpha=0.5)),
                                      ("orpo", {}), ("cpo", dict(loss_type="simpo"))])
def test_paired_preference_trainers(tmp_path, name, cfg):
    cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
    _run(cls(_args(acls, tmp_path, **cfg), model=_model(), train_dataset=_pairs()))


@pytest.mark.parametrize("name", ["kto", "bco"])
def test_unpaired_preference_trainers(tmp_path, name):
    g = torch.Generator().manual_seed(3)
    data = [{"prompt_input_ids": _rand(5, g=g), "completion_input_ids": _rand(4, g=g) + [2], "label": i % 2 == 0}
            for i in range(8)]
    cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
    _run(cls(_args(acls, tmp_path), model=_model(), train_dataset=data))


def test_reward_trainer(tmp_path):
    g = torch.Generator().manual_seed(4)
    data = [{"input_ids_chosen": _rand(6, g=g), "input_ids_rejected": _rand(8, g=g)} for _ in range(8)]
    model = _model(LlamaForSequenceClassification, num_labels=1)
    _run(T.RewardTrainer(_args(T.RewardConfig, tmp_path, center_rewards_coefficient=0.01), model=model,
                         train_dataset=data))


def _len_reward(prompts, completions, completion_mask=None, **kw):
    return (completion_mask.sum(1).float() / 4 + (completion_mask.sum(1) % 2).float()).tolist()


@pytest.mark.parametrize("name,cfg", [("grpo", dict(beta=0.04)), ("gspo", {}), ("gfpo", dict(gfpo_retain_count=2)),
                                      ("grpo", dict(loss_type="dr_grpo", beta=0.0))])
def test_group_relative_trainers(tmp_path, name, cfg):
    cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
    a = _args(acls, tmp_path, max_completion_length=6, num_return_sequences=4, total_batch_size=2, **cfg)
    out = _run(cls(a, model=_model(), reward_funcs=_len_reward, train_dataset=_prompts(), processing_class=CharTok()))
    assert "rewards/mean" in out.metrics_history[-1]


def test_rlvr_and_sdpo(tmp_path):
    tok = CharTok()
    a = _args(T.RLVRConfig, tmp_path, max_completion_length=5, num_return_sequences=2, total_batch_size=2)
    tr = T.RLVRTrainer(a, model=_model(), train_dataset=_prompts(), processing_class=tok)
    tr.train()          # rewards are all zero on random text: the step must still run
    a = _args(T.SDPOConfig, tmp_path, max_completion_length=5, num_return_sequences=2, total_batch_size=2,
              max_feedback_length=8)
    fb = lambda prompts, completions, rewards, **k: ["try again: shorter"] * len(completions)  # noqa: E731
    _run(T.SDPOTrainer(a, model=_model(), reward_funcs=_len_reward, feedback_func=fb, train_dataset=_prompts(),
                       processing_class=tok))


def test_ppo_xpo_nashmd(tmp_path):
    tok = CharTok()
    a = _args(T.PPOConfig, tmp_path, max_completion_length=5, total_batch_size=2)
    tr = T.PPOTrainer(a, model=_model(), reward_funcs=_len_reward, train_dataset=_prompts(), processing_class=tok)
    out = _run(tr)
    assert "train/ppo/value_loss" in out.metrics_history[-1] or any("value_loss" in k for k in out.metrics_history[-1])
    for name in ("xpo", "nash-md"):
        cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
        a = _args(acls, tmp_path, max_completion_length=5, total_batch_size=2)
        _run(cls(a, model=_model(), reward_funcs=_len_reward, train_dataset=_prompts(), processing_class=tok))


@pytest.mark.parametrize("name,cfg", [("distillation", dict(hidden_state_loss_weight=0.1)),
                                      ("sparse_distillation", dict(top_k=8))])
def test_logit_distillation(tmp_path, name, cfg):
    g = torch.Generator().manual_seed(5)
    data = [{"input_ids": torch.tensor(_rand(16, g=g))} for _ in range(8)]
    for d in data:
        d["labels"] = d["input_ids"]
    cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
    _run(cls(_args(acls, tmp_path, **cfg), student_model=_model(seed=0), teacher_model=_model(seed=1),
             dataset_train=data))


@pytest.mark.parametrize("name,cfg", [("seq_kd", {}), ("gkd", dict(lmbda=1.0)), ("gkd", dict(lmbda=0.0)),
                                      ("on_policy_distillation", {}),
                                      ("on_policy_distillation", dict(kl_mode="sampled"))])
def test_generation_based_distillation(tmp_path, name, cfg):
    cls, acls = T.get_trainer_class(name), T.get_trainer_arguments_class(name)
    a = _args(acls, tmp_path, max_completion_length=5, total_batch_size=2, **cfg)
    _run(cls(a, model=_model(seed=0), teacher_model=_model(seed=1), train_dataset=_prompts(),
             processing_class=CharTok()))


def test_embedding_trainer(tmp_path):
    g = torch.Generator().manual_seed(6)
    data = [{"query_input_ids": _rand(5, g=g), "positive_input_ids": _rand(7, g=g),
             "negative_input_ids": _rand(6, g=g)} for _ in range(8)]
    _run(T.EmbeddingTrainer(_args(T.EmbeddingConfig, tmp_path, pooling="mean", matryoshka_dims=(16, 32)),
                            model=_model(), train_dataset=data))


def test_agentic_moshpit(tmp_path):
    tok = CharTok()
    calls = []

    def factory():
        return T.ToolEnvironment({"echo": lambda s: calls.append(s) or s}, scorer=lambda task, ans: 1.0, max_turns=2)

    env = factory()
    assert env.reset({"prompt": "p"}) == "p"
    obs, r, done, _ = env.step("<tool>echo(hi)</tool>")
    assert obs == "<result>hi</result>" and not done
    _, r, done, _ = env.step("<answer>4</answer>")
    assert r == 1.0 and done
    a = _args(T.AgenticMoshPitConfig, tmp_path, num_return_sequences=2, total_batch_size=2, max_turns=2,
              max_turn_tokens=4, max_episode_tokens=48, beta=0.0)
    data = [{"input_ids": [3, 4], "task": {"prompt": "solve %d" % i}} for i in range(4)]
    tr = T.AgenticMoshPitTrainer(a, model=_model(), env_factory=factory, processing_class=tok, train_dataset=data)
    out = tr.train()
    assert out.state.step == 2 and "episodes/finished" in out.metrics_history[-1]


def test_ray_distributed_config_scaling():
    cfg = T.RayDistributedConfig(base_config=dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2),
                                 round_to=64)
    s = cfg.scaled_config(1)
    assert s == dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=4)
