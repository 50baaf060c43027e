"""Trainer loop on CPU: loss goes down on a repeated batch, metrics are reported, hooks fire."""

import torch

from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
from easydel_b200.trainers import Trainer, TrainingArguments


def _model():
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)


def _dataset(n=16, T=32):
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 256, (4, T), generator=g)
    return [{"input_ids": base[i % 4], "labels": base[i % 4]} for i in range(n)]


def test_trainer_reduces_loss_and_reports(tmp_path):
    args = TrainingArguments(model_name="t", save_directory=str(tmp_path), total_batch_size=4,
                             gradient_accumulation_steps=2, learning_rate=3e-3, num_train_epochs=6,
                             do_last_save=False, use_wandb=False, progress_bar_type="none", report_steps=1,
                             shuffle_train_dataset=False, weight_decay=0.0)
    seen = []
    tr = Trainer(arguments=args, model=_model(), dataset_train=_dataset())
    tr.register_hook("on_step_end", lambda t, s: seen.append(s))
    out = tr.train()
    hist = out.metrics_history
    assert out.state.step == 24 and seen == list(range(1, 25))
    assert hist[-1]["train/loss"] < hist[0]["train/loss"] - 0.5
    assert "train/tokens_per_second" in hist[-1] and "train/learning_rate" in hist[-1]


def test_max_steps_and_break_request(tmp_path):
    args = TrainingArguments(model_name="t", save_directory=str(tmp_path), total_batch_size=4, max_training_steps=5,
                             do_last_save=False, use_wandb=False, progress_bar_type="none")
    tr = Trainer(arguments=args, model=_model(), dataset_train=_dataset())
    tr.register_hook("on_step_end", lambda t, s: t.request_break() if s == 3 else None)
    out = tr.train()
    assert out.interrupted and out.state.step == 3


class _Tok:
    """A tokenizer stand-in: one token per character code."""

    def __call__(self, text, return_tensors=None):
        return {"input_ids": torch.tensor([[ord(c) % 256 for c in text]])}

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(i) for i in ids)


def test_preemption_signal_writes_a_checkpoint_and_stops(tmp_path):
    """SIGUSR1 during training: the loop finishes the running step, writes run-<step> and returns interrupted; a
    second trainer resumes from that checkpoint at the same step."""
    import os
    import signal

    args = TrainingArguments(model_name="t", save_directory=str(tmp_path), total_batch_size=4, max_training_steps=8,
                             do_last_save=False, use_wandb=False, progress_bar_type="none")
    tr = Trainer(arguments=args, model=_model(), dataset_train=_dataset())
    before = signal.getsignal(signal.SIGUSR1)
    tr.register_hook("on_step_end", lambda t, s: os.kill(os.getpid(), signal.SIGUSR1) if s == 3 else None)
    out = tr.train()
    assert out.interrupted and out.state.step == 3
    assert out.checkpoint_path and out.checkpoint_path.endswith("run-3") and os.path.isdir(out.checkpoint_path)
    assert signal.getsignal(signal.SIGUSR1) is before          # handlers are put back
    args2 = TrainingArguments(model_name="t", save_directory=str(tmp_path), total_batch_size=4, max_training_steps=5,
                              do_last_save=False, use_wandb=False, progress_bar_type="none",
                              resume_if_possible=True)
    tr2 = Trainer(arguments=args2, model=_model(), dataset_train=_dataset())
    assert tr2.model_state.step == 3
    assert tr2.train().state.step == 5


def test_generation_previews_and_benchmark_hook(tmp_path):
    args = TrainingArguments(model_name="t", save_directory=str(tmp_path), total_batch_size=4, max_training_steps=4,
                             do_last_save=False, use_wandb=False, progress_bar_type="none", generation_interval=2,
                             generation_prompts=["ab", "xyz"], generation_max_new_tokens=5, benchmark_interval=4)
    tr = Trainer(arguments=args, model=_model(), dataset_train=_dataset(), processing_class=_Tok())
    seen = []
    tr.register_hook("on_generation_preview", lambda t, step, texts: seen.append((step, list(texts))))
    tr.register_hook("on_benchmark", lambda t, step: {"toy_score": 0.5})
    out = tr.train()
    assert [s for s, _ in seen] == [2, 4] and all(len(t) == 2 and len(t[0].split()) == 5 for _, t in seen)
    assert tr.model.training                                    # previews leave the model in training mode
    assert tr.last_benchmarks == {"toy_score": 0.5}
    assert any("generation_preview" in h for h in out.metrics_history)
    assert any(h.get("benchmark/toy_score") == 0.5 for h in out.metrics_history)
