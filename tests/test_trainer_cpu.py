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
