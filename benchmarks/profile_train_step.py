"""Where a training step's time goes: device time per kernel name over one optimiser step of the Llama-3-8B SFT
configuration (full recompute, fp32-master AdamW), on one GPU.

    python -m benchmarks.profile_train_step --layers 8 --micro-batches 2

Runs a few un-profiled steps (CUDA-event time printed last, for reference), then records one step with
``torch.profiler`` (CUPTI activity records carry the start and end of every kernel) and prints, per kernel name,
launches per step, mean and total duration, the idle time in front of the kernel, and the share of the step. Layers
and micro-batches are reduced so that the record stays small; per-layer and per-micro-batch work is what repeats, so
shares of the decoder kernels carry over, while the embedding / LM-head / optimiser rows weigh more than in the
32-layer, 8-micro-batch step (the last lines scale them back). Durations under the profiler are for attribution,
not for quoting.
"""

from __future__ import annotations

import argparse
import collections

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--top", type=int, default=40)
    a = ap.parse_args()

    from bench import VOCAB, synth_packed_batches
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.trainers import Trainer, TrainingArguments

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = LlamaConfig(vocab_size=VOCAB, hidden_size=4096, intermediate_size=14336, num_hidden_layers=a.layers,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                      rope_theta=500000.0, max_position_embeddings=a.seq, tie_word_embeddings=False,
                      gradient_checkpointing="nothing_saveable", lmhead_chunksize=2048)
    model = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                             seed=1234)
    targs = TrainingArguments(model_name="profile", save_directory=None, total_batch_size=a.micro_batches,
                              gradient_accumulation_steps=a.micro_batches, learning_rate=1e-5, weight_decay=0.01,
                              optimizer="adamw", scheduler="none", clip_grad=1.0, max_training_steps=64,
                              max_length=a.seq, do_last_save=False, resume_if_possible=False, use_wandb=False,
                              report_metrics=False, progress_bar_type="none", report_steps=1, log_grad_norms=False,
                              extra_optimizer_kwargs={"b1": 0.9, "b2": 0.95, "eps": 1e-8})
    batches = synth_packed_batches(6, a.micro_batches, seed=7)
    for b in batches:
        b.pop("segment_ids", None)
    batches = [{k: v[:, :a.seq].to(dev) for k, v in b.items()} for b in batches]

    class _Batches:
        already_batched = True

        def __len__(self):
            return len(batches)

        def __iter__(self):
            return iter(batches)

    trainer = Trainer(arguments=targs, model=model, dataset_train=_Batches())
    for i in range(3):
        trainer.training_step(batches[i])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(3, 5):
        trainer.training_step(batches[i])
    e1.record()
    torch.cuda.synchronize()
    plain_ms = e0.elapsed_time(e1) / 2

    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.training_step(batches[5])
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end >
                  e.time_range.start), key=lambda e: e.time_range.start)
    dur, gap, cnt = collections.Counter(), collections.Counter(), collections.Counter()
    prev_end = None
    for e in evs:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:78]
        dur[name] += e.time_range.end - e.time_range.start
        if prev_end is not None:
            gap[name] += max(0.0, e.time_range.start - prev_end)
        cnt[name] += 1
        prev_end = max(prev_end or 0, e.time_range.end)
    total = sum(dur.values()) + sum(gap.values())
    print(f"{'kernel':78s} {'launches':>8s} {'mean us':>9s} {'total ms':>9s} {'idle ms':>8s} {'share':>6s}")
    for name, _ in sorted(dur.items(), key=lambda kv: -kv[1] - gap[kv[0]])[:a.top]:
        n = cnt[name]
        print(f"{name:78s} {n:8d} {dur[name] / n:9.1f} {dur[name] / 1e3:9.2f} {gap[name] / 1e3:8.2f} "
              f"{(dur[name] + gap[name]) / total:6.1%}")
    print(f"step under the profiler: kernels {sum(dur.values()) / 1e3:.1f} ms + idle {sum(gap.values()) / 1e3:.1f} ms; "
          f"{len(evs)} launches")
    tokens = a.micro_batches * a.seq
    print(f"step without the profiler ({a.layers} layers, {a.micro_batches} x {a.seq} tokens): {plain_ms:.1f} ms, "
          f"{tokens / plain_ms * 1e3:,.0f} tokens/s")


if __name__ == "__main__":
    main()
