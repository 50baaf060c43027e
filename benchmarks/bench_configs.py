"""Device-timed steps of the two non-headline baseline configurations, through the public trainers.

    # DPO on the Llama-3-8B architecture, tensor parallel x FSDP (frozen reference copy, sigmoid loss, beta 0.1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29520 \
        -m benchmarks.bench_configs dpo --tp 2 [--layers 32] [--pairs-per-rank 4]

    # SFT on the Qwen3-MoE-30B-A3B architecture with expert parallelism over all ranks (dropless top-8 of 128)
    python -m torch.distributed.run ... -m benchmarks.bench_configs moe [--layers 48] [--seqs-per-rank 4]

Synthetic data of the shapes the baseline names (preference pairs: prompt 128-512, completions 64-512 tokens; MoE:
sequences of 4096 tokens), random-initialised bf16 weights, fp32 master AdamW, full activation recompute.
``--layers`` shrinks the depth when fewer GPUs than the named configuration are available (the per-layer work is
unchanged). Timing: W warm-up steps, then K steps between CUDA events, maximum over ranks; one JSON line from rank 0.
"""

from __future__ import annotations

import argparse
import json

import torch


def _time_steps(trainer, batches, warmup, steps, dev, world):
    import torch.distributed as dist

    for i in range(warmup):
        b, _ = trainer._preprocess_batch_input(trainer.model_state, batches[i % len(batches)], True)
        trainer.training_step({k: v.to(dev) if isinstance(v, torch.Tensor) else v for k, v in b.items()})
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = None
    for i in range(steps):
        b, _ = trainer._preprocess_batch_input(trainer.model_state, batches[(warmup + i) % len(batches)], True)
        loss, _, _ = trainer.training_step({k: v.to(dev) if isinstance(v, torch.Tensor) else v for k, v in b.items()})
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item() / steps, float(loss)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["dpo", "moe"])
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--pairs-per-rank", type=int, default=4)
    ap.add_argument("--seqs-per-rank", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from easydel_b200.ops import _lib
    from easydel_b200.parallel.mesh import init_distributed

    rank, local, world = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(100 + rank)
    common = dict(model_name="bench", save_directory=None, learning_rate=1e-6, weight_decay=0.01, optimizer="adamw",
                  scheduler="none", clip_grad=1.0, max_training_steps=10 ** 6, do_last_save=False,
                  resume_if_possible=False, use_wandb=False, report_metrics=False, progress_bar_type="none",
                  log_grad_norms=False, extra_optimizer_kwargs={"b1": 0.9, "b2": 0.95, "eps": 1e-8})
    if a.what == "dpo":
        from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
        from easydel_b200.trainers import DPOConfig, DPOTrainer

        V = 128256
        tp = min(a.tp, world)
        dp = world // tp
        L = a.layers or 32
        cfg = LlamaConfig(vocab_size=V, hidden_size=4096, intermediate_size=14336, num_hidden_layers=L,
                          num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                          rope_theta=500000.0, max_position_embeddings=2048, tie_word_embeddings=False,
                          gradient_checkpointing="nothing_saveable", sharding_axis_dims=(1, dp, 1, tp, 1))
        model = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                                 seed=1234)
        ref = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                               seed=1234).eval().requires_grad_(False)
        n = a.pairs_per_rank
        # ranks of one tensor-parallel group see the same pairs; data-parallel groups see different ones
        gd = torch.Generator().manual_seed(100 + rank // tp)

        def rows(k):
            out = []
            for _ in range(k):
                lp, lc, lr = (int(torch.randint(lo, hi + 1, (1,), generator=gd)) for lo, hi in
                              ((128, 512), (64, 512), (64, 512)))
                out.append({"prompt_input_ids": torch.randint(0, V, (lp,), generator=gd).tolist(),
                            "chosen_input_ids": torch.randint(0, V, (lc,), generator=gd).tolist(),
                            "rejected_input_ids": torch.randint(0, V, (lr,), generator=gd).tolist()})
            return out

        args = DPOConfig(total_batch_size=n * dp, gradient_accumulation_steps=n, beta=0.1, loss_type="sigmoid",
                         max_length=2048, max_prompt_length=512, max_completion_length=512, **common)
        trainer = DPOTrainer(args, model=model, reference_model=ref, train_dataset=rows(n))
        batches = [trainer.data_collator(rows(n)) for _ in range(a.steps + a.warmup)]
        tokens = sum(int(b["chosen_attention_mask"].sum() + b["rejected_attention_mask"].sum()
                         + 2 * b["prompt_attention_mask"].sum()) for b in batches[a.warmup:]) / a.steps * dp
        ms, loss = _time_steps(trainer, batches, a.warmup, a.steps, dev, world)
        res = {"metric": "DPO pairs/s (Llama-3-8B architecture)", "value": n * dp / (ms / 1e3), "unit": "pairs/s",
               "tokens_per_s": tokens / (ms / 1e3), "ms_per_step": ms, "n_gpus": world,
               "config": {"layers": L, "parallelism": f"fsdp{dp} x tp{tp}", "global_batch_pairs": n * dp,
                          "beta": 0.1, "loss": "sigmoid", "reference": "frozen copy, forward every step"},
               "final_loss": loss}
    else:
        from easydel_b200.modules.families import Qwen3MoeConfig, Qwen3MoeForCausalLM
        from easydel_b200.trainers import Trainer, TrainingArguments

        V, S = 151936, 4096
        L = a.layers or 48
        cfg = Qwen3MoeConfig(vocab_size=V, hidden_size=2048, intermediate_size=6144, num_hidden_layers=L,
                             num_attention_heads=32, num_key_value_heads=4, head_dim=128, moe_intermediate_size=768,
                             num_experts=128, num_experts_per_tok=8, norm_topk_prob=True, router_aux_loss_coef=0.001,
                             max_position_embeddings=S, rope_theta=1e6, tie_word_embeddings=False,
                             gradient_checkpointing="nothing_saveable", sharding_axis_dims=(1, 1, world, 1, 1),
                             lmhead_chunksize=2048)
        model = Qwen3MoeForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                                    seed=1234)
        n = a.seqs_per_rank
        args = TrainingArguments(total_batch_size=n * world, gradient_accumulation_steps=n, max_length=S, **common)
        batches = []
        for _ in range(a.steps + a.warmup):
            ids = torch.randint(0, V, (n, S), generator=g)
            batches.append({"input_ids": ids, "labels": ids.clone()})

        class _B:
            already_batched = True

            def __len__(self):
                return len(batches)

            def __iter__(self):
                return iter(batches)

        trainer = Trainer(arguments=args, model=model, dataset_train=_B())
        ms, loss = _time_steps(trainer, batches, a.warmup, a.steps, dev, world)
        # one more (untimed) step with the exchange's row counter on: rows a rank stores into other ranks per
        # dispatch, against what an all-gather of the tokens would move ((world - 1) x tokens per rank)
        traffic = None
        if world > 1:
            from easydel_b200.parallel import ep as EP

            for ex in EP._TOKEN_EXCHANGES.values():
                ex.track = True
            _time_steps(trainer, batches[-1:], 0, 1, dev, world)
            exs = [ex for ex in EP._TOKEN_EXCHANGES.values() if ex.dispatches]
            if exs:
                ex = exs[0]
                per = float(ex.rows_remote) / ex.dispatches
                traffic = {"token_exchange": EP.ep_dispatch_mode(), "remote_rows_per_dispatch": per,
                           "all_gather_rows": (world - 1) * S, "fraction_of_all_gather": per / ((world - 1) * S),
                           "row_bytes": ex.x_bytes, "dispatches_per_step": ex.dispatches}
                ex.track = False
        res = {"metric": "SFT tokens/s (Qwen3-MoE-30B-A3B architecture)", "value": n * world * S / (ms / 1e3),
               "unit": "tokens/s", "ms_per_step": ms, "n_gpus": world,
               "config": {"layers": L, "parallelism": f"ep{world}", "global_batch": n * world, "seq_len": S,
                          "experts": 128, "top_k": 8, "aux_loss_coef": 0.001}, "final_loss": loss,
               "nvlink_traffic": traffic}
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        res.update({"dtype": "bf16", "data": "synthetic", "steps": a.steps, "warmup": a.warmup,
                    "timing": "CUDA events, max over ranks"})
        print(json.dumps(res))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
