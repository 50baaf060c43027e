"""Serving benchmark: Poisson arrivals into an eSurge engine; reports output tokens/s, TTFT and TPOT percentiles.

One GPU:
    python -m easydel_b200.inference.esurge.bench_serving --model llama-3-8b --requests 200 --rate 16
Tensor parallel (one rank per GPU; every rank runs the same scheduler on the same request stream):
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29512 \
        -m easydel_b200.inference.esurge.bench_serving --model llama-3-70b --requests 2000 --rate 8

Workload (the serving configuration named in the baseline): prompt lengths uniform in [128, 4096], 30 % of the
requests share a 1024-token prefix, output lengths uniform in [128, 1024] with EOS ignored, greedy sampling,
tokens uniform over the vocabulary, random-initialised weights, page size 128, prefix caching on, at most 256
running sequences. Rank 0's clock decides when a request has arrived; the count of arrived requests is broadcast
before every engine step so that all tensor-parallel ranks schedule identical batches.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch

MODELS = {
    "llama-3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                        num_attention_heads=64, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5,
                        max_position_embeddings=8192),
    "llama-3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5,
                       max_position_embeddings=8192),
    "llama-tiny": dict(vocab_size=32000, hidden_size=1024, intermediate_size=2816, num_hidden_layers=4,
                       num_attention_heads=8, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5,
                       max_position_embeddings=8192),
}


def make_workload(n: int, rate: float, vocab: int, seed: int, prompt_range, output_range, shared_frac: float,
                  shared_len: int):
    rng = np.random.default_rng(seed)
    arrivals = np.cumsum(rng.exponential(1.0 / rate, n)) if rate > 0 else np.zeros(n)
    prefix = rng.integers(0, vocab, shared_len).tolist()
    reqs = []
    for i in range(n):
        plen = int(rng.integers(prompt_range[0], prompt_range[1] + 1))
        olen = int(rng.integers(output_range[0], output_range[1] + 1))
        toks = rng.integers(0, vocab, plen).tolist()
        if rng.random() < shared_frac and plen > shared_len:
            toks[:shared_len] = prefix
        reqs.append((float(arrivals[i]), toks, olen))
    return reqs


def pct(x, q):
    return float(np.percentile(np.asarray(x), q)) if len(x) else float("nan")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (smoke runs)")
    ap.add_argument("--requests", type=int, default=200)
    ap.add_argument("--rate", type=float, default=8.0, help="Poisson arrival rate, requests/s (0 = all at once)")
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--output-min", type=int, default=128)
    ap.add_argument("--output-max", type=int, default=1024)
    ap.add_argument("--shared-prefix-frac", type=float, default=0.3)
    ap.add_argument("--shared-prefix-len", type=int, default=1024)
    ap.add_argument("--hbm-utilization", type=float, default=0.85)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-prefix-caching", action="store_true")
    ap.add_argument("--time-limit", type=float, default=0.0, help="stop admitting and finish after this many seconds")
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist

    if world > 1:
        from ...parallel.mesh import init_distributed

        init_distributed()
    from ...modules.llama import LlamaConfig, LlamaForCausalLM
    from ..sampling_params import SamplingParams
    from . import eSurge

    kw = dict(MODELS[args.model])
    if args.layers:
        kw["num_hidden_layers"] = args.layers
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                             seed=1234).eval()
    engine = eSurge(model, max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
                    max_num_batched_tokens=args.max_num_batched_tokens, hbm_utilization=args.hbm_utilization,
                    enable_prefix_caching=not args.no_prefix_caching)
    work = make_workload(args.requests, args.rate, kw["vocab_size"], args.seed, (args.prompt_min, args.prompt_max),
                         (args.output_min, args.output_max), args.shared_prefix_frac, args.shared_prefix_len)
    # warm-up: a few requests through prefill and every decode bucket that the run will meet
    for i in range(3):
        engine.generate(work[i][1][:256], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    counter = torch.zeros(1, dtype=torch.int64, device=dev)
    arrival_wall: dict[str, float] = {}
    first_wall: dict[str, float] = {}
    done_wall: dict[str, float] = {}
    n_out: dict[str, int] = {}
    admitted = 0
    t0 = time.perf_counter()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    stop_admitting = False
    while True:
        now = time.perf_counter() - t0
        if rank == 0:
            k = admitted
            if not stop_admitting:
                while k < len(work) and work[k][0] <= now:
                    k += 1
            if args.time_limit and now > args.time_limit:
                stop_admitting = True
            counter[0] = k if not stop_admitting else -k - 1
        if world > 1:
            dist.broadcast(counter, src=0)
        v = int(counter.item())
        if v < 0:
            stop_admitting, v = True, -v - 1
        for i in range(admitted, v):
            rid = engine.add_request(work[i][1], SamplingParams(max_tokens=work[i][2], temperature=0.0,
                                                                ignore_eos=True), request_id=f"r{i}")
            arrival_wall[rid] = t0 + max(work[i][0], 0.0) if args.rate > 0 else time.perf_counter()
        admitted = v
        if not engine.scheduler.has_unfinished():
            if admitted >= len(work) or stop_admitting:
                break
            time.sleep(0.0005)
            continue
        engine.step()
        t = time.perf_counter()
        for rid, tr in list(engine._tracked.items()):
            n = len(tr.req.output_token_ids)
            if n and rid not in first_wall:
                first_wall[rid] = t
            if tr.finished and rid not in done_wall:
                done_wall[rid] = t
                n_out[rid] = n
                engine._tracked.pop(rid, None)
    ev1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    dev_ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(dev_ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ttft = [first_wall[r] - arrival_wall[r] for r in done_wall]
        tpot = [(done_wall[r] - first_wall[r]) / max(1, n_out[r] - 1) for r in done_wall if n_out[r] > 1]
        e2e = [done_wall[r] - arrival_wall[r] for r in done_wall]
        total_out = sum(n_out.values())
        span = float(dev_ms) / 1e3
        tm = engine.runner.timings
        print(json.dumps({
            "metric": "eSurge output tokens/s", "value": total_out / span, "unit": "tokens/s", "n_gpus": world,
            "model": args.model + (f"-{args.layers}L" if args.layers else ""), "tp": world,
            "requests_finished": len(done_wall), "requests_offered": len(work), "rate_rps": args.rate,
            "duration_s": span, "wall_s": wall, "ttft_p50_ms": pct(ttft, 50) * 1e3, "ttft_p99_ms": pct(ttft, 99) * 1e3,
            "tpot_p50_ms": pct(tpot, 50) * 1e3, "tpot_p99_ms": pct(tpot, 99) * 1e3, "e2e_p50_s": pct(e2e, 50),
            "prefix_cache_hit_rate": engine.pool.stats.hit_rate, "kv_pages": engine.cache.num_pages,
            "steps": tm["steps"], "graph_steps": tm["graph_steps"],
            "host_prep_s": tm["prep"], "launch_s": tm["exec"], "sample_s": tm["sample"], "d2h_wait_s": tm["d2h"],
            "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around the whole run, max over ranks"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
