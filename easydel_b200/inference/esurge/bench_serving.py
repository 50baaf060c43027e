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


def build_parser() -> argparse.ArgumentParser:
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
    ap.add_argument("--sync-scheduling", action="store_true", help="read every step's tokens back before the next launch")
    ap.add_argument("--tp-shape-of", type=int, default=0,
                    help="one GPU, with the per-GPU layer shapes of this tensor-parallel degree (heads, KV heads and "
                         "FFN width divided by it): the compute side of a TP run without the other GPUs")
    ap.add_argument("--time-limit", type=float, default=0.0, help="stop admitting and finish after this many seconds")
    return ap


def run(args) -> dict | None:
    """Runs the workload on the ranks of the current job (tensor parallel over all of them) and returns the
    result dictionary on rank 0 (``None`` elsewhere). The caller owns the process group."""
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from ...modules.llama import LlamaConfig, LlamaForCausalLM
    from ..sampling_params import SamplingParams
    from . import eSurge

    kw = dict(MODELS[args.model])
    if args.layers:
        kw["num_hidden_layers"] = args.layers
    shape_note = ""
    if args.tp_shape_of and world == 1:
        d = args.tp_shape_of
        kw.update(num_attention_heads=kw["num_attention_heads"] // d,
                  num_key_value_heads=max(1, kw["num_key_value_heads"] // d),
                  intermediate_size=kw["intermediate_size"] // d,
                  head_dim=kw["hidden_size"] // kw["num_attention_heads"])
        shape_note = f"-tp{d}shape"
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device=dev,
                                             seed=1234).eval()
    engine = eSurge(model, max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
                    max_num_batched_tokens=args.max_num_batched_tokens, hbm_utilization=args.hbm_utilization,
                    enable_prefix_caching=not args.no_prefix_caching, async_scheduling=not args.sync_scheduling)
    work = make_workload(args.requests, args.rate, kw["vocab_size"], args.seed, (args.prompt_min, args.prompt_max),
                         (args.output_min, args.output_max), args.shared_prefix_frac, args.shared_prefix_len)
    # warm-up: a few requests through prefill and the first decode buckets
    for i in range(min(3, len(work))):
        engine.generate(work[i][1][:256], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    engine.runner.time_decode_steps = True      # CUDA events around every replayed decode step
    # The arrival count travels over a host-side (gloo) group: a device-side broadcast read back with .item()
    # would wait for the engine step that was just launched and serialise host and device again.
    ctl = None
    if world > 1:
        dist.barrier()
        ctl = dist.new_group(backend="gloo")
    counter = torch.zeros(1, dtype=torch.int64)
    arrival_wall: dict[str, float] = {}
    first_wall: dict[str, float] = {}
    done_wall: dict[str, float] = {}
    n_out: dict[str, int] = {}
    admitted = 0
    t0 = time.perf_counter()
    wall0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    stop_admitting = False
    try:
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
            if ctl is not None:
                dist.broadcast(counter, src=0, group=ctl)
            v = int(counter.item())
            if v < 0:
                stop_admitting, v = True, -v - 1
            for i in range(admitted, v):
                rid = engine.add_request(work[i][1], SamplingParams(max_tokens=work[i][2], temperature=0.0,
                                                                    ignore_eos=True), request_id=f"r{i}")
                arrival_wall[rid] = t0 + max(work[i][0], 0.0) if args.rate > 0 else time.perf_counter()
            admitted = v
            if not (engine.scheduler.has_unfinished() or engine._inflight is not None):
                if admitted >= len(work) or stop_admitting:
                    break
                time.sleep(0.0005)
                continue
            engine.step()
            t = time.perf_counter()
            for rid, tr in list(engine._tracked.items()):
                ft = tr.req.first_token_time        # set when the token reached the host
                if ft is not None and rid not in first_wall:
                    first_wall[rid] = t0 + (ft - wall0)
                if tr.finished and rid not in done_wall:
                    done_wall[rid] = t
                    n_out[rid] = len(tr.req.output_token_ids)
                    engine._tracked.pop(rid, None)
        ev1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        dev_ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(dev_ms, op=dist.ReduceOp.MAX)
        result = None
        if rank == 0:
            ttft = [first_wall[r] - arrival_wall[r] for r in done_wall if r in first_wall]
            tpot = [(done_wall[r] - first_wall[r]) / max(1, n_out[r] - 1) for r in done_wall
                    if n_out[r] > 1 and r in first_wall]
            e2e = [done_wall[r] - arrival_wall[r] for r in done_wall]
            total_out = sum(n_out.values())
            span = float(dev_ms) / 1e3
            tm = engine.runner.timings
            steps_ms = engine.runner.decode_step_times()
            decode_ms = {str(bp): {"n": len(v), "p50_ms": pct(v, 50), "p90_ms": pct(v, 90)}
                         for bp, v in sorted(steps_ms.items())}
            result = {
                "metric": "eSurge output tokens/s", "value": total_out / span, "unit": "tokens/s", "n_gpus": world,
                "model": args.model + (f"-{args.layers}L" if args.layers else "") + shape_note, "tp": world,
                "requests_finished": len(done_wall), "requests_offered": len(work), "rate_rps": args.rate,
                "duration_s": span, "wall_s": wall, "ttft_p50_ms": pct(ttft, 50) * 1e3,
                "ttft_p99_ms": pct(ttft, 99) * 1e3, "tpot_p50_ms": pct(tpot, 50) * 1e3,
                "tpot_p99_ms": pct(tpot, 99) * 1e3, "e2e_p50_s": pct(e2e, 50),
                "prefix_cache_hit_rate": engine.pool.stats.hit_rate, "kv_pages": engine.cache.num_pages,
                "max_num_seqs": args.max_num_seqs, "page_size": 128, "async_scheduling": engine.async_scheduling,
                "steps": tm["steps"], "graph_steps": tm["graph_steps"], "host_prep_s": tm["prep"],
                "launch_s": tm["exec"], "sample_s": tm["sample"], "d2h_wait_s": tm["d2h"],
                "decode_step_device_ms_by_rows": decode_ms, "dtype": "bf16",
                "data": "synthetic", "timing": "CUDA events around the whole run, max over ranks"}
        return result
    finally:
        # Teardown order matters for a clean exit: stop the engine and drop its captured graphs (they hold the
        # collectives of the tensor-parallel group) and the symmetric buffers before the caller destroys the groups.
        engine.close()
        from ...parallel import tp as tpar

        tpar.release_peer_buffers()
        del engine, model
        import gc

        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
            if ctl is not None:
                dist.destroy_process_group(ctl)


def main():
    args = build_parser().parse_args()
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        from ...parallel.mesh import init_distributed

        init_distributed()
    result = run(args)
    if result is not None:
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
