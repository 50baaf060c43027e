"""Device-timed comparison of the fused GEMM+collective kernels with GEMM + NCCL.

Run under torchrun, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \
        -m benchmarks.bench_fused [--tokens 8192] [--hidden 8192] [--ffn 28672] [--iters 20]

Shapes are the tensor-parallel linears of a Llama-70B layer at ``tokens`` rows. Every number is the maximum
over ranks of a CUDA-event time averaged over ``iters`` launches after 5 warm-up launches; operands are larger
than the L2 cache in total, and a 256 MB buffer is rewritten between timed launches. The roofline time of a
fused kernel is the slower of FLOPs / measured GEMM peak and NVLink bytes / 770 GB/s.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, flush):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    tot = 0.0
    for _ in range(iters):
        flush.add_(1)
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    t = torch.tensor([tot / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peak-tflops", type=float, default=1657.6)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from easydel_b200.ops import _lib
    from easydel_b200.ops import kernels as K
    from easydel_b200.parallel.fused import AllGatherGemm, GemmReduceScatter

    group = dist.group.WORLD
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    M = args.tokens
    results = []
    # row-parallel linears: K sharded, output reduce-scattered over rows
    for name, N, Kfull in (("o_proj", args.hidden, args.hidden), ("down_proj", args.hidden, args.ffn)):
        Kr = Kfull // world
        a = torch.randn(M, Kr, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, Kr, device=dev, dtype=torch.bfloat16) * 0.02
        op = GemmReduceScatter(group, M // world, N, dev)
        part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)

        def base():
            K.gemm(a, w, out=part)
            dist.reduce_scatter_tensor(out, part, group=group)

        t_f = _time(lambda: op(a, w), args.iters, flush)
        t_b = _time(base, args.iters, flush)
        t_g = _time(lambda: K.gemm(a, w, out=part), args.iters, flush)
        flops = 2.0 * M * N * Kr
        link = (world - 1) / world * M * N * 2
        roof = max(flops / (args.peak_tflops * 1e12), link / (args.link_gbs * 1e9)) * 1e3
        results.append(dict(op=f"gemm_reduce_scatter/{name}", M=M, N=N, K_local=Kr, fused_ms=t_f, gemm_plus_nccl_ms=t_b,
                            gemm_only_ms=t_g, roofline_ms=roof, frac_of_roofline=roof / t_f))
    # column-parallel linears: rows (sequence) sharded, gathered on the fly
    for name, Nfull, Kin in (("qkv_proj", args.hidden + 2 * args.hidden // 8, args.hidden),
                             ("gate_up_proj", 2 * args.ffn, args.hidden)):
        N = Nfull // world
        Ms = M // world
        a_sh = torch.randn(Ms, Kin, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, Kin, device=dev, dtype=torch.bfloat16) * 0.02
        op = AllGatherGemm(group, Ms, Kin, dev)
        op.shard.copy_(a_sh)
        full = torch.empty(M, Kin, device=dev, dtype=torch.bfloat16)
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

        def base():
            dist.all_gather_into_tensor(full, a_sh, group=group)
            K.gemm(full, w, out=c)

        t_f = _time(lambda: op(None, w), args.iters, flush)
        t_b = _time(base, args.iters, flush)
        t_g = _time(lambda: K.gemm(full, w, out=c), args.iters, flush)
        flops = 2.0 * M * N * Kin
        link = (world - 1) * Ms * Kin * 2
        roof = max(flops / (args.peak_tflops * 1e12), link / (args.link_gbs * 1e9)) * 1e3
        results.append(dict(op=f"allgather_gemm/{name}", M=M, N=N, K=Kin, fused_ms=t_f, nccl_plus_gemm_ms=t_b,
                            gemm_only_ms=t_g, roofline_ms=roof, frac_of_roofline=roof / t_f))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        for r in results:
            r["n_gpus"] = world
            print(json.dumps(r))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
