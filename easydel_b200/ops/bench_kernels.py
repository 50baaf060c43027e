"""Micro-benchmarks of the sm_100a kernels against the measured roofline.

``python -m easydel_b200.ops.bench_kernels gemm`` times the tcgen05 GEMM on the
linear-layer shapes of Llama-3-8B (forward, data-gradient and weight-gradient
layouts) and the same products through ``torch.matmul`` (cuBLAS) as the library
baseline. Timing uses CUDA events on the launching stream after warm-up; the L2
cache is flushed between timed launches by writing a 256 MiB buffer.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import kernels as K


def _peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": d["bf16_tflops"], "hbm_gbs": d["hbm_gbs"], "src": "measured"}
    return {"tflops": 1590.0, "hbm_gbs": 6650.0, "src": "fallback"}


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush: torch.Tensor | None = None) -> float:
    """Median milliseconds per call of ``fn`` (CUDA events, L2 flushed between calls)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return statistics.median(ts)


def bench_gemm(args) -> None:
    pk = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    T = args.tokens
    shapes = [
        ("qkv fwd", T, 6144, 4096, False, False),
        ("o fwd", T, 4096, 4096, False, False),
        ("gate_up fwd", T, 28672, 4096, False, False),
        ("down fwd", T, 4096, 14336, False, False),
        ("gate_up dgrad", T, 4096, 28672, False, True),
        ("down dgrad", T, 14336, 4096, False, True),
        ("gate_up wgrad", 28672, 4096, T, True, True),
        ("down wgrad", 4096, 14336, T, True, True),
        ("lm_head fwd (2048 tok)", 2048, 128256, 4096, False, False),
    ]
    rows = []
    for name, M, N, Kd, a_mn, b_mn in shapes:
        a = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda").to(torch.bfloat16)
        b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_cuda(lambda: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out), flush=flush)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        ms_lib = time_cuda(lambda: torch.matmul(A, B, out=out), flush=flush)
        fl = 2.0 * M * N * Kd
        tf, tf_lib = fl / ms / 1e9, fl / ms_lib / 1e9
        rows.append((name, M, N, Kd, ms, tf, tf / pk["tflops"], ms_lib, tf_lib))
        print(f"{name:26s} M={M:6d} N={N:6d} K={Kd:6d}  ours {ms:8.3f} ms {tf:7.1f} TFLOP/s "
              f"({tf / pk['tflops']:.2f} of {pk['src']} peak)   cuBLAS {ms_lib:8.3f} ms {tf_lib:7.1f} TFLOP/s",
              flush=True)
    from . import _lib

    _lib.check_status()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("what", choices=["gemm"])
    ap.add_argument("--tokens", type=int, default=8192)
    a = ap.parse_args()
    {"gemm": bench_gemm}[a.what](a)


if __name__ == "__main__":
    main()
