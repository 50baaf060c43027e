"""Runs one kernel a handful of times on a small, L2-exceeding case so that it can be captured by a profiler.

    python -m benchmarks.profile_case gemm          # 4096 x 6144 x 4096 bf16 (151 MB of operands + output)
    python -m benchmarks.profile_case gemm_decode   # 256 x 7168 x 8192: a decode step's weight-streaming product
    python -m benchmarks.profile_case gemm_wgrad    # fp32-accumulating weight gradient, MN-major operands
    python -m benchmarks.profile_case attn_fwd      # 8192 tokens, 32 / 8 heads, D = 128, causal
    python -m benchmarks.profile_case attn_bwd
    python -m benchmarks.profile_case gemm_rs       # one-rank form of the GEMM -> reduce-scatter kernel
    python -m benchmarks.profile_case ag_gemm       # one-rank form of the all-gather -> GEMM kernel
    python -m benchmarks.profile_case qgemv         # 4-bit fused dequant-GEMV, 4 rows x 14336 x 4096
    python -m benchmarks.profile_case qgemv_plain   # the same kernel as single launches (profiler captures)
    python -m benchmarks.profile_case adamw         # fused AdamW over 256M parameters

Prints the CUDA-event time of the last launch. Everything held on the device stays below 4 GB.
"""

from __future__ import annotations

import sys

import torch


def main() -> None:
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    from easydel_b200.ops import kernels as K

    bf = lambda *s: torch.randn(*s, device=dev, dtype=torch.bfloat16)  # noqa: E731
    if what == "gemm":
        a, w = bf(4096, 4096), bf(6144, 4096)
        out = torch.empty(4096, 6144, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.gemm(a, w, out=out)  # noqa: E731
        work = 2.0 * 4096 * 6144 * 4096
    elif what == "gemm_decode":
        # a decode step's gate / up projection at the per-GPU shape of a 70B model under 8-way tensor parallelism:
        # 256 rows against a 7168 x 8192 weight (117 MB streamed once); two weight copies alternate so that the
        # second launch does not find its weights in L2
        a = bf(256, 8192)
        ws = [bf(7168, 8192), bf(7168, 8192)]
        out = torch.empty(256, 7168, device=dev, dtype=torch.bfloat16)
        state = {"i": 0}

        def fn():
            state["i"] ^= 1
            K.gemm(a, ws[state["i"]], out=out, force_bn=-1)

        work = 2.0 * 7168 * 8192        # bytes of weights: the roofline of this product is HBM
    elif what == "gemm_wgrad":
        dy, x = bf(8192, 4096), bf(8192, 4096)
        out = torch.zeros(4096, 4096, device=dev, dtype=torch.float32)
        fn = lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True)  # noqa: E731
        work = 2.0 * 8192 * 4096 * 4096
    elif what in ("attn_fwd", "attn_bwd"):
        from easydel_b200.ops import attention as A

        q, k, v = bf(1, 8192, 32, 128), bf(1, 8192, 8, 128), bf(1, 8192, 8, 128)
        o, lse = A.attn_fwd(q, k, v, causal=True)
        do = bf(1, 8192, 32, 128)
        if what == "attn_fwd":
            fn = lambda: A.attn_fwd(q, k, v, causal=True)  # noqa: E731
            work = 4.0 * 8192 * 8192 * 32 * 128 / 2
        else:
            fn = lambda: A.attn_bwd(q, k, v, o, lse, do, causal=True)  # noqa: E731
            work = 10.0 * 8192 * 8192 * 32 * 128 / 2
    elif what == "gemm_rs":
        from easydel_b200.parallel.fused import GemmReduceScatter

        a, w = bf(4096, 4096), bf(4096, 4096)
        op = GemmReduceScatter(None, 4096, 4096, dev)
        fn = lambda: op(a, w)  # noqa: E731
        work = 2.0 * 4096 * 4096 * 4096
    elif what == "ag_gemm":
        from easydel_b200.parallel.fused import AllGatherGemm

        a, w = bf(4096, 4096), bf(4096, 4096)
        op = AllGatherGemm(None, 4096, 4096, dev)
        fn = lambda: op(a, w)  # noqa: E731
        work = 2.0 * 4096 * 4096 * 4096
    elif what == "qgemv_plain":      # single launches (for a profiler capture); timing is host-bound, see "qgemv"
        from easydel_b200.layers.quantization import quantize, quantized_matmul

        q1 = quantize(bf(14336, 4096) * 0.05, "nf4")
        x = bf(4, 4096)
        fn = lambda: quantized_matmul(x, q1)  # noqa: E731
        work = 14336 * 4096 * 0.5 + 14336 * 64 * 2
    elif what == "qgemv":
        from easydel_b200.layers.quantization import quantize, quantized_matmul

        # a launch is a few microseconds: 32 launches over 8 different weight matrices (250 MB, twice the L2) are
        # captured in one CUDA graph, so that neither the host nor the L2 decides the number
        qs = [quantize(bf(14336, 4096) * 0.05, "nf4") for _ in range(8)]
        x = bf(4, 4096)
        graphed = 32

        def many():
            for i in range(graphed):
                quantized_matmul(x, qs[i % 8])

        many()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            many()
        fn = g.replay
        work = graphed * (14336 * 4096 * 0.5 + 14336 * 64 * 2)     # bytes: the roofline of this kernel is HBM
    elif what == "adamw":
        n = 256 << 20
        p, g = torch.zeros(n, device=dev), torch.randn(n, device=dev)
        m, v2 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        w16 = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.adamw_(p, w16, m, v2, g, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,  # noqa: E731
                              step=3)
        work = n * (4 * 4 + 3 * 4 + 2)
    else:
        raise SystemExit(f"unknown case {what!r}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    unit = "GB/s" if what in ("qgemv", "qgemv_plain", "adamw", "gemm_decode") else "TFLOP/s"
    rate = work / ms / 1e6 if unit == "GB/s" else work / ms / 1e9
    from easydel_b200.ops import _lib

    _lib.check_status(dev)
    print(f"{what}: {ms:.3f} ms, {rate:.1f} {unit}")


if __name__ == "__main__":
    main()
