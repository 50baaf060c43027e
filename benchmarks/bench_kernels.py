"""Micro-benchmarks of the sm_100a kernels against the measured roofline.

``python -m benchmarks.bench_kernels gemm`` times the tcgen05 GEMM on the
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

from easydel_b200.ops import kernels as K


def _peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
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
        ms1 = time_cuda(lambda: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, force_bn=-1), flush=flush)
        ms2 = time_cuda(lambda: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, force_bn=512), flush=flush)
        ms = min(ms1, ms2)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        ms_lib = time_cuda(lambda: torch.matmul(A, B, out=out), flush=flush)
        fl = 2.0 * M * N * Kd
        tf, tf_lib = fl / ms / 1e9, fl / ms_lib / 1e9
        rows.append((name, M, N, Kd, ms, tf, tf / pk["tflops"], ms_lib, tf_lib))
        print(f"{name:26s} M={M:6d} N={N:6d} K={Kd:6d}  ours {ms:8.3f} ms {tf:7.1f} TFLOP/s "
              f"({tf / pk['tflops']:.2f} of {pk['src']} peak; 1-CTA {ms1:.3f} ms, CTA pair {ms2:.3f} ms)   cuBLAS {ms_lib:8.3f} ms {tf_lib:7.1f} TFLOP/s",
              flush=True)
    from easydel_b200.ops import _lib

    _lib.check_status()


def bench_attention(args) -> None:
    from easydel_b200.ops import attention as A

    pk = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    T, Hq, Hkv, D = args.tokens, 32, 8, 128
    qkv = torch.randn(1, T, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    q = qkv[..., : Hq * D].view(1, T, Hq, D)
    k = qkv[..., Hq * D:(Hq + Hkv) * D].view(1, T, Hkv, D)
    v = qkv[..., (Hq + Hkv) * D:].view(1, T, Hkv, D)
    do = torch.randn(1, T, Hq, D, device="cuda").to(torch.bfloat16)
    o, lse = A.attn_fwd(q, k, v, causal=True)
    ms_f = time_cuda(lambda: A.attn_fwd(q, k, v, causal=True), flush=flush)
    ms_b = time_cuda(lambda: A.attn_bwd(q, k, v, o, lse, do, causal=True), flush=flush)
    fl = 4.0 * T * T * D * Hq * 0.5
    print(f"attention fwd  T={T} Hq={Hq} Hkv={Hkv} D={D} causal: {ms_f:.3f} ms  {fl / ms_f / 1e9:.1f} TFLOP/s "
          f"({fl / ms_f / 1e9 / pk['tflops']:.2f} of {pk['src']} peak)")
    print(f"attention bwd  (2.5x fwd FLOPs):                    {ms_b:.3f} ms  {2.5 * fl / ms_b / 1e9:.1f} TFLOP/s "
          f"({2.5 * fl / ms_b / 1e9 / pk['tflops']:.2f} of {pk['src']} peak)")
    try:
        import torch.nn.functional as tF

        qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
        ms_l = time_cuda(lambda: tF.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True),
                         flush=flush)
        print(f"library SDPA fwd:                                   {ms_l:.3f} ms  {fl / ms_l / 1e9:.1f} TFLOP/s")
    except Exception as e:  # the library baseline is informative only
        print("library SDPA unavailable:", e)
    from easydel_b200.ops import _lib

    _lib.check_status()


def bench_layer(args) -> None:
    """One micro-batch (1 x tokens) forward + backward of a 2-layer Llama-3-8B-shaped model: the
    launch list of this run under ncu gives the per-kernel time shares of a training step."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig

    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=args.layers,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                      rope_theta=500000.0, max_position_embeddings=args.tokens,
                      gradient_checkpointing="nothing_saveable", lmhead_chunksize=2048)
    model = LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device="cuda")
    model.train()
    tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-5), weight_decay=0.01)
    state = EasyDeLState.create(model=model, tx=tx, init_opt_state=True)
    ids = torch.randint(0, 128256, (1, args.tokens), device="cuda")

    def step():
        _, m = model.compute_loss(input_ids=ids, labels=ids)
        m.loss.backward()

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    step()
    e.record()
    torch.cuda.synchronize()
    state.apply_gradients()
    torch.cuda.synchronize()
    from easydel_b200.ops import _lib

    _lib.check_status()
    print(f"layers={args.layers} tokens={args.tokens}: fwd+bwd micro-batch {s.elapsed_time(e):.2f} ms")


def bench_decode(args) -> None:
    """Decode-step kernels at the per-GPU shapes of Llama-3-70B under 8-way tensor parallelism (8 query heads on one
    KV head, hidden 8192, FFN 3584) with 256 running sequences: the streaming decode-attention kernel against the
    general paged kernel, and the four skinny GEMMs of a layer against the weight-streaming bound."""
    from easydel_b200.ops import serving as S

    pk = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    B, Hq, Hkv, D = 256, 8, 1, 128
    for ctx in (700, 2700):
        pages_per = (ctx + 127) // 128
        P = B * pages_per + 1
        kp = torch.randn(P, 128, Hkv, D, device="cuda").to(torch.bfloat16)
        vp = torch.randn(P, 128, Hkv, D, device="cuda").to(torch.bfloat16)
        table = (torch.randperm(P - 1, device="cuda")[: B * pages_per] + 1).to(torch.int32).view(B, pages_per)
        lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
        kv_bytes = 2.0 * B * ctx * Hkv * D * 2
        ms_new = time_cuda(lambda: S.decode_attention(q, kp, vp, lens, table), flush=flush)
        ms_old = time_cuda(lambda: S.paged_attention(q, kp, vp, cu, lens, table, 1), flush=flush)
        print(f"decode attention B={B} ctx={ctx} Hq/Hkv={Hq}/{Hkv}: streaming kernel {ms_new * 1e3:7.1f} us "
              f"({kv_bytes / ms_new / 1e6:6.0f} GB/s, {kv_bytes / ms_new / 1e6 / pk['hbm_gbs']:.2f} of {pk['src']} copy "
              f"bandwidth)   general paged kernel {ms_old * 1e3:7.1f} us", flush=True)
    for name, M, N, Kd in (("qkv", B, 1280, 8192), ("o", B, 8192, 1024), ("gate_up", B, 7168, 8192),
                           ("down", B, 8192, 3584)):
        a = torch.randn(M, Kd, device="cuda").to(torch.bfloat16)
        w = torch.randn(N, Kd, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_cuda(lambda: K.gemm(a, w, out=out), flush=flush)
        ms_lib = time_cuda(lambda: torch.matmul(a, w.t(), out=out), flush=flush)
        wbytes = 2.0 * N * Kd
        print(f"decode GEMM {name:8s} M={M} N={N:5d} K={Kd:5d}: ours {ms * 1e3:6.1f} us ({wbytes / ms / 1e6:5.0f} GB/s of "
              f"weights, {wbytes / ms / 1e6 / pk['hbm_gbs']:.2f} of {pk['src']} copy bandwidth)   cuBLAS "
              f"{ms_lib * 1e3:6.1f} us", flush=True)
        ref = torch.matmul(a.float(), w.float().t())
        t1 = time_cuda(lambda: K.gemm(a, w, out=out, force_bn=-1), flush=flush)
        t384 = time_cuda(lambda: K.gemm(a, w, out=out, force_bn=384), flush=flush)
        e384 = float((out.float() - ref).abs().max() / ref.abs().max())
        print(f"    128-wide single-CTA kernel {t1 * 1e3:.1f} us   CTA pair, 256 x 128 tiles {t384 * 1e3:.1f} us"
              + ("" if e384 < 1e-2 else f" (ERR {e384:.3f})") + f"   planned: "
              f"{'pair 256x128' if K._pair128_plan(M, N, Kd, a.device) else 'other'}", flush=True)
        sweep = []
        for sp in (1, 2, 3, 4, 5, 6, 8):
            t = time_cuda(lambda: K.gemm(a, w, out=out, pair_splits=sp), flush=flush)
            err = float((out.float() - ref).abs().max() / ref.abs().max())
            sweep.append(f"{sp}:{t * 1e3:.1f}us" + ("" if err < 1e-2 else f"(ERR {err:.3f})"))
        print(f"    CTA-pair split-K by slices  {'  '.join(sweep)}   planned slices "
              f"{K._pair_splitk_plan(M, N, Kd, a.device)}", flush=True)
    from easydel_b200.ops import _lib

    _lib.check_status()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("what", choices=["gemm", "attention", "layer", "decode"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=2)
    a = ap.parse_args()
    {"gemm": bench_gemm, "attention": bench_attention, "layer": bench_layer, "decode": bench_decode}[a.what](a)


if __name__ == "__main__":
    main()
