"""Kernels between guard bands: ragged shapes of the GEMM, norm, attention, MoE and serving kernels write nothing
outside their outputs, and a table index that is out of range is reported through the status word and skipped."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_guard_detects_a_stray_write():
    from easydel_b200.utils.canary import CanaryGuard

    with pytest.raises(AssertionError, match="guard byte"):
        with CanaryGuard():
            t = torch.empty(1000, dtype=torch.float32, device="cuda")
            # the tensor's storage is the guarded buffer: a view built past the end stands in for a bad kernel index
            torch.as_strided(t, (1001,), (1,))[1000:].fill_(1.0)


def test_kernels_stay_inside_their_outputs():
    from easydel_b200.layers.moe import MoEBlock
    from easydel_b200.ops import attention as A, functional as F, kernels as K, serving as S, _lib
    from easydel_b200.utils.canary import CanaryGuard

    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn(300, 264, device=dev).to(torch.bfloat16)
    w = torch.randn(520, 264, device=dev).to(torch.bfloat16)
    bias = torch.randn(520, device=dev).to(torch.bfloat16)
    x = torch.randn(77, 1000, device=dev).to(torch.bfloat16)
    nw = torch.randn(1000, device=dev).to(torch.bfloat16)
    q = torch.randn(1, 333, 4, 128, device=dev).to(torch.bfloat16)
    k = torch.randn(1, 333, 2, 128, device=dev).to(torch.bfloat16)
    v = torch.randn(1, 333, 2, 128, device=dev).to(torch.bfloat16)
    block = MoEBlock(256, 128, 8, 2, dtype=torch.bfloat16).to(dev)
    xm = torch.randn(1, 150, 256, device=dev).to(torch.bfloat16)
    pages_k = torch.randn(9, 128, 1, 128, device=dev).to(torch.bfloat16)
    pages_v = torch.randn(9, 128, 1, 128, device=dev).to(torch.bfloat16)
    table = torch.arange(1, 9, dtype=torch.int32, device=dev).view(2, 4)
    lens = torch.tensor([500, 129], dtype=torch.int32, device=dev)
    qd = torch.randn(2, 8, 128, device=dev).to(torch.bfloat16)
    with CanaryGuard() as guard:
        c1 = K.gemm(a, w, bias=bias)                       # ragged M, N, K on the single-CTA kernel
        c2 = K.gemm(a, w, force_bn=512)                    # the CTA-pair kernel with partial tiles
        c3 = K.gemm(a[:200], w, pair_splits=2)             # split-K epilogue
        y, h, rstd = K.rmsnorm_fwd(x, nw, 1e-5, residual=x)
        o, lse = A.attn_fwd(q, k, v, causal=True)
        dq, dk, dv = A.attn_bwd(q, k, v, o, lse, torch.randn_like(o), causal=True)
        ym, _ = block(xm)
        od = S.decode_attention(qd, pages_k, pages_v, lens, table)
        od2 = S.decode_attention(qd, pages_k, pages_v, lens, table, num_splits=2)
        logits = torch.randn(5, 1000, device=dev)
        toks, _ = S.sample(logits)
        assert len(guard.live) >= 10
    ref = a.float() @ w.float().t()
    assert (c1.float() - ref - bias.float()).abs().max() < 2e-2 * ref.abs().max()
    assert (c2.float() - ref).abs().max() < 2e-2 * ref.abs().max()
    assert (c3.float() - ref[:200]).abs().max() < 2e-2 * ref.abs().max()
    assert torch.isfinite(ym.float()).all() and torch.isfinite(od.float()).all() and torch.isfinite(od2.float()).all()
    _lib.check_status(torch.device(dev))


def test_out_of_range_slot_is_reported_and_skipped():
    """A page slot beyond the pool: the append kernel records EDL_BAD_INDEX, writes nothing for that token, and the
    context keeps working."""
    from easydel_b200.ops import _lib, serving as S
    from easydel_b200.utils.canary import CanaryGuard

    dev = torch.device("cuda")
    with CanaryGuard():
        kp = torch.zeros(4, 128, 1, 64, dtype=torch.bfloat16, device=dev)
        vp = torch.zeros(4, 128, 1, 64, dtype=torch.bfloat16, device=dev)
        k = torch.ones(3, 1, 64, dtype=torch.bfloat16, device=dev)
        slots = torch.tensor([5, 4 * 128 + 7, -1], dtype=torch.int32, device=dev)     # in range, beyond the pool, padding
        S.kv_append(k, k, kp, vp, slots)
        torch.cuda.synchronize()
        assert float(kp.view(-1, 64)[5].sum()) == 64.0 and float(kp.sum()) == 64.0
    with pytest.raises(RuntimeError):
        _lib.check_status(dev)
    _lib.status_word(dev).zero_()
    S.kv_append(k[:1], k[:1], kp, vp, slots[:1])
    torch.cuda.synchronize()
    _lib.check_status(dev)
