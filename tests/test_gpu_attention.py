"""Flash-attention kernels (tcgen05) against dense fp32 attention."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _qkv(B, T, Hq, Hkv, D, seed=0, packed=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if packed:
        buf = torch.randn(B, T, (Hq + 2 * Hkv) * D, device="cuda", generator=g).to(torch.bfloat16)
        q = buf[..., : Hq * D].view(B, T, Hq, D)
        k = buf[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
        v = buf[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
        return q, k, v
    mk = lambda h: torch.randn(B, T, h, D, device="cuda", generator=g).to(torch.bfloat16)
    return mk(Hq), mk(Hkv), mk(Hkv)


@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(1, 128, 2, 1, 128), (2, 384, 4, 2, 128), (1, 1000, 4, 4, 64),
                                          (1, 2048, 8, 2, 128), (3, 77, 2, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_fwd(B, T, Hq, Hkv, D, causal):
    from easydel_b200.ops import attention as A, reference as R

    q, k, v = _qkv(B, T, Hq, Hkv, D, seed=T)
    o, lse = A.attn_fwd(q, k, v, causal=causal)
    ref, lse_ref = R.attention(q, k, v, causal=causal, return_lse=True)
    assert torch.allclose(o.float(), ref.float(), atol=2e-2, rtol=2e-2), (o.float() - ref.float()).abs().max()
    assert torch.allclose(lse.view(Hq, B, T).permute(1, 0, 2), lse_ref, atol=2e-2, rtol=1e-3)


def test_attn_fwd_window_softcap_sinks():
    from easydel_b200.ops import attention as A, reference as R

    q, k, v = _qkv(1, 700, 4, 2, 128, seed=5)
    sinks = torch.randn(4, device="cuda")
    o, _ = A.attn_fwd(q, k, v, causal=True, window=200, softcap=30.0, sinks=sinks)
    ref = R.attention(q, k, v, causal=True, sliding_window=200, softcap=30.0, sinks=sinks)
    assert torch.allclose(o.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_attn_fwd_varlen_matches_segments():
    from easydel_b200.ops import attention as A, reference as R

    B, T, Hq, Hkv, D = 2, 512, 4, 2, 128
    q, k, v = _qkv(B, T, Hq, Hkv, D, seed=6)
    seg = torch.ones(B, T, dtype=torch.int32, device="cuda")
    seg[0, 100:300] = 2
    seg[0, 300:] = 3
    seg[1, 257:] = 2
    cu, mx = A.segment_ids_to_cu_seqlens(seg)
    o, _ = A.attn_fwd(q.view(-1, Hq, D), k.view(-1, Hkv, D), v.view(-1, Hkv, D), causal=True, cu_q=cu, cu_k=cu,
                      max_q=mx, max_k=mx)
    ref = R.attention(q, k, v, causal=True, segment_ids=seg)
    assert torch.allclose(o.view(B, T, Hq, D).float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_attn_fwd_prefix_offset():
    """Fewer queries than keys: the queries are the last rows (chunked prefill over a cached prefix)."""
    from easydel_b200.ops import attention as A, reference as R

    q, k, v = _qkv(1, 640, 4, 2, 128, seed=7, packed=False)
    qs = q[:, 400:].contiguous()
    o, _ = A.attn_fwd(qs, k, v, causal=True)
    ref = R.attention(qs, k, v, causal=True)
    assert torch.allclose(o.float(), ref.float(), atol=2e-2, rtol=2e-2)


def _grads_ref(q, k, v, do, **kw):
    from easydel_b200.ops import reference as R

    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o = R.attention(qf, kf, vf, **kw)
    o.backward(do.float())
    return o.detach(), qf.grad, kf.grad, vf.grad


def _check_grad(name, got, ref):
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= 3e-2 * scale + 2e-2, f"{name}: max err {err} (scale {scale})"


@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(1, 128, 1, 1, 128), (2, 384, 4, 2, 128), (1, 520, 4, 1, 64),
                                          (1, 1024, 8, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attn_bwd(B, T, Hq, Hkv, D, causal):
    from easydel_b200.ops import attention as A

    q, k, v = _qkv(B, T, Hq, Hkv, D, seed=T + 1)
    do = torch.randn(B, T, Hq, D, device="cuda").to(torch.bfloat16)
    o, lse = A.attn_fwd(q, k, v, causal=causal)
    dq, dk, dv = A.attn_bwd(q, k, v, o, lse, do, causal=causal)
    _, rq, rk, rv = _grads_ref(q, k, v, do, causal=causal)
    _check_grad("dq", dq, rq)
    _check_grad("dk", dk, rk)
    _check_grad("dv", dv, rv)


def test_attn_bwd_varlen_window_softcap():
    from easydel_b200.ops import attention as A

    B, T, Hq, Hkv, D = 1, 640, 4, 2, 128
    q, k, v = _qkv(B, T, Hq, Hkv, D, seed=11)
    do = torch.randn(B, T, Hq, D, device="cuda").to(torch.bfloat16)
    seg = torch.ones(B, T, dtype=torch.int32, device="cuda")
    seg[0, 200:450] = 2
    seg[0, 450:] = 3
    cu, mx = A.segment_ids_to_cu_seqlens(seg)
    q3, k3, v3, do3 = (t.reshape(-1, t.shape[-2], D) for t in (q, k, v, do))
    o, lse = A.attn_fwd(q3, k3, v3, causal=True, window=150, softcap=20.0, cu_q=cu, cu_k=cu, max_q=mx, max_k=mx)
    dq, dk, dv = A.attn_bwd(q3, k3, v3, o, lse, do3, causal=True, window=150, softcap=20.0, cu_q=cu, cu_k=cu,
                            max_q=mx, max_k=mx)
    _, rq, rk, rv = _grads_ref(q, k, v, do, causal=True, segment_ids=seg, sliding_window=150, softcap=20.0)
    _check_grad("dq", dq.view(B, T, Hq, D), rq)
    _check_grad("dk", dk.view(B, T, Hkv, D), rk)
    _check_grad("dv", dv.view(B, T, Hkv, D), rv)


def test_flash_attention_autograd():
    from easydel_b200.ops import functional as F_, reference as R

    q, k, v = _qkv(2, 256, 4, 2, 128, seed=13, packed=False)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o = F_.attention(q, k, v, causal=True)
    w = torch.randn_like(o)
    (o.float() * w.float()).sum().backward()
    _, rq, rk, rv = _grads_ref(q, k, v, w, causal=True)
    _check_grad("dq", q.grad, rq)
    _check_grad("dk", k.grad, rk)
    _check_grad("dv", v.grad, rv)


def test_attention_sinks_backward():
    """Sliding window + sinks (the gpt-oss layer form): gradients of q, k, v and of the sink logits against autograd
    through the dense fp32 attention."""
    from easydel_b200.ops import attention as A, reference as R

    q, k, v = _qkv(2, 320, 4, 2, 64, seed=21, packed=False)
    sinks = torch.randn(4, device="cuda")
    w = torch.randn(2, 320, 4, 64, device="cuda")
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, sinks)]
    o = A.flash_attention(*leaves[:3], causal=True, sliding_window=96, sinks=leaves[3])
    (o.float() * w).sum().backward()
    ref_leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, sinks)]
    ro = R.attention(*ref_leaves[:3], causal=True, sliding_window=96, sinks=ref_leaves[3])
    (ro.float() * w).sum().backward()
    for name, a, b in zip(("dq", "dk", "dv"), leaves[:3], ref_leaves[:3]):
        _check_grad(name, a.grad, b.grad)
    assert torch.allclose(leaves[3].grad, ref_leaves[3].grad, rtol=3e-2, atol=3e-2 * float(ref_leaves[3].grad.abs().max()))


def test_attn_benchmarked_shape_against_oracle():
    """The shape the training benchmark runs (8192 tokens, 32 query / 8 KV heads, D = 128, causal), forward and
    backward, against dense fp32 attention. The reference is formed one GQA group at a time (1 GB of scores)."""
    from easydel_b200.ops import attention as A

    B, T, Hq, Hkv, D = 1, 8192, 32, 8, 128
    q, k, v = _qkv(B, T, Hq, Hkv, D, seed=21)
    do = torch.randn(B, T, Hq, D, device="cuda").to(torch.bfloat16)
    o, lse = A.attn_fwd(q, k, v, causal=True)
    dq, dk, dv = A.attn_bwd(q, k, v, o, lse, do, causal=True)
    G = Hq // Hkv
    for g in (0, 5, 7):
        hs = slice(g * G, (g + 1) * G)
        ref_o, rq, rk, rv = _grads_ref(q[:, :, hs], k[:, :, g:g + 1], v[:, :, g:g + 1], do[:, :, hs], causal=True)
        assert torch.allclose(o[:, :, hs].float(), ref_o, atol=2e-2, rtol=2e-2), (o[:, :, hs].float() - ref_o).abs().max()
        _check_grad("dq", dq[:, :, hs], rq)
        _check_grad("dk", dk[:, :, g:g + 1], rk)
        _check_grad("dv", dv[:, :, g:g + 1], rv)
        del ref_o, rq, rk, rv
