"""Layer kernels (RMSNorm, gated activation, RoPE, embedding, CE, AdamW) against fp32 PyTorch math."""

import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("D", [256, 4096, 8192, 2048 + 8])
def test_rmsnorm_fwd_bwd(D):
    from easydel_b200.ops import kernels as K

    T = 300
    x, res, w, dy = _bf(T, D, seed=1), _bf(T, D, seed=2), _bf(D, seed=3) * 0.1 + 1, _bf(T, D, seed=4)
    y, h, rstd = K.rmsnorm_fwd(x, w, 1e-5, residual=res)
    hf = (x.float() + res.float()).to(torch.bfloat16).float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    yr = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    assert torch.allclose(h.float(), hf.detach(), atol=0, rtol=0)
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    yr.backward(dy.float())
    dx, dw = K.rmsnorm_bwd(h, w, dy, rstd)
    assert torch.allclose(dx.float(), hf.grad, atol=3e-2, rtol=2e-2)
    assert torch.allclose(dw, wf.grad, atol=0.15, rtol=2e-2)
    y2, h2, _ = K.rmsnorm_fwd(x, w, 1e-5)
    xr = x.float()
    assert torch.allclose(y2.float(), xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float(),
                          atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "gelu", "relu"])
def test_gated_act(act):
    from easydel_b200.ops import kernels as K

    T, Fd = 257, 688
    gu, dh = _bf(T, 2 * Fd, seed=5), _bf(T, Fd, seed=6)
    guf = gu.float().requires_grad_(True)
    fn = {"silu": F.silu, "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "gelu": F.gelu, "relu": F.relu}[act]
    ref = fn(guf[:, :Fd]) * guf[:, Fd:]
    h = K.gated_act_fwd(gu, act)
    assert torch.allclose(h.float(), ref, atol=3e-2, rtol=2e-2)
    ref.backward(dh.float())
    dgu = K.gated_act_bwd(gu, dh, act)
    assert torch.allclose(dgu.float(), guf.grad, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(interleaved):
    from easydel_b200.ops import kernels as K

    T, H, Hkv, D = 100, 8, 4, 64
    qkv = _bf(T, (H + 2 * Hkv) * D, seed=7)
    pos = torch.randint(0, 512, (T,), device="cuda")
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(512, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ref = qkv.float().clone().view(T, H + 2 * Hkv, D)
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    qk = ref[:, : H + Hkv]
    if interleaved:
        x1, x2 = qk[..., 0::2], qk[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], -1).flatten(-2)
    else:
        x1, x2 = qk[..., : D // 2], qk[..., D // 2:]
        o = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    ref[:, : H + Hkv] = o
    out = qkv.clone()
    K.rope_(out, pos, cos, sin, H + Hkv, D, interleaved=interleaved)
    assert torch.allclose(out.float().view(T, -1, D), ref, atol=3e-2, rtol=2e-2)
    # backward is the transpose: applying it to the output restores the input
    K.rope_(out, pos, cos, sin, H + Hkv, D, interleaved=interleaved, backward=True)
    assert torch.allclose(out.float(), qkv.float(), atol=6e-2, rtol=3e-2)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("col0", [0, 128])
def test_rope_vector_copy(interleaved, col0):
    """The one-pass vector form (rotate the heads, copy the other columns) against the scalar in-place kernel, out of
    place and in place, forward and transpose, and through autograd."""
    from easydel_b200.ops import functional as F
    from easydel_b200.ops import kernels as K

    T, H, Hkv, D = 203, 8, 2, 128
    width = col0 + (H + 2 * Hkv) * D
    qkv = _bf(T, width, seed=17)
    pos = torch.randint(0, 1024, (T,), device="cuda")
    inv = 1.0 / (500000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(1024, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    assert K.rope_copy_supported(qkv, cos, sin, H + Hkv, D, col0, None)
    rot = slice(col0, col0 + (H + Hkv) * D)

    def same(a, b):
        # rotated columns: the two kernels may contract their multiply-adds differently (one bf16 ulp); the copied
        # columns are bit-identical
        keep = torch.ones(width, dtype=torch.bool, device="cuda")
        keep[rot] = False
        return (torch.allclose(a[:, rot].float(), b[:, rot].float(), atol=4e-2, rtol=2e-2)
                and torch.equal(a[:, keep], b[:, keep]))

    for backward in (False, True):
        ref = qkv.clone()
        K.rope_(ref, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved, backward=backward)
        out = torch.full_like(qkv, float("nan"))
        K.rope_copy(qkv, out, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved, backward=backward)
        assert same(out, ref)
        inplace = qkv.clone()
        K.rope_copy(inplace, inplace, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved, backward=backward)
        assert same(inplace, ref)
    x = qkv.clone().requires_grad_(True)
    y = F.rope_packed(x, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved)
    ref = qkv.clone()
    K.rope_(ref, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved)
    assert same(y.detach(), ref)
    dy = _bf(T, width, seed=18)
    y.backward(dy)
    dref = dy.clone()
    K.rope_(dref, pos, cos, sin, H + Hkv, D, col0=col0, interleaved=interleaved, backward=True)
    assert same(x.grad, dref)


def test_embedding():
    from easydel_b200.ops import kernels as K

    V, D, T = 1000, 256, 777
    table = _bf(V, D, seed=8)
    ids = torch.randint(0, V, (T,), device="cuda")
    out = K.embed_fwd(table, ids)
    assert torch.equal(out, table[ids])
    dout = _bf(T, D, seed=9)
    g = torch.zeros(V, D, device="cuda")
    K.embed_bwd_(g, dout, ids)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, ids, dout.float())
    assert torch.allclose(g, ref, atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("ls,zl", [(0.0, 0.0), (0.1, 1e-4)])
def test_cross_entropy(ls, zl):
    from easydel_b200.ops import kernels as K

    T, V = 65, 1024 + 8
    logits = _bf(T, V, seed=10, scale=3.0)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    lf = logits.float().requires_grad_(True)
    lse = torch.logsumexp(lf, -1)
    per = F.cross_entropy(lf, labels, ignore_index=-100, label_smoothing=ls, reduction="none")
    per = per + zl * lse.pow(2) * (labels != -100)
    n = (labels != -100).sum()
    (per.sum() / n).backward()
    work = logits.clone()
    loss, lse_k, correct = K.cross_entropy_(work, labels, label_smoothing=ls, z_loss=zl, grad_scale=1.0 / n.item(),
                                            want_correct=True)
    assert torch.allclose(loss, per.detach(), atol=2e-3, rtol=1e-3)
    assert torch.allclose(lse_k, lse.detach(), atol=2e-3, rtol=1e-3)
    assert torch.allclose(work.float(), lf.grad, atol=2e-4, rtol=2e-2)
    pred_ok = (lf.argmax(-1) == labels) & (labels != -100)
    assert torch.equal(correct.bool(), pred_ok)


def test_token_logprob():
    from easydel_b200.ops import kernels as K

    T, V = 33, 2048
    logits = _bf(T, V, seed=11, scale=2.0)
    labels = torch.randint(0, V, (T,), device="cuda")
    lf = logits.float().requires_grad_(True)
    lp_all = torch.log_softmax(lf, -1)
    ref = lp_all.gather(-1, labels[:, None]).squeeze(-1)
    ent_ref = -(lp_all.exp() * lp_all).sum(-1)
    logp, lse, ent = K.token_logprob(logits, labels, want_entropy=True)
    assert torch.allclose(logp, ref.detach(), atol=2e-3, rtol=1e-3)
    assert torch.allclose(ent, ent_ref.detach(), atol=2e-3, rtol=1e-3)
    dl = torch.randn(T, device="cuda")
    ref.backward(dl)
    work = logits.clone()
    K.token_logprob_bwd_(work, labels, lse, dl)
    assert torch.allclose(work.float(), lf.grad, atol=5e-3, rtol=2e-2)


def test_adamw_and_gradnorm():
    from easydel_b200.ops import kernels as K

    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        pr.grad = g.clone() * 0.5
        opt.step()
        K.adamw_(p, p16, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=step, gscale=0.5)
    assert torch.allclose(p, pr.detach(), atol=1e-5, rtol=1e-5)
    assert torch.equal(p16, p.to(torch.bfloat16))
    ss = torch.zeros(1, device="cuda")
    K.sumsq_(ss, g)
    norm, coef, skip = K.clip_coef(ss, 0.5, 1.0)
    ref_norm = g.norm().item() * 0.5
    assert math.isclose(norm.item(), ref_norm, rel_tol=1e-4)
    assert math.isclose(coef.item(), min(1.0, 1.0 / (ref_norm + 1e-6)), rel_tol=1e-4)
    assert skip.item() == 0
