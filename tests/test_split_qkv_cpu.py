"""The packed q / k / v split: same values and gradients as three slices, no copies when the incoming gradients
already are the slices of one packed buffer."""

import torch

from easydel_b200.ops import functional as F


def _loss(q, k, v):
    return (q ** 2).sum() + (k * 3).sum() + v.sin().sum()


def test_split_qkv_matches_slices_and_their_gradients():
    B, T, Hq, Hkv, D = 2, 5, 4, 2, 8
    torch.manual_seed(0)
    x = torch.randn(B, T, (Hq + 2 * Hkv) * D, requires_grad=True)
    q, k, v = F.split_qkv(x, Hq, Hkv, D)
    assert q.shape == (B, T, Hq, D) and k.shape == v.shape == (B, T, Hkv, D)
    assert q.data_ptr() == x.data_ptr()                      # views, not copies
    _loss(q, k, v).backward()
    got, x.grad = x.grad.clone(), None
    q2 = x[..., : Hq * D].view(B, T, Hq, D)
    k2 = x[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v2 = x[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
    _loss(q2, k2, v2).backward()
    assert torch.allclose(got, x.grad)
    # a branch that gets no gradient contributes zeros
    x.grad = None
    q, k, v = F.split_qkv(x, Hq, Hkv, D)
    q.sum().backward()
    assert x.grad[..., : Hq * D].eq(1).all() and x.grad[..., Hq * D:].eq(0).all()
    # without autograd the plain views come back
    with torch.no_grad():
        q, k, v = F.split_qkv(x, Hq, Hkv, D)
    assert q.grad_fn is None and torch.equal(v, v2)


def test_packed_gradient_buffers_are_recognised():
    B, T, Hq, Hkv, D = 2, 3, 4, 2, 8
    base, dq, dk, dv = F.packed_qkv_buffers(B, T, Hq, Hkv, D, torch.float32, "cpu")
    base.normal_()
    packed = F.packed_qkv_base(dq, dk, dv, B, T, Hq, Hkv, D)
    assert packed is not None and packed.data_ptr() == base.data_ptr() and torch.equal(packed, base)
    # anything else (fresh tensors, swapped order, another buffer) is not mistaken for it
    assert F.packed_qkv_base(dq.clone(), dk, dv, B, T, Hq, Hkv, D) is None
    assert F.packed_qkv_base(dq, dv, dk, B, T, Hq, Hkv, D) is None
    _, _, dk2, _ = F.packed_qkv_buffers(B, T, Hq, Hkv, D, torch.float32, "cpu")
    assert F.packed_qkv_base(dq, dk2, dv, B, T, Hq, Hkv, D) is None
    # the split's backward hands such a buffer through untouched
    x = torch.randn(B, T, (Hq + 2 * Hkv) * D, requires_grad=True)
    q, k, v = F.split_qkv(x, Hq, Hkv, D)
    torch.autograd.backward([q, k, v], [dq, dk, dv])
    assert x.grad.data_ptr() == base.data_ptr() or torch.equal(x.grad, base)
