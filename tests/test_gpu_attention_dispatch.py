"""Head sizes outside 64 / 128 on the GPU: zero-padded into the flash kernels, or the fused library attention."""

import pytest
import torch

from easydel_b200.ops import functional as F
from easydel_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,Dv,causal", [(80, 80, True), (32, 32, False), (72, 72, False), (192, 128, True),
                                         (256, 256, True)])
def test_odd_head_sizes_match_reference(D, Dv, causal):
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    B, T, Hq, Hkv = 2, 300, 4, 2
    q = torch.randn(B, T, Hq, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, Dv, device=dev, dtype=torch.bfloat16, requires_grad=True)
    o = F.attention(q, k, v, causal=causal)
    want = R.attention(q.float(), k.float(), v.float(), causal=causal)
    assert o.shape == (B, T, Hq, Dv)
    assert (o.float() - want).abs().max() < 3e-2
    o.float().pow(2).sum().backward()
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all() and q.grad.abs().sum() > 0


def test_fp32_inputs_take_the_library_path():
    dev = torch.device("cuda", 0)
    q, k, v = (torch.randn(1, 64, 4, 64, device=dev) for _ in range(3))
    o = F.attention(q, k, v, causal=True)
    assert o.dtype == torch.float32
    assert (o - R.attention(q, k, v, causal=True)).abs().max() < 2e-3
