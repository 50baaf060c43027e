"""The attention dispatcher's path for shapes outside the flash kernels against the dense fp32 form."""

import pytest
import torch

from easydel_b200.ops import functional as F
from easydel_b200.ops import reference as R


@pytest.mark.parametrize("case", ["causal", "decode_suffix", "window", "segments", "bidirectional_segments",
                                  "wide_keys_narrow_values"])
def test_library_attention_matches_dense_form(case):
    torch.manual_seed(0)
    B, Tq, Tk, Hq, Hkv, D, Dv = 2, 12, 12, 4, 2, 24, 24
    kw = dict(causal=True, scale=None, segment_ids=None, sliding_window=None)
    if case == "decode_suffix":
        Tq = 3
    elif case == "window":
        kw["sliding_window"] = 5
    elif case in ("segments", "bidirectional_segments"):
        seg = torch.tensor([[1] * 5 + [2] * 4 + [0] * 3, [1] * 12], dtype=torch.int32)
        kw["segment_ids"] = seg
        kw["causal"] = case == "segments"
    elif case == "wide_keys_narrow_values":
        D, Dv, kw["scale"] = 48, 16, 0.2
    q, k, v = torch.randn(B, Tq, Hq, D), torch.randn(B, Tk, Hkv, D), torch.randn(B, Tk, Hkv, Dv)
    want = R.attention(q, k, v, **kw)
    got = F._library_attention(q, k, v, kw["causal"], kw["scale"], kw["segment_ids"], kw["sliding_window"], 0.0, None)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
    q.requires_grad_(True)
    F._library_attention(q, k, v, kw["causal"], kw["scale"], kw["segment_ids"], kw["sliding_window"], 0.0,
                         None).sum().backward()
    assert torch.isfinite(q.grad).all()
