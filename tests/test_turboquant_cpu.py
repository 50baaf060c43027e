"""TurboQuant KV compression: codebook optimality, reconstruction error, unbiased key scores, attention accuracy."""

import torch

from easydel_b200.layers import turboquant as TQ


def test_lloyd_max_codebook_is_symmetric_sorted_and_beats_uniform():
    cb = TQ.solve_lloyd_max(3, 128)
    assert cb.shape == (8,) and torch.all(cb[1:] > cb[:-1]) and torch.allclose(cb, -cb.flip(0), atol=1e-5)
    u = torch.nn.functional.normalize(torch.randn(4000, 128), dim=-1).reshape(-1)
    err = (u - cb[TQ._nearest(u, cb)]).pow(2).mean()
    uni = torch.linspace(-float(u.abs().max()), float(u.abs().max()), 8)
    assert err < (u - uni[TQ._nearest(u, uni)]).pow(2).mean() * 0.7


def test_value_roundtrip_error_shrinks_with_bits():
    v = torch.randn(2, 4, 50, 64)
    errs = []
    for bits in (2, 4, 6):
        k = TQ.TurboQuantConstants.create(TQ.TurboQuantConfig(bits=bits), 64)
        rec = TQ.dequantize_values(*TQ.quantize_values(v, k), k)
        errs.append(float((rec - v).pow(2).sum() / v.pow(2).sum()))
    assert errs[0] > errs[1] > errs[2] and errs[1] < 0.02


def test_key_scores_are_unbiased_and_sketch_helps():
    torch.manual_seed(0)
    d = 64
    key = torch.randn(1, d)
    q = key * 0.5 + torch.randn(1, d) * 0.2              # correlated with the key: where the bias shows
    exact = float(q @ key.t())
    est, est_nosketch = [], []
    for seed in range(300):
        k = TQ.TurboQuantConstants.create(TQ.TurboQuantConfig(bits=3, seed=seed), d)
        codes, norms, signs, rn = TQ.quantize_keys(key, k)
        est.append(float(TQ.key_scores(q, codes, norms, signs, rn, k)))
        est_nosketch.append(float(TQ.key_scores(q, codes, norms, signs, torch.zeros_like(rn), k)))
    m, m0 = sum(est) / len(est), sum(est_nosketch) / len(est_nosketch)
    assert abs(m - exact) < 0.02 * abs(exact)                      # unbiased with the sign sketch
    assert abs(m0 - exact) > 2 * abs(m - exact)                    # biased (shrunk) without it


def test_attention_over_compressed_cache_is_close_to_exact():
    torch.manual_seed(1)
    B, H, T, d = 1, 2, 96, 128
    q, kk, v = torch.randn(B, H, T, d), torch.randn(B, H, T, d), torch.randn(B, H, T, d)
    cfg = TQ.TurboQuantConfig(bits=4)
    k = TQ.TurboQuantConstants.create(cfg, d)
    out = TQ.attention(q, TQ.quantize_keys(kk, k), TQ.quantize_values(v, k), k)
    s = (q @ kk.transpose(-1, -2)) * d ** -0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    ref = torch.softmax(s, -1) @ v
    rel = float((out - ref).norm() / ref.norm())
    k2 = TQ.TurboQuantConstants.create(TQ.TurboQuantConfig(bits=2), d)
    out2 = TQ.attention(q, TQ.quantize_keys(kk, k2), TQ.quantize_values(v, k2), k2)
    assert rel < 0.3 and rel < float((out2 - ref).norm() / ref.norm()), rel
    assert 3.0 < TQ.compression_ratio(cfg, d) < 4.2
