"""Named attention operations: every name resolves, the dense-input operations agree with the fp32 oracle, the
block-sparse form matches an explicit block-diagonal mask, and the paged operations agree with the dense result."""

import pytest
import torch

import easydel_b200 as ed
from easydel_b200.infra.etils import AttentionMechanisms
from easydel_b200.ops import reference as R
from easydel_b200.ops.registry import (BlockSparseAttentionConfig, FlashAttentionConfig, OperationMetadata,
                                       OperationRegistry)


def _qkv(B=2, T=24, Hq=4, Hkv=2, D=16):
    torch.manual_seed(0)
    return torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)


def test_every_mechanism_name_but_mla_has_an_operation():
    names = set(OperationRegistry.list_implementations())
    for m in AttentionMechanisms:
        if m.value != "multi_latent_ragged_page_attention_v1":     # lives in the latent-attention layer itself
            assert m.value in names, m
    with pytest.raises(KeyError):
        OperationRegistry.get("no_such_attention")
    assert ed.FlashAttn is OperationRegistry.get("flash_attn2") and ed.RingAttn.get_impl_name() == "ring"


@pytest.mark.parametrize("name", ["flash_attn2", "vanilla", "sdpa", "auto"])
def test_dense_operations_match_the_oracle(name):
    q, k, v = _qkv()
    op = OperationRegistry.create(name, OperationMetadata(runtime_dtype=torch.float32))
    want = R.attention(q, k, v, causal=True)
    got = op(q, k, v).attention_outputs
    assert got.shape == q.shape and torch.allclose(got, want, atol=1e-5)
    got = op(q, k, v, causal=False).attention_outputs               # a per-call override of the configuration
    assert torch.allclose(got, R.attention(q, k, v, causal=False), atol=1e-5)


def test_configuration_is_applied_and_weights_are_returned():
    q, k, v = _qkv()
    op = ed.FlashAttn(config=FlashAttentionConfig(sliding_window=5, logits_soft_cap=3.0, softmax_scale=0.2))
    want = R.attention(q, k, v, causal=True, sliding_window=5, softcap=3.0, scale=0.2)
    assert torch.allclose(op(q, k, v).attention_outputs, want, atol=1e-5)
    out = ed.VanillaAttn()(q, k, v, output_attentions=True)
    w = out.attention_weights
    assert w.shape == (2, 4, 24, 24) and torch.allclose(w.sum(-1), torch.ones(2, 4, 24), atol=1e-5)
    assert (w.triu(1) == 0).all()
    with pytest.raises(NotImplementedError):
        ed.ScaledDotProductAttn()(q, k, v, sliding_window=4)


def test_blocksparse_is_block_diagonal_causal():
    q, k, v = _qkv(B=1, T=24)
    op = ed.BlockSparseAttn(config=BlockSparseAttentionConfig(chunk_size=8))
    got = op(q, k, v).attention_outputs
    want = torch.cat([R.attention(q[:, i:i + 8], k[:, i:i + 8], v[:, i:i + 8], causal=True) for i in (0, 8, 16)], 1)
    assert torch.allclose(got, want, atol=1e-5)
    assert not torch.allclose(got, R.attention(q, k, v, causal=True), atol=1e-3)


def test_paged_operations_match_dense_attention():
    from easydel_b200.caching.paged import PAGE_SIZE

    torch.manual_seed(0)
    Hq, Hkv, D = 4, 2, 16
    lens, new = [150, 40], [3, 1]                       # keys per sequence (after the append), new tokens of each
    P = 6
    k_pages, v_pages = torch.randn(P, PAGE_SIZE, Hkv, D), torch.randn(P, PAGE_SIZE, Hkv, D)
    table = torch.tensor([[2, 4, -1], [1, -1, -1]], dtype=torch.int32)
    q = torch.randn(sum(new), Hq, D)
    cu = torch.tensor([0, 3, 4], dtype=torch.int32)
    kv_lens = torch.tensor(lens, dtype=torch.int32)
    want = []
    for b in range(2):
        pages = [int(p) for p in table[b] if p >= 0]
        kk = torch.cat([k_pages[p] for p in pages])[:lens[b]][None]
        vv = torch.cat([v_pages[p] for p in pages])[:lens[b]][None]
        want.append(R.attention(q[cu[b]:cu[b + 1]][None], kk, vv, causal=True)[0])
    want = torch.cat(want)
    for name in ("ragged_page_attention_v2", "ragged_page_attention_v3", "paged_flash_attention", "page_attention"):
        out = OperationRegistry.create(name)(q, k_pages=k_pages, v_pages=v_pages, cu_q=cu, kv_lens=kv_lens,
                                             page_table=table, max_q=3)
        assert torch.allclose(out.attention_outputs, want, atol=1e-5), name
    dec = ed.AutoRegressiveDecodeAttn()(q[[2, 3]], k_pages, v_pages, kv_lens, table).attention_outputs
    assert torch.allclose(dec, want[[2, 3]], atol=1e-5)


def test_flexible_module_follows_the_configs_mechanism():
    class Cfg:
        attn_mechanism = "vanilla"
        mesh = None

    q, k, v = _qkv()
    mod = ed.FlexibleAttentionModule(Cfg(), softmax_scale=0.3)
    assert mod.mechanism == "vanilla" and isinstance(mod.impl, ed.VanillaAttn)
    assert torch.allclose(mod(q, k, v).attention_outputs, R.attention(q, k, v, causal=True, scale=0.3), atol=1e-5)
    assert isinstance(ed.FlexibleAttentionModule(attn_mechanism="ring").impl, ed.RingAttn)
    with pytest.raises(ValueError):
        ed.FlexibleAttentionModule(attn_mechanism="ring")(q, k, v)          # no process group given
    assert ed.AttentionModule is ed.layers.attention.Attention
