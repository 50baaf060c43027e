"""TurboQuant-compressed paged KV cache: bit packing, the paged attention against the dense compressed attention of
``layers/turboquant``, memory accounting, and the serving engine running on it."""

import types

import torch

from easydel_b200.caching.paged import PagedBatchMeta
from easydel_b200.caching.turboquant_paged import (TurboQuantPagedKVCache, pack_bits, pack_nibbles, unpack_bits,
                                                   unpack_nibbles)
from easydel_b200.layers import turboquant as TQ


def test_packing_round_trips():
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (3, 5, 64), generator=g, dtype=torch.uint8)
    assert pack_nibbles(codes).shape == (3, 5, 32) and torch.equal(unpack_nibbles(pack_nibbles(codes)), codes)
    bits = torch.rand(4, 7, 128, generator=g) > 0.5
    assert pack_bits(bits).shape == (4, 7, 16) and torch.equal(unpack_bits(pack_bits(bits)), bits)


def test_paged_compressed_attention_matches_the_dense_compressed_form():
    torch.manual_seed(1)
    Hq, Hkv, D = 4, 2, 64
    cfg = TQ.TurboQuantConfig(bits=4)
    cache = TurboQuantPagedKVCache(num_layers=1, num_pages=8, num_kv_heads=Hkv, head_dim=D, config=cfg, device="cpu")
    assert 3.0 < cache.compression_ratio() < 3.6        # 256 bf16 bytes against 32 + 8 + 4 + 32 + 2
    attn = types.SimpleNamespace(scale=D ** -0.5, softcap=None, sliding_window=None, sinks=None)
    view = cache.view(0)
    lens = [150, 40]                                     # sequence 0 spans two pages
    pages = [[1, 2], [3]]
    K = [torch.randn(n + 1, Hkv, D) for n in lens]       # one more token arrives in the decode step
    V = [torch.randn(n + 1, Hkv, D) for n in lens]
    Q = [torch.randn(n + 1, Hq, D) for n in lens]
    table = torch.zeros(2, 4, dtype=torch.int32)
    for b, pg in enumerate(pages):
        table[b, :len(pg)] = torch.tensor(pg)

    def slots(b, lo, hi):
        return [pages[b][i // 128] * 128 + i % 128 for i in range(lo, hi)]

    # prefill of both sequences in one step
    meta = PagedBatchMeta(cu_q=torch.tensor([0, 150, 190], dtype=torch.int32),
                          kv_lens=torch.tensor(lens, dtype=torch.int32), page_table=table,
                          slot_mapping=torch.tensor(slots(0, 0, 150) + slots(1, 0, 40), dtype=torch.int32),
                          max_q=150, num_seqs=2)
    q = torch.cat([Q[0][:150], Q[1][:40]])[None]
    k = torch.cat([K[0][:150], K[1][:40]])[None]
    v = torch.cat([V[0][:150], V[1][:40]])[None]
    out = view.attend(attn, q, k, v, attn_meta=meta)[0]
    consts = cache.constants

    def dense(b, n_q, n_k):
        kq = TQ.quantize_keys(K[b][:n_k].permute(1, 0, 2)[None], consts)
        vq = TQ.quantize_values(V[b][:n_k].permute(1, 0, 2)[None], consts)
        # norms go through bf16 in the pools
        kq = (kq[0], kq[1].bfloat16().float(), kq[2], kq[3].bfloat16().float())
        vq = (vq[0], vq[1].bfloat16().float())
        qq = Q[b][n_k - n_q:n_k].permute(1, 0, 2)[None]                     # [1, Hq, Tq, D]
        qq = qq.view(1, Hkv, Hq // Hkv, n_q, D)
        o = torch.stack([TQ.attention(qq[:, :, g], kq, vq, consts, scale=attn.scale) for g in range(Hq // Hkv)], 2)
        return o.reshape(1, Hq, n_q, D)[0].permute(1, 0, 2)

    assert torch.allclose(out[:150], dense(0, 150, 150), atol=2e-4, rtol=2e-4)
    assert torch.allclose(out[150:], dense(1, 40, 40), atol=2e-4, rtol=2e-4)
    # one decode token per sequence on top of the stored pages
    meta = PagedBatchMeta(cu_q=torch.tensor([0, 1, 2], dtype=torch.int32),
                          kv_lens=torch.tensor([151, 41], dtype=torch.int32), page_table=table,
                          slot_mapping=torch.tensor(slots(0, 150, 151) + slots(1, 40, 41), dtype=torch.int32),
                          max_q=1, num_seqs=2)
    out = view.attend(attn, torch.stack([Q[0][150], Q[1][40]])[None], torch.stack([K[0][150], K[1][40]])[None],
                      torch.stack([V[0][150], V[1][40]])[None], attn_meta=meta)[0]
    assert torch.allclose(out[0], dense(0, 1, 151)[0], atol=2e-4, rtol=2e-4)
    assert torch.allclose(out[1], dense(1, 1, 41)[0], atol=2e-4, rtol=2e-4)
    # and the compressed result is close to exact attention (8 bits: nearly lossless)
    fine = TurboQuantPagedKVCache(1, 8, Hkv, D, TQ.TurboQuantConfig(bits=8), device="cpu")
    meta = PagedBatchMeta(cu_q=torch.tensor([0, 40], dtype=torch.int32), kv_lens=torch.tensor([40], dtype=torch.int32),
                          page_table=table[1:2], slot_mapping=torch.tensor(slots(1, 0, 40), dtype=torch.int32),
                          max_q=40, num_seqs=1)
    got = fine.view(0).attend(attn, Q[1][:40][None], K[1][:40][None], V[1][:40][None], attn_meta=meta)[0]
    kk = K[1][:40].repeat_interleave(Hq // Hkv, 1).permute(1, 0, 2)
    vv = V[1][:40].repeat_interleave(Hq // Hkv, 1).permute(1, 0, 2)
    s = (Q[1][:40].permute(1, 0, 2) @ kk.transpose(1, 2)) * attn.scale
    s = s.masked_fill(torch.triu(torch.ones(40, 40, dtype=torch.bool), 1), float("-inf"))
    exact = (s.softmax(-1) @ vv).permute(1, 0, 2)
    assert (got - exact).abs().max() < 0.08


def test_engine_serves_from_the_compressed_cache():
    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=512,
                      eos_token_id=255)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 250, (n,), generator=g).tolist() for n in (140, 9)]
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    plain = eSurge(model, max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64, num_pages=8)
    try:
        want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    finally:
        plain.close()
    eng = eSurge(model, max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64, num_pages=8,
                 kv_quantization=TQ.TurboQuantConfig(bits=8))
    try:
        assert isinstance(eng.cache, TurboQuantPagedKVCache) and not eng.runner.use_graphs
        got = [o.outputs[0].token_ids for o in eng.generate(prompts, sp)]
    finally:
        eng.close()
    assert all(len(t) == 8 for t in got)
    assert [t[0] for t in got] == [t[0] for t in want]        # 8 bits: the first tokens agree with the exact cache
    assert eng.cache.memory_bytes() < 0.7 * 2 * 2 * 8 * 128 * 2 * 16 * 4
