"""eSurge on the GPU kernels: paged path agrees with the dense path; mixed batches run; metrics are sane."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(layers=2):
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=layers,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      eos_token_id=4095, initializer_range=0.08)
    return LlamaForCausalLM.sequential_init(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16, device="cuda",
                                            seed=3).eval()


def test_paged_forward_matches_dense_forward_logits():
    """Same tokens through the paged engine step and through a plain forward: last-position logits agree."""
    from easydel_b200.caching.paged import PagedBatchMeta, PagedKVCache

    model = _model()
    lens = [300, 5, 129]
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, 4000, (n,), generator=g) for n in lens]
    cache = PagedKVCache.init_for_model(model, num_pages=16)
    ids = torch.cat(seqs).cuda()
    pos = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    cu = torch.tensor([0, 300, 305, 434], dtype=torch.int32).cuda()
    pages = [[1, 2, 3], [4], [5, 6]]
    table = torch.zeros(3, 4, dtype=torch.int32)
    slots = []
    for b, n in enumerate(lens):
        table[b, :len(pages[b])] = torch.tensor(pages[b])
        slots += [pages[b][i // 128] * 128 + i % 128 for i in range(n)]
    meta = PagedBatchMeta(cu_q=cu, kv_lens=torch.tensor(lens, dtype=torch.int32).cuda(), page_table=table.cuda(),
                          slot_mapping=torch.tensor(slots, dtype=torch.int32).cuda(), max_q=300, num_seqs=3)
    with torch.no_grad():
        h = model(input_ids=ids[None], position_ids=pos[None], past_key_values=cache, cache_metadata=meta,
                  apply_lm_head=False).last_hidden_state[0]
        for b, n in enumerate(lens):
            ref = model(input_ids=seqs[b][None].cuda(), apply_lm_head=False).last_hidden_state[0, -1]
            got = h[int(cu[b + 1]) - 1]
            assert torch.allclose(got.float(), ref.float(), atol=6e-2, rtol=5e-2), b


def test_engine_runs_mixed_batches_and_prefix_cache():
    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge

    model = _model()
    eng = eSurge(model, max_model_len=2048, max_num_seqs=16, max_num_batched_tokens=512, num_pages=64)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 4000, (256,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 4000, (n,), generator=g).tolist() for n in (3, 50, 700, 17)]
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    outs = eng.generate(prompts, sp)
    assert all(len(o.outputs[0].token_ids) == 24 for o in outs)
    # greedy decoding through the dense cache gives (nearly) the same continuation
    ref = model.generate(torch.tensor([prompts[1]]).cuda(), max_new_tokens=24, eos_token_id=-1).sequences[0, len(prompts[1]):]
    got = outs[1].outputs[0].token_ids
    assert got[:2] == ref[:2].tolist()
    again = eng.generate([shared + [1, 2, 3]], sp)[0]
    assert again.num_cached_tokens == 256
    # sampling rows with penalties go through the sampler kernel
    sp2 = SamplingParams(max_tokens=8, temperature=0.8, top_k=40, top_p=0.9, seed=5, presence_penalty=0.5,
                         ignore_eos=True)
    a = eng.generate([prompts[0]], sp2)[0].outputs[0].token_ids
    b = eng.generate([prompts[0]], sp2)[0].outputs[0].token_ids
    assert a == b and len(a) == 8
    m = eng.get_metrics_summary()
    assert m["requests_completed"] == 7 and m["ttft_p50"] is not None


def test_preemption_chunked_prefix_hit_and_bucket_padding_on_the_gpu():
    """Three scheduler situations on the kernels: (a) a page pool too small for all requests, so that the newest is
    preempted and recomputed; (b) a prompt that hits the prefix cache and is then prefilled in chunks smaller than
    the rest of it; (c) three decode rows replayed from the four-row graph bucket (one padding row). In each, greedy
    continuations must agree with the same request served alone by a roomy engine (first tokens exactly; later
    ones may flip on bf16 near-ties, so agreement of most positions is asked for)."""
    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge

    model = _model()
    g = torch.Generator().manual_seed(11)
    shared = torch.randint(0, 4000, (384,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 4000, (n,), generator=g).tolist() for n in (116, 121, 126)]   # 500, 505, 510 tokens
    sp = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)

    def alone(prompt):
        eng = eSurge(model, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=1024, num_pages=32,
                     enable_prefix_caching=False)
        try:
            return eng.generate([prompt], sp)[0].outputs[0].token_ids
        finally:
            eng.close()

    want = [alone(p) for p in prompts]

    def agree(a, b):
        assert len(a) == len(b) == 40 and a[:2] == b[:2], (a[:4], b[:4])
        assert sum(x == y for x, y in zip(a, b)) >= 30 or a[:8] == b[:8]

    # (a) all three fit at admission (4 pages of 128 tokens each, 13 usable pages) and each crosses into a fifth page
    # while decoding, which the pool cannot give to all of them
    tight = eSurge(model, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=1024, num_pages=14,
                   enable_prefix_caching=False)
    try:
        outs = tight.generate(prompts, sp)
        assert tight.scheduler.num_preemptions >= 1
        for o, w in zip(outs, want):
            agree(o.outputs[0].token_ids, w)
    finally:
        tight.close()
    # (b) prefix hit of three pages, then the rest of the prompt in chunks of 64 tokens; (c) three rows -> bucket 4
    eng = eSurge(model, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=64, num_pages=48)
    try:
        first = eng.generate([prompts[0]], sp)[0]
        agree(first.outputs[0].token_ids, want[0])
        hit = eng.generate([prompts[1]], sp)[0]
        assert hit.num_cached_tokens == 384
        agree(hit.outputs[0].token_ids, want[1])
        outs = eng.generate(prompts, sp)
        assert eng.runner.timings["graph_steps"] > 0 and 4 in eng.runner._graphs
        for o, w in zip(outs, want):
            agree(o.outputs[0].token_ids, w)
    finally:
        eng.close()


def test_engine_on_the_compressed_cache_on_the_gpu():
    """The TurboQuant page pools and their tensor-code attention with CUDA tensors (eager steps): 8-bit codes keep the
    first greedy tokens of the exact cache."""
    from easydel_b200.caching.turboquant_paged import TurboQuantPagedKVCache
    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge
    from easydel_b200.layers.turboquant import TurboQuantConfig

    model = _model()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 4000, (n,), generator=g).tolist() for n in (200, 33)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    plain = eSurge(model, max_model_len=512, max_num_seqs=2, max_num_batched_tokens=256, num_pages=16)
    try:
        want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    finally:
        plain.close()
    eng = eSurge(model, max_model_len=512, max_num_seqs=2, max_num_batched_tokens=256, num_pages=16,
                 kv_quantization=TurboQuantConfig(bits=8))
    try:
        assert isinstance(eng.cache, TurboQuantPagedKVCache) and eng.cache.k_codes.is_cuda
        got = [o.outputs[0].token_ids for o in eng.generate(prompts, sp)]
    finally:
        eng.close()
    # random bf16 weights put many logits within the quantisation noise of one another: only the short prompt's
    # first token is required to agree
    assert all(len(t) == 6 for t in got) and got[1][0] == want[1][0]
    # the cache's own arithmetic on the GPU equals the same arithmetic on the CPU
    import types

    from easydel_b200.caching.paged import PagedBatchMeta

    torch.manual_seed(0)
    attn = types.SimpleNamespace(scale=128 ** -0.5, softcap=None, sliding_window=None, sinks=None)
    q, k, v = torch.randn(1, 70, 8, 128), torch.randn(1, 70, 2, 128), torch.randn(1, 70, 2, 128)
    outs = []
    for dev in ("cpu", "cuda"):
        cache = TurboQuantPagedKVCache(1, 4, 2, 128, TurboQuantConfig(bits=4), device=dev)
        meta = PagedBatchMeta(cu_q=torch.tensor([0, 70], dtype=torch.int32, device=dev),
                              kv_lens=torch.tensor([70], dtype=torch.int32, device=dev),
                              page_table=torch.tensor([[1, 0]], dtype=torch.int32, device=dev),
                              slot_mapping=(128 + torch.arange(70, dtype=torch.int32)).to(dev), max_q=70, num_seqs=1)
        outs.append(cache.view(0).attend(attn, q.to(dev), k.to(dev), v.to(dev), attn_meta=meta).cpu())
    assert torch.allclose(outs[0], outs[1], atol=2e-3, rtol=2e-3)
