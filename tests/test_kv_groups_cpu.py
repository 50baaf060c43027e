"""Cache groups: specs and memory planning, window-bounded page managers, prefix hits across groups, and an engine
whose sliding-window layers hold a bounded number of pages while the output still equals plain generate()."""

import pytest
import torch

from easydel_b200.caching import specs as SP
from easydel_b200.inference import SamplingParams
from easydel_b200.inference.esurge import EngineRequest, eSurge, hash_request_pages
from easydel_b200.inference.esurge.kv_manager import GroupManager, KVCacheCoordinator
from easydel_b200.inference.esurge.page_pool import NULL_PAGE


def _gemma3(window=64, layers=4, pattern=2):
    from easydel_b200.infra.factory import TaskType, registry
    import easydel_b200.modules  # noqa: F401

    cfg = registry.get_config("gemma3_text")(
        vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=layers, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=2048, sliding_window=window,
        query_pre_attn_scalar=16, sliding_window_pattern=pattern, eos_token_id=199)
    torch.manual_seed(0)
    return registry.get_module_registration(TaskType.CAUSAL_LM, "gemma3_text").module(
        cfg, dtype=torch.float32, param_dtype=torch.float32).eval()


def test_specs_page_math():
    full = SP.FullAttentionSpec(num_kv_heads=8, head_dim=128)
    assert full.page_size_bytes == 2 * 128 * 8 * 128 * 2
    assert full.pages_per_sequence(8192) == 64 and full.first_useful_token(5000) == 0
    sw = SP.SlidingWindowSpec(num_kv_heads=8, head_dim=128, sliding_window=1024)
    assert sw.first_useful_token(100) == 0 and sw.first_useful_token(5000) == 5000 - 1024 + 1
    assert sw.pages_per_sequence(8192) == 9 and sw.pages_per_sequence(512) == 4
    assert sw.max_memory_usage_bytes(8192) == 9 * sw.page_size_bytes
    ch = SP.ChunkedLocalAttentionSpec(num_kv_heads=8, head_dim=128, attention_chunk_size=2048)
    assert ch.first_useful_token(2047) == 0 and ch.first_useful_token(2048) == 2048 and ch.first_useful_token(5000) == 4096
    mla = SP.MLAAttentionSpec(num_kv_heads=1, head_dim=576)
    assert mla.page_size_bytes == 128 * 576 * 2
    assert SP.MambaSpec(state_elements=1000).pages_per_sequence(8192) == 1


def test_groups_from_model_and_plan():
    model = _gemma3(window=64, layers=4, pattern=2)
    groups = SP.build_groups(model, element_size=4)
    assert [g.kind for g in groups] == ["full", "sliding"]
    assert groups[0].layers == [1, 3] and groups[1].layers == [0, 2] and groups[1].window == 64
    counts = SP.plan_pages(groups, budget_bytes=64 << 20, max_num_seqs=8, max_model_len=2048,
                           max_num_batched_tokens=256)
    per_seq = groups[1].spec.pages_per_sequence(2048)
    assert per_seq == 2
    assert 8 * per_seq <= counts[1] <= 2 * (8 * per_seq + 3) + 2          # bounded by the window, not the length
    assert counts[0] == min(8 * 16 + 1, (64 << 20 - 0) // groups[0].bytes_per_page) or counts[0] <= 8 * 16 + 1
    assert counts[0] > counts[1]


def test_sliding_and_chunked_managers_release_out_of_window_pages():
    m = GroupManager(SP.SlidingWindowSpec(sliding_window=200), num_pages=32)
    pages = m.pool.allocate(6)            # 768 tokens
    orig = list(pages)
    assert m.remove_skipped(pages, 200) == 0
    # 700 tokens computed: the next query (position 700) reads keys > 500 -> first useful 501 -> pages 0..2 go
    assert m.remove_skipped(pages, 700) == 3
    assert pages[:3] == [NULL_PAGE] * 3 and pages[3:] == orig[3:]
    assert m.remove_skipped(pages, 700) == 0 and m.pool.num_free == 31 - 3
    # after the pages that were never used, the oldest released page is the first to be reused
    m.pool.allocate(25)
    assert m.pool.allocate(1) == [orig[0]]
    c = GroupManager(SP.ChunkedLocalAttentionSpec(attention_chunk_size=256), num_pages=16)
    pages = c.pool.allocate(5)
    assert c.remove_skipped(pages, 255) == 0
    assert c.remove_skipped(pages, 256) == 2 and c.remove_skipped(pages, 600) == 2
    assert pages[:4] == [NULL_PAGE] * 4 and pages[4] != NULL_PAGE
    f = GroupManager(SP.FullAttentionSpec(), num_pages=8)
    pages = f.pool.allocate(3)
    assert f.remove_skipped(pages, 10_000) == 0


def test_prefix_hit_needs_window_pages_in_bounded_groups():
    groups = [SP.KVCacheGroup(SP.FullAttentionSpec(), [1], 16), SP.KVCacheGroup(SP.SlidingWindowSpec(sliding_window=100), [0], 16)]
    kv = KVCacheCoordinator(groups)
    toks = list(range(700))
    hs = hash_request_pages(toks, 128)           # 5 full pages
    a = EngineRequest("a", toks, SamplingParams(max_tokens=4))
    assert kv.try_allocate(a, 700)
    assert len(a.pages) == 6 and len(a.group_pages[0]) == 6
    for i, h in enumerate(hs):
        kv.register(a, i, h)
    a.num_computed_tokens = 700
    assert kv.remove_skipped(a) == 4             # sliding group: first useful token 601 -> pages 0..3
    assert kv.pages_held(a) == [6, 2]
    kv.release(a)
    # every page is still findable: a full 5-page hit needs sliding pages [4] only (window reaches back to 541)
    b = EngineRequest("b", toks, SamplingParams(max_tokens=4))
    assert kv.admit_with_prefix(b, hs) == 5
    assert b.group_pages[0][:4] == [NULL_PAGE] * 4 and b.group_pages[0][4] != NULL_PAGE and len(b.pages) == 5
    kv.release(b)
    # the sliding group loses page 4 to another request: the hit shrinks to the longest prefix whose window pages
    # are still there (4 pages = 512 tokens, window reaches back to 413 -> sliding page 3)
    sl = kv.managers[1].pool
    victim = sl.cached.pop(hs[4])
    sl.page_hash[victim] = None
    c = EngineRequest("c", toks, SamplingParams(max_tokens=4))
    assert kv.admit_with_prefix(c, hs) == 4
    assert c.group_pages[0][:3] == [NULL_PAGE] * 3 and c.group_pages[0][3] != NULL_PAGE and len(c.pages) == 4
    kv.release(c)
    d = EngineRequest("d", list(range(1, 300)), SamplingParams(max_tokens=4))
    assert kv.admit_with_prefix(d, hash_request_pages(d.prompt_token_ids, 128)) == 0 and d.pages == []
    for m in kv.managers:
        assert m.pool.num_free == 15


@pytest.mark.parametrize("async_scheduling", [False, True])
def test_engine_sliding_layers_hold_bounded_pages_and_match_generate(async_scheduling):
    model = _gemma3(window=64, layers=4, pattern=2)
    eng = eSurge(model, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=160, num_pages=24,
                 async_scheduling=async_scheduling)
    assert eng.cache.num_groups == 2 and [g.kind for g in eng.cache.groups] == ["full", "sliding"]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 198, (n,), generator=g).tolist() for n in (300, 45)]
    sp = SamplingParams(max_tokens=120, temperature=0.0, ignore_eos=True)
    held = []
    rids = [eng.add_request(p, sp) for p in prompts]
    while eng.scheduler.has_unfinished() or getattr(eng, "_inflight", None) is not None:
        eng.step()
        for r in eng.scheduler.running:
            held.append((r.num_computed_tokens, *eng.kv.pages_held(r)))
    longest = max(held)
    assert longest[0] >= 400 and longest[1] == 4          # full-attention group: every page of 419 tokens
    assert max(h[2] for h in held) <= 3                   # sliding group: window 64 + a 160-token step, never more
    assert all(h[2] <= 2 for h in held if h[0] > 300)     # while decoding: the window's pages only
    for rid, p in zip(rids, prompts):
        out = eng._tracked[rid].req.output_token_ids
        ref = model.generate(torch.tensor([p]), max_new_tokens=120, eos_token_id=-1).sequences[0, len(p):].tolist()
        assert out == ref
    for m in eng.kv.managers:
        assert m.pool.num_free == m.pool.num_pages - 1    # everything was given back


def test_data_parallel_router_keeps_pages_local_and_follows_cached_prefixes():
    """Two engine replicas behind the data-parallel front: requests spread by load, a request whose prompt shares a
    cached prefix goes to the replica that holds those pages, outputs equal plain generate()."""
    from easydel_b200.inference.esurge.dp_router import DataParallelEngine, pages_per_dp_shard
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    assert pages_per_dp_shard(64, 4) == 16 and pages_per_dp_shard(5, 4) is None
    cfg = LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024, eos_token_id=199)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    engines = [eSurge(model, max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=256, num_pages=16)
               for _ in range(2)]
    dp = DataParallelEngine(engines)
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(0, 198, (260,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    first = [shared + [1, 2, 3], torch.randint(0, 198, (40,), generator=g).tolist()]
    rids = [dp.add_request(p, sp) for p in first]
    assert {dp.shard_of(r) for r in rids} == {0, 1}               # spread by load
    while dp.has_unfinished():
        dp.step()
    home = dp.shard_of(rids[0])
    # the same 256-token prefix again: routed to the replica that cached it, and served from its pages
    out = dp.generate([shared + [9, 8, 7, 6]], sp)[0]
    rid = max(dp.owner, key=lambda r: int(r.split("-")[1]))
    assert dp.shard_of(rid) == home and out.num_cached_tokens == 256
    ref = model.generate(torch.tensor([shared + [9, 8, 7, 6]]), max_new_tokens=6, eos_token_id=-1).sequences[0, 264:]
    assert out.outputs[0].token_ids == ref.tolist()
    m = dp.get_metrics_summary()
    assert m["replicas"] == 2 and sum(m["requests_routed"]) == 3 and m["requests_completed"] == 3
    for e in engines:
        assert e.pool.num_free == e.pool.num_pages - 1
    dp.close()
