"""eSurge on CPU: page pool / prefix cache, scheduler policy, and engine output equal to plain generate()."""

import pytest
import torch

from easydel_b200.inference import SamplingParams
from easydel_b200.inference.esurge import (EngineRequest, PagePool, Scheduler, SchedulerConfig, eSurge,
                                           hash_request_pages)
from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM


def _model():
    cfg = LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=2048, eos_token_id=199)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()


def test_page_pool_refcount_prefix_and_eviction():
    pool = PagePool(6, enable_caching=True)
    a = pool.allocate(3)
    assert 0 not in a and pool.num_free == 2
    hs = hash_request_pages(list(range(256)), 128)
    assert len(hs) == 2 and hs[0] != hs[1]
    assert hash_request_pages(list(range(256)), 128) == hs          # deterministic
    assert hash_request_pages([1] + list(range(1, 256)), 128)[1] != hs[1]  # chained on the prefix
    pool.register(a[0], hs[0])
    pool.register(a[1], hs[1])
    pool.release(a)
    assert pool.num_free == 5
    hit = pool.lookup(hs)
    assert hit == a[:2]
    pool.touch(hit)
    assert pool.num_free == 3 and pool.ref[a[0]] == 1
    pool.release(hit)
    got = pool.allocate(5)   # forces eviction of the cached pages
    assert set(got) == {1, 2, 3, 4, 5} and pool.lookup(hs) == []
    assert pool.stats.evictions >= 2


def test_scheduler_budget_chunking_and_preemption():
    pool = PagePool(8)  # 7 usable pages
    sch = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=1024), pool)
    r1 = EngineRequest("a", list(range(300)), SamplingParams(max_tokens=300, ignore_eos=True))
    r2 = EngineRequest("b", list(range(100)), SamplingParams(max_tokens=4, ignore_eos=True))
    sch.add_request(r1)
    sch.add_request(r2)
    o = sch.schedule()
    assert [(s.request.request_id, s.num_new_tokens) for s in o.scheduled] == [("a", 256)]   # budget-limited chunk
    sch.update_from_output(o, {})
    o = sch.schedule()
    got = {s.request.request_id: (s.num_new_tokens, s.samples) for s in o.scheduled}
    assert got == {"a": (44, True), "b": (100, True)}
    sch.update_from_output(o, {"a": 5, "b": 6})
    assert r1.output_token_ids == [5] and r2.output_token_ids == [6]
    o = sch.schedule()
    assert o.num_decode == 2 and o.total_tokens == 2
    # exhaust the pool: r1 grows until it needs a page nobody can give -> the newest request is preempted
    sch.update_from_output(o, {"a": 1, "b": 2})
    for _ in range(3000):
        o = sch.schedule()
        if o.preempted or not sch.has_unfinished():
            break
        sch.update_from_output(o, {s.request.request_id: 7 for s in o.scheduled if s.samples})
    assert r2.status.finished  # b only wanted 4 tokens
    assert pool.num_free >= 0


@pytest.mark.parametrize("async_scheduling", [False, True])
def test_engine_matches_generate_and_uses_prefix_cache(async_scheduling):
    model = _model()
    eng = eSurge(model, max_model_len=1024, max_num_seqs=8, max_num_batched_tokens=256, num_pages=32,
                 async_scheduling=async_scheduling)
    assert eng.async_scheduling == async_scheduling
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 198, (130,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 198, (n,), generator=g).tolist() for n in (5, 40, 300)]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    outs = eng.generate(prompts, sp)
    for p, o in zip(prompts, outs):
        ref = model.generate(torch.tensor([p]), max_new_tokens=12, eos_token_id=-1).sequences[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref, (len(p), o.outputs[0].token_ids, ref)
        assert o.finished and o.outputs[0].finish_reason == "length"
    # a second wave shares the first full page of the common prefix
    outs2 = eng.generate([shared + [3, 4, 5]], sp)
    assert outs2[0].num_cached_tokens == 128
    ref = model.generate(torch.tensor([shared + [3, 4, 5]]), max_new_tokens=12, eos_token_id=-1).sequences[0, 133:]
    assert outs2[0].outputs[0].token_ids == ref.tolist()
    m = eng.get_metrics_summary()
    assert m["requests_completed"] == 4 and m["tokens_generated"] == 48 and m["prefix_cache_hit_rate"] > 0


def test_engine_background_thread_stream_and_abort():
    model = _model()
    eng = eSurge(model, max_model_len=512, max_num_seqs=4, num_pages=16).initiate()
    try:
        chunks = list(eng.stream(list(range(1, 20)), SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)))
        assert chunks[-1].finished and chunks[-1].num_generated_tokens == 6
        assert sum(len(c.delta_token_ids) for c in chunks) == 6
        rid = eng.add_request(list(range(1, 30)), SamplingParams(max_tokens=400, ignore_eos=True))
        eng.abort_request(rid)
        assert eng._tracked[rid].finished
    finally:
        eng.terminate()


def test_sampling_with_seed_is_reproducible():
    model = _model()
    eng = eSurge(model, max_model_len=256, max_num_seqs=4, num_pages=8)
    sp = SamplingParams(max_tokens=8, temperature=0.9, top_k=20, top_p=0.95, seed=123, ignore_eos=True,
                        repetition_penalty=1.2)
    a = eng.generate([list(range(1, 10))], sp)[0].outputs[0].token_ids
    b = eng.generate([list(range(1, 10))], sp)[0].outputs[0].token_ids
    assert a == b and len(a) == 8


def test_engine_profiling_and_monitoring_hooks(tmp_path):
    eng = eSurge(_model(), max_model_len=128, max_num_seqs=2, num_pages=8)
    eng.start_profiling(str(tmp_path))
    eng.generate([1, 2, 3], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    path = eng.stop_profiling()
    assert path and path.endswith(".json") and (tmp_path / path.split("/")[-1]).exists()
    assert eng.stop_profiling() is None
    info = eng.start_monitoring(prometheus_port=0)
    assert "prometheus" in info
    eng.stop_monitoring()


def test_latent_attention_models_are_served_from_latent_pages():
    """DeepSeek-style latent attention: the paged cache holds one compressed row per token and the engine's greedy
    continuations equal ``model.generate`` for prompts of different lengths scheduled together."""
    from easydel_b200.infra.factory import TaskType, registry

    torch.manual_seed(0)
    cfg = registry.get_config("deepseek_v3")(
        vocab_size=128, hidden_size=48, intermediate_size=64, moe_intermediate_size=32, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=8,
        qk_rope_head_dim=8, v_head_dim=8, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2, n_group=2,
        topk_group=1, first_k_dense_replace=1, max_position_embeddings=512)
    model = registry.get_module_registration(TaskType.CAUSAL_LM, "deepseek_v3").module(cfg, dtype=torch.float32).eval()
    eng = eSurge(model, max_model_len=256, max_num_seqs=4, num_pages=8)
    assert eng.runner.cache.latent and eng.runner.cache.k.shape[-2:] == (1, 24)
    assert eng.runner.cache.v is eng.runner.cache.k
    prompts = [[5, 9, 2, 77, 31], list(range(3, 40)), [1, 2]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for p, o in zip(prompts, outs):
        want = model.generate(torch.tensor([p]), max_new_tokens=6).sequences[0, len(p):].tolist()
        assert o.outputs[0].token_ids == want


@pytest.mark.parametrize("family", ["qwen3_next", "falcon_h1", "minimax", "llama4_text"])
def test_hybrid_recurrent_models_are_served_with_per_slot_states(family):
    """Linear-attention / state-space layers keep one state row per engine slot; a ragged step gathers the rows of
    the scheduled sequences, the layer walks the sequence bounds, and the rows are scattered back."""
    import test_model_families_cpu as fam

    torch.manual_seed(0)
    model = fam._build(family, fam.CASES[family])
    model = (model[0] if isinstance(model, tuple) else model).eval()
    eng = eSurge(model, max_model_len=256, max_num_seqs=4, num_pages=8)
    if family != "llama4_text":     # (Llama-4 is here for its block-diagonal attention over the pages)
        assert eng.cache.linear and not eng.pool.enable_caching
    prompts = [[5, 9, 2, 77, 31], list(range(3, 40)), [8, 1]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=5, temperature=0.0))
    for p, o in zip(prompts, outs):
        want = model.generate(torch.tensor([p]), max_new_tokens=5).sequences[0, len(p):].tolist()
        assert o.outputs[0].token_ids == want
    # a slot taken by a new request starts from a zero state
    again = eng.generate([prompts[1]], SamplingParams(max_tokens=5, temperature=0.0))[0]
    assert again.outputs[0].token_ids == outs[1].outputs[0].token_ids


def test_async_scheduling_eos_stop_preemption_and_unknown_options():
    """Step t+1 is launched before step t's tokens are read: a request that stops on a token (not on its length)
    has one row too many in flight, whose result must be dropped; preempted requests keep the token sampled
    before the preemption; outputs equal the synchronous engine's."""
    model = _model()
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 198, (n,), generator=g).tolist() for n in (7, 150, 33, 260, 90)]
    sync = eSurge(model, max_model_len=512, max_num_seqs=4, max_num_batched_tokens=128, num_pages=12,
                  async_scheduling=False)
    ref = sync.generate(prompts, SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True))
    # stop on the 5th token of the longest-running request: a token-triggered stop
    stop_tok = ref[0].outputs[0].token_ids[4]
    sp = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True, stop_token_ids=[stop_tok])
    want = eSurge(model, max_model_len=512, max_num_seqs=4, max_num_batched_tokens=128, num_pages=12,
                  async_scheduling=False).generate(prompts, sp)
    eng = eSurge(model, max_model_len=512, max_num_seqs=4, max_num_batched_tokens=128, num_pages=12,
                 async_scheduling=True)
    got = eng.generate(prompts, sp)
    for a, b in zip(got, want):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
        assert a.outputs[0].finish_reason == b.outputs[0].finish_reason
    assert got[0].outputs[0].finish_reason == "stop" and len(got[0].outputs[0].token_ids) <= 5
    assert eng._inflight is None and not eng.scheduler.has_unfinished()
    assert eng.pool.num_free == eng.pool.num_pages - 1 or eng.pool.num_free > 0
    with pytest.raises(TypeError):
        eSurge(model, max_model_len=64, max_num_seqs=2, num_pages=4, overlap_executon=True)   # misspelt
    eSurge(model, max_model_len=64, max_num_seqs=2, num_pages=4, compile_runner=True)         # reference AOT knob
