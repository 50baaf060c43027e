"""Serving paths beyond plain attention on the GPU: latent pages, recurrent-state pools, block-diagonal attention."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("family", ["deepseek_v3", "qwen3_next", "falcon_h1", "llama4_text"])
def test_engine_serves_family_in_bf16(family):
    import test_model_families_cpu as fam

    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge

    from easydel_b200.infra.factory import TaskType, registry

    extra = dict(fam.CASES[family])
    model_type = extra.pop("_type", family)
    base = extra.pop("_replace", None)
    cfg = registry.get_config(model_type)(**({**fam._COMMON, **extra} if base is None else base))
    torch.manual_seed(0)
    model = registry.get_module_registration(TaskType.CAUSAL_LM, model_type).module(
        cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16).cuda().eval()
    eng = eSurge(model, max_model_len=512, max_num_seqs=4, num_pages=16)
    prompts = [[5, 9, 2, 77, 31], list(range(3, 140)), [8, 1]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0))
    assert [len(o.outputs[0].token_ids) for o in outs] == [8, 8, 8]
    # the first sampled token follows the prompt exactly as in a dense forward pass (later ones may differ in bf16)
    for p, o in zip(prompts, outs):
        logits = model(input_ids=torch.tensor([p], device="cuda")).logits[0, -1].float()
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) > 0.05:
            assert o.outputs[0].token_ids[0] == int(logits.argmax())
    from easydel_b200.ops import _lib

    _lib.check_status(model.device)


def test_engine_serves_latent_attention_through_the_decode_kernel():
    """A DeepSeek-V3-shaped model with the 512 + 64 latent layout: decode steps run the latent decode kernel inside
    replayed CUDA graphs, and the tokens equal those of the same engine forced onto the gathered-pages path."""
    import os

    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge
    from easydel_b200.infra.factory import TaskType, registry
    from easydel_b200.ops import _lib, serving as S

    cfg = registry.get_config("deepseek_v3")(
        vocab_size=512, hidden_size=256, intermediate_size=512, moe_intermediate_size=128, num_hidden_layers=3,
        num_attention_heads=16, num_key_value_heads=16, n_shared_experts=1, n_routed_experts=8, kv_lora_rank=512,
        q_lora_rank=128, qk_rope_head_dim=64, v_head_dim=64, qk_nope_head_dim=64, num_experts_per_tok=2,
        first_k_dense_replace=1, max_position_embeddings=2048, n_group=1, topk_group=1)
    torch.manual_seed(0)
    model = registry.get_module_registration(TaskType.CAUSAL_LM, "deepseek_v3").module(
        cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16).cuda().eval()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (300, 17, 130)]
    sp = SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True)

    calls = {"n": 0}
    real = S.mla_decode_attention

    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    S.mla_decode_attention = counted
    try:
        eng = eSurge(model, max_model_len=1024, max_num_seqs=4, num_pages=24)
        assert eng.runner.use_graphs and eng.cache.latent and eng.cache.k.shape[-1] == 576
        got = [o.outputs[0].token_ids for o in eng.generate(prompts, sp)]
        assert calls["n"] > 0 and eng.runner.timings["graph_steps"] > 0
        eng.close()
    finally:
        S.mla_decode_attention = real
    # the same requests with the kernel switched off (gathered pages, batched matrix products, eager steps)
    supports = S.mla_decode_kernel_supports
    S.mla_decode_kernel_supports = lambda *a, **k: False
    os.environ["EDL_ESURGE_CUDA_GRAPHS"] = "0"
    try:
        eng = eSurge(model, max_model_len=1024, max_num_seqs=4, num_pages=24)
        ref = [o.outputs[0].token_ids for o in eng.generate(prompts, sp)]
        eng.close()
    finally:
        S.mla_decode_kernel_supports = supports
        os.environ.pop("EDL_ESURGE_CUDA_GRAPHS", None)
    same = sum(a == b for r, gt in zip(ref, got) for a, b in zip(r, gt))
    assert same >= 0.8 * sum(len(r) for r in ref), (ref, got)
    assert all(r[:3] == gt[:3] for r, gt in zip(ref, got)), (ref, got)
    _lib.check_status(model.device)
