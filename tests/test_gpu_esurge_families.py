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
