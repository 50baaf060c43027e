"""RWKV-4 against Hugging Face on CPU: logits, training step, incremental decoding with the recurrent state."""

import torch
import transformers

from easydel_b200.modules.rwkv import RwkvConfig, RwkvForCausalLM
from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

KW = dict(vocab_size=128, hidden_size=32, num_hidden_layers=3, attention_hidden_size=32, intermediate_size=64,
          context_length=64)


def test_rwkv_matches_hf_trains_and_decodes():
    torch.manual_seed(0)
    m = RwkvForCausalLM(RwkvConfig(**KW), dtype=torch.float32, param_dtype=torch.float32).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() != 2:
                p.add_(torch.randn_like(p) * 0.3)
    hf = transformers.RwkvForCausalLM(transformers.RwkvConfig(**KW)).float().eval()
    missing, unexpected = hf.load_state_dict(internal_to_hf(m), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    ids = torch.randint(0, 128, (2, 20))
    with torch.no_grad():
        a, b = m(input_ids=ids).logits, hf(input_ids=ids).logits
    assert (a - b).abs().max() < 2e-4, (a - b).abs().max()
    back = hf_to_internal(m, hf.state_dict())
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.rwkv.blocks[1].attention.time_decay.grad.abs().sum() > 0
    st = m.init_cache(2)
    with torch.no_grad():
        o1 = m(input_ids=ids[:, :13], past_key_values=st).logits
        assert (o1 - a[:, :13]).abs().max() < 2e-4
        for t in range(13, 20):
            o = m(input_ids=ids[:, t:t + 1], past_key_values=st).logits
            assert (o[:, 0] - a[:, t]).abs().max() < 2e-4, t
