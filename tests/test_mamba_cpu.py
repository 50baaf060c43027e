"""Mamba-1, Falcon-Mamba and Mamba-2 against Hugging Face on CPU, plus incremental decoding with the state cache."""

import pytest
import torch
import transformers

from easydel_b200.modules.mamba import (FalconMambaConfig, FalconMambaForCausalLM, Mamba2Config, Mamba2ForCausalLM,
                                        MambaConfig, MambaForCausalLM)

CASES = {
    "mamba": (MambaConfig, MambaForCausalLM, dict(vocab_size=128, hidden_size=32, state_size=8, num_hidden_layers=2)),
    "falcon_mamba": (FalconMambaConfig, FalconMambaForCausalLM,
                     dict(vocab_size=128, hidden_size=32, state_size=8, num_hidden_layers=2)),
    "mamba2": (Mamba2Config, Mamba2ForCausalLM,
               dict(vocab_size=128, hidden_size=32, state_size=16, num_hidden_layers=2, num_heads=8, head_dim=8,
                    n_groups=2, expand=2)),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_matches_hf_and_decodes_incrementally(name):
    cfg_cls, cls, kw = CASES[name]
    cfg = cfg_cls(**kw)
    torch.manual_seed(0)
    model = cls(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf_cfg = transformers.CONFIG_MAPPING[name](**kw, tie_word_embeddings=cfg.tie_word_embeddings)
    hf = transformers.AutoModelForCausalLM.from_config(hf_cfg).float().eval()
    missing, unexpected = hf.load_state_dict(model.state_dict(), strict=False)
    assert not unexpected and all("lm_head" in m for m in missing), (missing, unexpected)
    ids = torch.randint(0, 128, (2, 14))
    with torch.no_grad():
        ours, theirs = model(input_ids=ids).logits, hf(input_ids=ids).logits
    assert (ours - theirs).abs().max() < 2e-4
    cache = model.init_cache(2)
    with torch.no_grad():
        parts = [model(input_ids=ids[:, :9], past_key_values=cache).logits]
        parts += [model(input_ids=ids[:, t:t + 1], past_key_values=cache).logits for t in range(9, 14)]
    assert (torch.cat(parts, 1) - ours).abs().max() < 2e-4
    _, m = model.compute_loss(input_ids=ids, labels=ids)
    m.loss.backward()
    assert all(p.grad is not None or getattr(p, "main_grad", None) is not None for p in model.parameters())
