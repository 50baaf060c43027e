"""Tiny Llama on CPU in fp32: logits / loss parity with Hugging Face and a 10-step AdamW trajectory.

Architecture and hyper-parameters: vocab 1024, hidden 256, 4 layers, 8 query / 4 KV heads
(head_dim 32), SwiGLU 688, RMSNorm eps 1e-6, RoPE theta 10000, untied embeddings, batch 4 x 128,
AdamW lr 1e-4, betas (0.9, 0.95), weight decay 0.01.
"""

import copy

import pytest
import torch

from easydel_b200.infra.base_state import EasyDeLState
from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
from easydel_b200.utils.parameters_transformation import ModelConverter, internal_to_hf


def _tiny():
    cfg = LlamaConfig(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                      num_attention_heads=8, num_key_value_heads=4, rms_norm_eps=1e-6, rope_theta=10000.0,
                      max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)


def test_logits_and_loss_match_hf():
    model = _tiny()
    hf = ModelConverter.easydel_to_huggingface(model, dtype=torch.float32)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1024, (4, 128), generator=g)
    with torch.no_grad():
        ours = model(input_ids=ids).logits
        theirs = hf(input_ids=ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4, rtol=1e-4), (ours - theirs).abs().max()
    _, met = model.compute_loss(input_ids=ids, labels=ids)
    ref = hf(input_ids=ids, labels=ids).loss
    assert abs(met.loss.item() - ref.item()) < 1e-4


def test_ten_step_adamw_trajectory_matches_hf():
    model = _tiny()
    hf = ModelConverter.easydel_to_huggingface(model, dtype=torch.float32)
    opt_hf = torch.optim.AdamW(hf.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01, eps=1e-8)
    tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-4), weight_decay=0.01, b1=0.9,
                                    b2=0.95, eps=1e-8)
    state = EasyDeLState.create(model=model, tx=tx, init_opt_state=True)
    g = torch.Generator().manual_seed(2)
    ours, theirs = [], []
    for _ in range(10):
        ids = torch.randint(0, 1024, (4, 128), generator=g)
        _, met = model.compute_loss(input_ids=ids, labels=ids)
        met.loss.backward()
        state.apply_gradients()
        ours.append(met.loss.item())
        opt_hf.zero_grad()
        l = hf(input_ids=ids, labels=ids).loss
        l.backward()
        opt_hf.step()
        theirs.append(l.item())
    assert max(abs(a - b) for a, b in zip(ours, theirs)) < 2e-4, (ours, theirs)
    # weights agree after training
    sd = internal_to_hf(model)
    for k, v in hf.state_dict().items():
        if k in sd:
            assert torch.allclose(sd[k], v, atol=1e-4), k


def test_gradient_accumulation_equivalence():
    """Two micro-batches scaled by 1/2 accumulate the same gradient as the full batch."""
    torch.manual_seed(3)
    ids = torch.randint(0, 1024, (4, 64))
    m1, m2 = _tiny(), _tiny()
    tx1, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-3), weight_decay=0.0)
    tx2, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-3), weight_decay=0.0)
    s1 = EasyDeLState.create(model=m1, tx=tx1, init_opt_state=True)
    s2 = EasyDeLState.create(model=m2, tx=tx2, init_opt_state=True)
    _, met = m1.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    s1.flat.fold_param_grads()
    for i in range(2):
        _, met = m2.compute_loss(input_ids=ids[2 * i:2 * i + 2], labels=ids[2 * i:2 * i + 2], loss_scale=0.5)
        met.loss.backward()
    s2.flat.fold_param_grads()
    assert torch.allclose(s1.flat.grad, s2.flat.grad, atol=1e-6, rtol=1e-4)
    assert s1.flat.grad.abs().max() > 0
