"""Routing strategies, capacity and auxiliary losses of the mixture-of-experts block, against direct fp32 restatements."""

import pytest
import torch

from easydel_b200.layers.moe import (MoEBlock, MoeLoadBalancingStrategy as LB, MoeRoutingStrategy as RS, apply_capacity,
                                     load_balancing_loss_by_strategy, router_z_loss)


def _block(**kw):
    torch.manual_seed(0)
    return MoEBlock(16, 32, 4, 2, dtype=torch.float32, **kw)


def _dense_reference(block: MoEBlock, x2: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Every token through every chosen expert, one at a time."""
    out = torch.zeros_like(x2)
    gu, dn = block.gate_up_proj.weight, block.down_proj.weight
    for t in range(x2.shape[0]):
        for j in range(idx.shape[1]):
            if w[t, j] == 0:
                continue
            e = int(idx[t, j])
            h = x2[t] @ gu[e].t()
            g, u = h.chunk(2)
            out[t] += w[t, j] * ((torch.nn.functional.silu(g) * u) @ dn[e].t())
    return out


@pytest.mark.parametrize("strategy", [RS.TOP_K, RS.TOP_K_NDIV, RS.SWITCH, RS.EMPTY_CHOICE, RS.HASH])
def test_strategy_weights_and_output(strategy):
    m = _block(routing_strategy=strategy)
    x = torch.randn(2, 6, 16)
    y, logits = m(x)
    w, idx, probs = m.route(logits)
    T = 12
    assert w.shape == (T, 2) and idx.shape == (T, 2) and probs.shape == (T, 4)
    if strategy == RS.TOP_K:
        torch.testing.assert_close(w.sum(-1), torch.ones(T))
        assert torch.equal(idx, probs.topk(2, -1).indices)
    elif strategy == RS.TOP_K_NDIV:
        torch.testing.assert_close(w, probs.topk(2, -1).values)
    elif strategy == RS.SWITCH:
        assert torch.equal(idx[:, 0], probs.argmax(-1))
        assert torch.equal(w[:, 0], torch.ones(T)) and torch.equal(w[:, 1], torch.zeros(T))
    elif strategy == RS.HASH:
        assert torch.equal(idx, (torch.arange(T)[:, None] * 2 + torch.arange(2)[None]) % 4)
        torch.testing.assert_close(w, torch.full((T, 2), 0.5))
    else:   # expert choice: an expert never holds more than its capacity, and only tokens it ranked highest
        cap = T * 2 // 4
        loads = torch.bincount(idx[w > 0], minlength=4)
        assert int(loads.max()) <= cap
        chosen = probs.topk(cap, dim=0).indices
        for t in range(T):
            for j in range(2):
                if w[t, j] > 0:
                    assert t in chosen[:, idx[t, j]].tolist()
    ref = _dense_reference(m, x.reshape(-1, 16), w, idx)
    torch.testing.assert_close(y.reshape(-1, 16), ref, rtol=1e-4, atol=1e-5)


def test_capacity_drops_late_choices():
    idx = torch.tensor([[0, 1], [0, 1], [0, 2], [0, 3]])
    w = torch.full((4, 2), 0.5)
    w2, keep = apply_capacity(idx, w, 4, capacity=2)
    # expert 0 keeps tokens 0 and 1 (first choices, token order); expert 1 keeps both of its second choices
    assert keep.tolist() == [[True, True], [True, True], [False, True], [False, True]]
    assert torch.equal(w2, w * keep)
    m = _block(capacity_factor=0.5)
    wr, ir, _ = m.route(m.gate(torch.randn(12, 16)))
    assert int(torch.bincount(ir[wr > 0], minlength=4).max()) <= 3


def test_load_balancing_losses_match_formulas():
    torch.manual_seed(1)
    probs = torch.softmax(torch.randn(20, 4), -1)
    loads = torch.tensor([9.0, 3.0, 6.0, 2.0])
    E, k = 4, 1
    std = load_balancing_loss_by_strategy(probs, loads, E, k, LB.STANDARD, 0.1)
    torch.testing.assert_close(std, 0.1 * sum((loads[i] * E / k) * probs[:, i].mean() for i in range(E)))
    sw = load_balancing_loss_by_strategy(probs, loads, E, k, LB.SWITCH_TRANSFORMER, 0.1)
    torch.testing.assert_close(sw, 0.1 * E * sum((loads[i] / 20) * probs[:, i].mean() for i in range(E)))
    ec = load_balancing_loss_by_strategy(probs, loads, E, k, LB.EMPTY_CHOICE, 0.1)
    torch.testing.assert_close(ec, 0.1 * ((loads - loads.mean()) ** 2).mean())
    assert load_balancing_loss_by_strategy(probs, loads, E, k, LB.NONE, 0.1) is None
    assert load_balancing_loss_by_strategy(probs, loads, E, k, LB.STANDARD, None) is None
    with pytest.raises(ValueError):
        load_balancing_loss_by_strategy(probs, loads, E, k, "nope", 0.1)


def test_block_aux_losses_backpropagate_to_router():
    m = _block(lbl_coef=0.01, rzl_coef=0.001)
    x = torch.randn(1, 8, 16)
    _, logits = m(x)
    aux = m.last_aux_losses
    assert set(aux) == {"load_balancing_loss", "router_z_loss"}
    torch.testing.assert_close(aux["router_z_loss"], 0.001 * router_z_loss(logits))
    sum(aux.values()).backward()
    assert m.gate.weight.grad is not None and float(m.gate.weight.grad.abs().sum()) > 0


def test_model_adds_block_aux_losses_to_training_loss():
    from easydel_b200.infra.factory import TaskType, registry
    from easydel_b200.infra.loss_utils import LossConfig
    import easydel_b200.modules  # noqa: F401  (registers the families)

    def build(**kw):
        cfg = registry.get_config("qwen3_moe")(
            vocab_size=64, hidden_size=16, intermediate_size=32, moe_intermediate_size=16, num_hidden_layers=2,
            num_attention_heads=2, num_key_value_heads=1, head_dim=8, num_experts=4, num_experts_per_tok=2,
            max_position_embeddings=32, **kw)
        torch.manual_seed(0)
        return registry.get_module_registration(TaskType.CAUSAL_LM, "qwen3_moe").module(
            cfg, dtype=torch.float32, param_dtype=torch.float32)

    ids = torch.randint(0, 64, (2, 8))
    _, base = build().compute_loss(input_ids=ids, labels=ids, loss_config=LossConfig())
    _, m = build(moe_lbl_coef=0.05, moe_rzl_coef=0.01).compute_loss(input_ids=ids, labels=ids,
                                                                    loss_config=LossConfig())
    extra = m.other_metrics["load_balancing_loss"] + m.other_metrics["router_z_loss"]
    assert float(extra) > 0
    torch.testing.assert_close(m.loss.detach(), base.loss.detach() + extra, rtol=1e-5, atol=1e-6)
