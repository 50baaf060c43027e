"""Functional cross-entropy variants and loss strategies against torch.nn.functional and each other."""

import torch
import torch.nn.functional as tF

from easydel_b200.infra import loss_utils as L


def _data(B=3, T=10, V=37, seed=0):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, T, V, generator=g) * 2
    labels = torch.randint(0, V, (B, T), generator=g)
    return logits, labels


def test_weighted_cross_entropy_matches_torch():
    logits, labels = _data()
    w = (torch.rand(3, 10) > 0.3).float()
    total, z, ws = L.compute_weighted_cross_entropy(logits, labels, w)
    ref = (tF.cross_entropy(logits.reshape(-1, 37), labels.reshape(-1), reduction="none") * w.reshape(-1)).sum()
    assert torch.allclose(total, ref, atol=1e-4) and float(z) == 0.0 and float(ws) == float(w.sum())
    # smoothing: a perfect (very confident) prediction of the smoothed target still scores ~ the KL to it, >= 0
    total_s, _, _ = L.compute_weighted_cross_entropy(logits, labels, w, label_smoothing=0.1)
    kl = tF.cross_entropy(logits.reshape(-1, 37), labels.reshape(-1), reduction="none", label_smoothing=0.0)
    assert float(total_s) > 0 and kl.numel() == 30
    # z-loss term and the normalising factor
    t2, z2, _ = L.compute_weighted_cross_entropy(logits, labels, w, z_loss=1e-3, loss_normalizing_factor=5.0)
    lse = torch.logsumexp(logits, -1)
    assert torch.allclose(z2, (1e-3 * lse.pow(2) * w).sum() / 5.0, atol=1e-5)
    assert torch.allclose(t2, (ref + (1e-3 * lse.pow(2) * w).sum()) / 5.0, atol=1e-4)
    _, _, _, acc = L.compute_weighted_cross_entropy_and_accuracy(logits, labels, w)
    assert torch.allclose(acc, ((logits.argmax(-1) == labels).float() * w).sum() / w.sum())


def test_simple_and_dynamic_variants():
    logits, labels = _data(seed=1)
    valid = torch.rand(3, 10) > 0.2
    loss, acc = L.cross_entropy_loss_and_accuracy(logits, labels, valid)
    lab = torch.where(valid, labels, torch.full_like(labels, -100))
    assert torch.allclose(loss, tF.cross_entropy(logits.reshape(-1, 37), lab.reshape(-1)), atol=1e-5)
    for red in ("mean", "sum", "none"):
        got, _ = L.dynamic_cross_entropy_loss(logits, lab, reduction=red, label_smoothing=0.1)
        ref = tF.cross_entropy(logits.reshape(-1, 37), lab.reshape(-1), reduction=red, label_smoothing=0.1)
        assert torch.allclose(got.reshape(ref.shape), ref, atol=1e-4), red
    cw = torch.rand(37) + 0.5
    got, _ = L.dynamic_cross_entropy_loss(logits, lab, weight=cw)
    assert torch.allclose(got, tF.cross_entropy(logits.reshape(-1, 37), lab.reshape(-1), weight=cw), atol=1e-4)
    x, z = torch.randn(4, 6), (torch.rand(4, 6) > 0.5).float()
    assert torch.allclose(L.sigmoid_cross_entropy_with_logits(x, z),
                          tF.binary_cross_entropy_with_logits(x, z, reduction="none"), atol=1e-6)
    assert torch.equal(L.onehot(torch.tensor([1, 0]), 3), torch.tensor([[0., 1, 0], [1, 0, 0]]))
    m = L.fixed_cross_entropy(logits, lab, config=L.LossConfig(divide_weight_sum=True))
    assert torch.allclose(m.loss, tF.cross_entropy(logits.reshape(-1, 37), lab.reshape(-1)), atol=1e-5)


def test_chunked_forms_equal_the_dense_one():
    logits, labels = _data(B=2, T=50, V=1000, seed=2)
    dense = tF.cross_entropy(logits.reshape(-1, 1000), labels.reshape(-1), reduction="none").view(2, 50)
    assert torch.allclose(L.sparse_cross_entropy_chunked_vocab(logits, labels, chunk_size=128), dense, atol=1e-4)
    g = torch.Generator().manual_seed(3)
    hidden, W = torch.randn(2, 50, 32, generator=g), torch.randn(1000, 32, generator=g) * 0.2
    lab = labels.clone()
    lab[0, :7] = -100
    ref = tF.cross_entropy((hidden @ W.t()).reshape(-1, 1000), lab.reshape(-1))
    assert torch.allclose(L.cross_entropy_blockwise_logits(hidden, W, lab, block_tokens=16), ref, atol=1e-4)


def test_normalising_factors():
    targets = torch.tensor([[5, 6, 7, 0], [8, 0, 0, 0]])
    f, w = L.get_factor_and_weight("NUM_REAL_TARGET_TOKENS", {"decoder_target_tokens": targets})
    assert float(f) == 4.0 and torch.equal(w, (targets > 0).float())
    f, _ = L.get_factor_and_weight("NUM_TOTAL_TARGET_TOKENS", {"decoder_target_tokens": targets})
    assert f == 8.0
    f, w = L.get_factor_and_weight("AVERAGE_PER_SEQUENCE", {"decoder_target_tokens": targets})
    assert f == 2.0 and torch.allclose(w.sum(-1), torch.ones(2))
    seg = torch.tensor([[1, 1, 2, 0], [1, 0, 0, 0]])
    f, w = L.get_factor_and_weight("AVERAGE_PER_SEQUENCE", {"decoder_target_tokens": targets,
                                                            "decoder_segment_ids": seg})
    assert f == 3.0 and torch.allclose(w[0], torch.tensor([0.5, 0.5, 1.0, 0.0]))
    assert L.get_factor_and_weight(7.0, {"decoder_loss_weights": targets})[0] == 7.0
    assert L.convert_special_loss_normalizing_factor_to_enum("average_per_sequence") == "AVERAGE_PER_SEQUENCE"


def test_causal_lm_strategy_skips_the_head_and_matches_the_logits_loss():
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=32)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    ids = torch.randint(0, 64, (2, 12))
    batch = {"input_ids": ids}
    st = L.resolve_loss_strategy(L.ForCausalLMLoss)
    assert isinstance(st, L.CausalLMLossStrategy)
    plan = st.plan_forward(module=model, labels=ids, loss_config=None, batch=batch, loss_kwargs={})
    assert plan.forward_kwargs == {"apply_lm_head": False}
    out = model(input_ids=ids, **plan.forward_kwargs)
    assert out.logits is None
    m = st.compute(module=model, outputs=out, labels=ids, loss_config=L.LossConfig(), batch=batch, loss_kwargs={})
    ref = L.ForCausalLMLoss(model(input_ids=ids).logits, ids)
    assert torch.allclose(m.loss, ref.loss, atol=1e-5)
    fn = L.resolve_loss_strategy(L.ForTokenClassification)
    assert isinstance(fn, L.FunctionalLossStrategy) and fn.plan_forward(
        module=model, labels=ids, loss_config=None, batch=batch, loss_kwargs={}).forward_kwargs == {}
