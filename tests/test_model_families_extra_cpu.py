"""Families without a ``transformers`` class: exported checkpoints are re-read with independent code (the documented
tensor layout + the Hugging Face Llama block they are equivalent to) and must give the same logits."""

import torch
import transformers

import easydel_b200.modules as M
from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

KW = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_attention_heads=4, num_key_value_heads=2,
          max_position_embeddings=64)


def _llama(sd, bias, eps):
    cfg = transformers.LlamaConfig(**KW, num_hidden_layers=2, attention_bias=bias, rms_norm_eps=eps)
    hf = transformers.LlamaForCausalLM(cfg).float().eval()
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not unexpected and not [m for m in missing if "rotary" not in m], (missing, unexpected)
    return hf


def _jitter(m):
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
    return m.eval()


def test_internlm2_grouped_wqkv_layout():
    torch.manual_seed(0)
    m = _jitter(M.InternLM2ForCausalLM(M.InternLM2Config(**KW, num_hidden_layers=2, bias=True), dtype=torch.float32,
                                       param_dtype=torch.float32))
    sd = internal_to_hf(m)
    hq, hkv, d = 4, 2, 16
    g = hq // hkv
    llama = {}
    for k, t in sd.items():
        k2 = (k.replace("model.tok_embeddings", "model.embed_tokens").replace("output.", "lm_head.")
              .replace("attention_norm", "input_layernorm").replace("ffn_norm", "post_attention_layernorm")
              .replace("feed_forward.w1", "mlp.gate_proj").replace("feed_forward.w3", "mlp.up_proj")
              .replace("feed_forward.w2", "mlp.down_proj").replace("attention.wo", "self_attn.o_proj"))
        if "attention.wqkv" in k:
            x = t.view(hkv, g + 2, d, -1) if t.dim() == 2 else t.view(hkv, g + 2, d)
            tail = k.rsplit(".", 1)[1]
            base = k.split("attention.wqkv")[0] + "self_attn."
            llama[base + "q_proj." + tail] = x[:, :g].reshape(hq * d, *t.shape[1:])
            llama[base + "k_proj." + tail] = x[:, g].reshape(hkv * d, *t.shape[1:])
            llama[base + "v_proj." + tail] = x[:, g + 1].reshape(hkv * d, *t.shape[1:])
        else:
            llama[k2] = t
    hf = _llama(llama, True, 1e-6)
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        assert (m(input_ids=ids).logits - hf(input_ids=ids).logits).abs().max() < 2e-4
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())


def test_exaone_is_llama_under_other_names():
    torch.manual_seed(0)
    kw = dict(KW)
    m = _jitter(M.ExaoneForCausalLM(M.ExaoneConfig(**kw, num_layers=2), dtype=torch.float32,
                                    param_dtype=torch.float32))
    assert m.config.num_hidden_layers == 2
    sd = internal_to_hf(m)
    ren = [("transformer.wte", "model.embed_tokens"), ("transformer.ln_f", "model.norm"),
           ("transformer.h.", "model.layers."), ("attn.attention.out_proj", "self_attn.o_proj"),
           ("attn.attention.", "self_attn."), ("ln_1", "input_layernorm"), ("ln_2", "post_attention_layernorm"),
           ("mlp.c_fc_0", "mlp.gate_proj"), ("mlp.c_fc_1", "mlp.up_proj"), ("mlp.c_proj", "mlp.down_proj")]
    llama = {}
    for k, t in sd.items():
        for a, b in ren:
            k = k.replace(a, b)
        llama[k] = t
    hf = _llama(llama, False, 1e-5)
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        assert (m(input_ids=ids).logits - hf(input_ids=ids).logits).abs().max() < 2e-4
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())


def test_grok1_block_structure_and_names():
    torch.manual_seed(0)
    cfg = M.Grok1Config(**KW, num_hidden_layers=2, num_experts=4, num_experts_per_tok=2, max_attn_value=5.0,
                        attn_output_multiplier=0.2, embedding_multiplier_scale=3.0, output_multiplier_scale=0.5)
    m = _jitter(M.Grok1ForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    sd = internal_to_hf(m)
    for frag in ("layers.0.attn.q_proj", "pre_attn_norm", "post_attn_norm", "pre_moe_norm", "post_moe_norm",
                 "moe_block.gate", "moe_block.experts.3.linear.", "experts.0.linear_v.", "experts.0.linear_1."):
        assert any(frag in k for k in sd), frag
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    # one layer by hand: x + post(attn(pre(x))) then x + post(moe(pre(x))), logits scaled
    ids = torch.randint(0, 128, (1, 10))
    out = m(input_ids=ids, output_hidden_states=True)
    layer = m.model.layers[0]
    x = out.hidden_states[0]
    pos = torch.arange(10)[None]
    a = layer.post_attn_out_layernorm(layer.self_attn(layer.input_layernorm(x), pos))
    x1 = x + a
    mo, _ = layer.mlp(layer.pre_feedforward_layernorm(x1))
    x2 = x1 + layer.post_feedforward_layernorm(mo)
    assert (x2 - out.hidden_states[1]).abs().max() < 1e-5
    assert (x - m.model.embed_tokens(ids) * 3.0).abs().max() < 1e-6
    assert layer.self_attn.softcap == 5.0 and abs(layer.self_attn.scale - 0.2) < 1e-9
    assert torch.allclose(out.logits, m.lm_head(out.last_hidden_state) * 0.5, atol=1e-5)


def test_arctic_parallel_residual_mlp_and_names():
    torch.manual_seed(0)
    cfg = M.ArcticConfig(**KW, num_hidden_layers=2, num_local_experts=4, num_experts_per_tok=2, moe_layer_frequency=2,
                         parallel_attn_mlp_res=True)
    m = _jitter(M.ArcticForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    l0, l1 = m.model.layers
    assert not l0.is_moe and l1.is_moe and l1.has_residual_mlp and not l0.has_residual_mlp
    assert l1.residual_mlp.down_proj.weight.shape == (64, 64)
    sd = internal_to_hf(m)
    for frag in ("layers.0.block_sparse_moe.mlp.w1.", "layers.1.block_sparse_moe.gate.",
                 "layers.1.block_sparse_moe.experts.3.w2.", "layers.1.residual_mlp.w3.", "layers.1.residual_layernorm."):
        assert any(frag in k for k in sd), frag
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    ids = torch.randint(0, 128, (1, 10))
    out = m(input_ids=ids, output_hidden_states=True)
    x = out.hidden_states[1]
    pos = torch.arange(10)[None]
    x1 = x + l1.self_attn(l1.input_layernorm(x), pos)
    want = x1 + l1.residual_mlp(l1.residual_layernorm(x1)) + l1.mlp(l1.post_attention_layernorm(x))[0]
    raw, _, _ = l1(x, None, pos)
    assert (raw - want).abs().max() < 1e-5
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    assert l1.residual_mlp.gate_up_proj.weight.grad.abs().sum() > 0


def test_dbrx_nested_config_fused_qkv_and_expert_layout():
    """The exported w1 / v1 / w2 matrices ([E * F, H] each) reproduce the block's expert output when used the way the
    original implementation uses them: ``silu(x w1_e^T) * (x v1_e^T)`` then ``@ w2_e``."""
    torch.manual_seed(0)
    cfg = M.DbrxConfig(d_model=64, n_heads=4, n_layers=2, max_seq_len=64, vocab_size=128,
                       attn_config=dict(kv_n_heads=2, clip_qkv=0.5, rope_theta=5000.0),
                       ffn_config=dict(ffn_hidden_size=96, moe_num_experts=4, moe_top_k=2))
    assert cfg.hidden_size == 64 and cfg.num_key_value_heads == 2 and cfg.intermediate_size == 96
    m = _jitter(M.DbrxForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    sd = internal_to_hf(m)
    assert sd["transformer.blocks.0.norm_attn_norm.attn.Wqkv.weight"].shape == (64 + 2 * 32, 64)
    assert sd["transformer.blocks.0.ffn.experts.mlp.w1"].shape == (4 * 96, 64)
    assert "transformer.blocks.1.norm_attn_norm.norm_2.weight" in sd and "transformer.blocks.0.ffn.router.layer.weight" in sd
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    layer = m.model.layers[0]
    assert layer.self_attn.clip_qkv == 0.5 and layer.input_layernorm.bias is None
    x = torch.randn(5, 64)
    got, logits = layer.mlp(x[None])
    p = torch.softmax(logits.float(), -1)
    w, idx = p.topk(2, -1)
    w = w / w.sum(-1, keepdim=True)
    w1, v1, w2 = (sd[f"transformer.blocks.0.ffn.experts.mlp.{n}"].view(4, 96, 64) for n in ("w1", "v1", "w2"))
    want = torch.zeros(5, 64)
    for t in range(5):
        for s in range(2):
            e = int(idx[t, s])
            h = torch.nn.functional.silu(x[t] @ w1[e].t()) * (x[t] @ v1[e].t())
            want[t] += w[t, s] * (h @ w2[e])
    assert (got[0] - want).abs().max() < 1e-5
    ids = torch.randint(0, 128, (1, 12))
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    assert torch.isfinite(met.loss)


def test_openelm_layerwise_scaling_shapes_names_and_decoding():
    torch.manual_seed(0)
    cfg = M.OpenELMConfig(vocab_size=128, max_context_length=64, num_transformer_layers=3, model_dim=64, head_dim=16,
                          qkv_multipliers=[0.5, 1.0], num_gqa_groups=2, ffn_multipliers=[0.5, 2.0], ffn_dim_divisor=16,
                          normalize_qk_projections=True, share_input_output_layers=True)
    assert cfg.num_query_heads == [2, 4, 4] and cfg.num_kv_heads == [1, 2, 2]
    m = _jitter(M.OpenELMForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    widths = [l.mlp.down_proj.weight.shape[1] for l in m.model.layers]
    assert widths == [32, 80, 128] and [l.self_attn.num_heads for l in m.model.layers] == [2, 4, 4]
    sd = internal_to_hf(m)
    assert sd["transformer.layers.0.attn.qkv_proj.weight"].shape == ((2 + 2 * 1) * 16, 64)
    assert sd["transformer.layers.2.ffn.proj_1.weight"].shape == (256, 64)
    assert "transformer.layers.1.attn.q_norm.weight" in sd and "lm_head.weight" not in sd
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    ids = torch.randint(0, 128, (2, 14))
    with torch.no_grad():
        full = m(input_ids=ids).logits
        cache = m.init_cache(2, 16)
        o = m(input_ids=ids[:, :10], past_key_values=cache).logits
        cache.advance(10)
        assert (o - full[:, :10]).abs().max() < 2e-4
        o = m(input_ids=ids[:, 10:11], past_key_values=cache).logits
        assert (o[:, 0] - full[:, 10]).abs().max() < 2e-4
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss)


def test_kimi_linear_hybrid_of_delta_attention_and_latent_attention():
    torch.manual_seed(0)
    cfg = M.KimiLinearConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                             num_attention_heads=4, num_key_value_heads=4, kv_lora_rank=16, qk_nope_head_dim=16,
                             qk_rope_head_dim=8, v_head_dim=16, num_experts=4, num_experts_per_token=2,
                             moe_intermediate_size=32, num_shared_experts=1, first_k_dense_replace=1,
                             max_position_embeddings=64,
                             linear_attn_config=dict(kda_layers=[1, 2, 3], full_attn_layers=[4], num_heads=4,
                                                     head_dim=16, short_conv_kernel_size=4, gate_low_rank_dim=8))
    m = _jitter(M.KimiLinearForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    kinds = [type(getattr(l, "linear_attn", l.self_attn if hasattr(l, "self_attn") else None)).__name__
             for l in m.model.layers]
    assert kinds == ["KimiDeltaAttention"] * 3 + ["MLAttention"]
    assert not m.model.layers[3].self_attn.use_rope and [l.is_moe for l in m.model.layers] == [False, True, True, True]
    sd = internal_to_hf(m)
    for frag in ("layers.0.linear_attn.q_conv1d.weight", "layers.1.linear_attn.f_b_proj.weight",
                 "layers.3.self_attn.kv_a_proj_with_mqa.weight", "layers.1.block_sparse_moe.gate.weight",
                 "layers.2.block_sparse_moe.gate.e_score_correction_bias", "layers.1.block_sparse_moe.experts.0.w1.",
                 "layers.1.block_sparse_moe.shared_experts.down_proj.", "layers.0.mlp.gate_proj.weight"):
        assert any(frag in k for k in sd), frag
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    ids = torch.randint(0, 128, (2, 14))
    with torch.no_grad():
        full = m(input_ids=ids).logits
        cache = m.init_cache(2, 16)
        assert set(cache.linear) == {0, 1, 2}
        o = m(input_ids=ids[:, :9], past_key_values=cache).logits
        cache.advance(9)
        assert (o - full[:, :9]).abs().max() < 3e-4
        for t in range(9, 14):
            o = m(input_ids=ids[:, t:t + 1], past_key_values=cache).logits
            cache.advance(1)
            assert (o[:, 0] - full[:, t]).abs().max() < 3e-4, t
    _, met = m.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    assert torch.isfinite(met.loss) and m.model.layers[0].linear_attn.A_log.grad is not None


def test_gidd_bidirectional_diffusion_lm():
    torch.manual_seed(0)
    cfg = M.GiddConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                       num_attention_heads=4, max_position_embeddings=64, resid_scale=2.0)
    m = _jitter(M.GiddForDiffusionLM(cfg, dtype=torch.float32, param_dtype=torch.float32))
    att = m.model.layers[0].self_attn
    assert not att.causal and att.scale == 1.0
    assert abs(float(att.head_scale.mean()) - 2 * torch.log(torch.tensor(64.0)).item()) < 0.5
    sd = internal_to_hf(m)
    assert sd["model.layers.0.self_attn.qk_scale"].shape == (1, 1, 4, 1) and "model.layers.1.mlp.up_proj.weight" in sd
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    ids = torch.randint(0, 128, (1, 10))
    with torch.no_grad():
        a = m(input_ids=ids).logits
        ids2 = ids.clone()
        ids2[0, -1] = (ids2[0, -1] + 1) % 128
        b = m(input_ids=ids2).logits
    assert (a[0, 0] - b[0, 0]).abs().max() > 1e-6        # a later token changes an earlier position: not causal
    # one block by hand: q, k normalised over the whole projection, per-head temperature, residual scale
    layer = m.model.layers[0]
    x = m.model.embed_tokens(ids)
    h = layer.input_layernorm(x)
    qkv = att.qkv_proj(h)
    q, k, v = qkv[..., :64], qkv[..., 64:128], qkv[..., 128:]
    q = q / (q.pow(2).sum(-1, keepdim=True) + 1e-6).sqrt()
    k = k / (k.pow(2).sum(-1, keepdim=True) + 1e-6).sqrt()
    q, k = att.rotary(torch.arange(10)[None], q.view(1, 10, 4, 16), k.view(1, 10, 4, 16))
    s = torch.einsum("bqhd,bkhd->bhqk", q * att.head_scale[None, None, :, None], k)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.view(1, 10, 4, 16)).reshape(1, 10, 64)
    x1 = x + 2.0 * att.o_proj(o)
    want = x1 + 2.0 * layer.mlp.fc2(torch.relu(layer.mlp.fc1(layer.post_attention_layernorm(x1))).square())
    got, _, _ = layer(x, None, torch.arange(10)[None])
    assert (got - want).abs().max() < 1e-4
    labels = torch.full_like(ids, -100)
    labels[0, 3], labels[0, 7] = 5, 9
    _, met = m.compute_loss(input_ids=ids, labels=labels)
    with torch.no_grad():
        ref = torch.nn.functional.cross_entropy(a[0, [3, 7]].float(), torch.tensor([5, 9]))
    assert abs(float(met.loss) - float(ref)) < 1e-5


def test_xerxes_block_variants_and_xerxes2_latent_attention():
    torch.manual_seed(0)
    ids = torch.randint(0, 128, (2, 12))
    # four-norm block with a sliding / global pattern
    m = _jitter(M.XerxesForCausalLM(M.XerxesConfig(**KW, num_hidden_layers=2, head_dim=16, window_pattern=2,
                                                   sliding_window=4), dtype=torch.float32,
                                    param_dtype=torch.float32))
    l0, l1 = m.model.layers
    assert l0.self_attn.sliding_window == 4 and l1.self_attn.sliding_window is None
    sd = internal_to_hf(m)
    assert {"model.layers.0.post_attention_layernorm.weight", "model.layers.0.pre_feedforward_layernorm.weight",
            "model.layers.0.post_feedforward_layernorm.weight"} <= set(sd)
    back = hf_to_internal(m, sd)
    assert all(torch.equal(back[k], v) for k, v in m.state_dict().items())
    x = m.model.embed_tokens(ids) * 8.0            # sqrt(64)
    pos = torch.arange(12)[None].expand(2, 12)
    x1 = x + l0.post_attn_out_layernorm(l0.self_attn(l0.input_layernorm(x), pos))
    want = x1 + l0.post_feedforward_layernorm(l0.mlp(l0.pre_feedforward_layernorm(x1)))
    out = m(input_ids=ids, output_hidden_states=True)
    assert (out.hidden_states[1] - want).abs().max() < 1e-4
    # QK norm without experts: the plain pre-norm block, unscaled embeddings
    p = M.XerxesForCausalLM(M.XerxesConfig(**KW, num_hidden_layers=1, head_dim=16, xe_kvnorm=True), dtype=torch.float32,
                            param_dtype=torch.float32)
    assert not p.spec.sandwich_norm and p.spec.embed_scale == 1.0 and hasattr(p.model.layers[0].self_attn, "q_norm")
    assert "model.layers.0.post_attention_layernorm.weight" in internal_to_hf(p)
    # xerxes2: latent attention + four norms + experts every layer
    c2 = M.Xerxes2Config(vocab_size=128, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                         num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=64, num_experts=4,
                         num_experts_per_tok=2, q_lora_dim=24, kv_lora_dim=16, qk_rope_head_dim=8,
                         qk_nope_head_dim=16, vhead_dim=16, mlp_only_layers=[0])
    m2 = _jitter(M.Xerxes2ForCausalLM(c2, dtype=torch.float32, param_dtype=torch.float32))
    assert type(m2.model.layers[0].self_attn).__name__ == "MLAttention"
    assert [l.is_moe for l in m2.model.layers] == [False, True]
    sd2 = internal_to_hf(m2)
    assert "model.layers.1.self_attn.kv_a_proj_with_mqa.weight" in sd2 and "model.layers.1.mlp.gate.weight" in sd2
    back = hf_to_internal(m2, sd2)
    assert all(torch.equal(back[k], v) for k, v in m2.state_dict().items())
    with torch.no_grad():
        full = m2(input_ids=ids).logits
        cache = m2.init_cache(2, 16)
        o = m2(input_ids=ids[:, :8], past_key_values=cache).logits
        cache.advance(8)
        o2 = m2(input_ids=ids[:, 8:9], past_key_values=cache).logits
    assert (o - full[:, :8]).abs().max() < 3e-4 and (o2[:, 0] - full[:, 8]).abs().max() < 3e-4
