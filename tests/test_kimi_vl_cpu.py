"""Kimi-VL: the MoonViT tower against a restatement in complex arithmetic, placeholder merge, training, decoding and
the checkpoint-name round trip (the architecture ships as remote code, so Hugging Face has no class to compare with)."""

import torch

from easydel_b200.modules.kimi_vl import KimiVLConfig, KimiVLForConditionalGeneration
from easydel_b200.modules.kimi_vl.modeling_kimi_vl import grid_rope_angles
from easydel_b200.utils.parameters_transformation import hf_to_internal, internal_to_hf

IMG = 99


def _model():
    torch.manual_seed(0)
    cfg = KimiVLConfig(
        vision_config=dict(patch_size=4, init_pos_emb_height=6, init_pos_emb_width=6, num_attention_heads=2,
                           num_hidden_layers=2, hidden_size=32, intermediate_size=48, merge_kernel_size=(2, 2)),
        text_config=dict(vocab_size=128, hidden_size=48, intermediate_size=64, moe_intermediate_size=32,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, q_lora_rank=24,
                         kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=8, n_routed_experts=4,
                         n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1,
                         max_position_embeddings=128),
        media_placeholder_token_id=IMG)
    m = KimiVLForConditionalGeneration(cfg, dtype=torch.float32).eval()
    with torch.no_grad():
        for p in m.vision_tower.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    return cfg, m


def _tower_reference(m, pix, grid):
    """fp32 restatement: complex rotation with the published frequency layout, dense block-diagonal attention."""
    vt, c = m.vision_tower, m.config.vision_config
    heads, hd = c.num_attention_heads, c.hidden_size // c.num_attention_heads
    w = vt.patch_embed.proj.weight
    x = torch.nn.functional.conv2d(pix, w, vt.patch_embed.proj.bias, stride=c.patch_size).flatten(1)
    tab = vt.patch_embed.pos_emb.weight
    pos, cis, blocks = [], [], []
    freqs = 1.0 / (10000.0 ** (torch.arange(0, hd, 4).float() / hd))
    for h, wd in grid.tolist():
        if (h, wd) == tuple(tab.shape[:2]):
            pos.append(tab.reshape(h * wd, -1))
        else:
            pos.append(torch.nn.functional.interpolate(tab.permute(2, 0, 1)[None], size=(h, wd), mode="bicubic",
                                                       antialias=True)[0].permute(1, 2, 0).reshape(h * wd, -1))
        flat = torch.arange(h * wd)
        xp, yp = (flat % wd).float(), (flat // wd).float()
        xc = torch.polar(torch.ones(h * wd, hd // 4), torch.outer(xp, freqs))
        yc = torch.polar(torch.ones(h * wd, hd // 4), torch.outer(yp, freqs))
        cis.append(torch.stack([xc, yc], -1).reshape(h * wd, -1))
        blocks.append(torch.ones(h * wd, h * wd))
    x = x + torch.cat(pos)
    cis = torch.cat(cis)[:, None]
    allow = torch.block_diag(*blocks).bool()
    T = x.shape[0]
    for b in vt.encoder.blocks:
        qkv = b.wqkv(b.norm0(x)).view(T, 3, heads, hd)
        rot = lambda t: torch.view_as_real(torch.view_as_complex(t.reshape(T, heads, hd // 2, 2).contiguous()) * cis
                                           ).reshape(T, heads, hd)                    # noqa: E731
        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        s = torch.einsum("thd,shd->hts", q, k) * hd ** -0.5
        s = s.masked_fill(~allow[None], float("-inf")).softmax(-1)
        x = x + b.wo(torch.einsum("hts,shd->thd", s, v).reshape(T, -1))
        x = x + b.mlp.fc1(torch.nn.functional.gelu(b.mlp.fc0(b.norm1(x)), approximate="tanh"))
    x = vt.encoder.final_layernorm(x)
    out, at = [], 0
    for h, wd in grid.tolist():
        seq = x[at:at + h * wd].reshape(h // 2, 2, wd // 2, 2, -1).permute(0, 2, 1, 3, 4)
        out.append(seq.reshape(-1, 4, x.shape[-1]))
        at += h * wd
    pr = m.multi_modal_projector
    y = pr.pre_norm(torch.cat(out)).reshape(-1, pr.inner)
    return pr.linear_2(torch.nn.functional.gelu(pr.linear_1(y)))


def _inputs():
    grid = torch.tensor([[4, 6], [6, 6], [2, 4]])
    n_patch = int((grid[:, 0] * grid[:, 1]).sum())
    pix = torch.randn(n_patch, 3, 4, 4)
    n_tok = n_patch // 4
    ids = torch.randint(0, 90, (1, n_tok + 9))
    ids[0, 3:3 + n_tok] = IMG
    return grid, pix, ids


def test_rope_angles_pair_layout():
    ang = grid_rope_angles(torch.tensor([[2, 3]]), 8)
    f = 1.0 / (10000.0 ** (torch.arange(0, 8, 4).float() / 8))
    assert ang.shape == (6, 4)
    # patch (row 1, col 2) is index 5: pairs 0, 2 follow the column, 1, 3 the row
    torch.testing.assert_close(ang[5], torch.stack([2 * f[0], 1 * f[0], 2 * f[1], 1 * f[1]]))


def test_tower_matches_complex_restatement_and_merges():
    cfg, m = _model()
    grid, pix, ids = _inputs()
    with torch.no_grad():
        feats = m.get_image_features(pix, image_grid_hws=grid)
        ref = _tower_reference(m, pix, grid)
        assert feats.shape == (int((grid[:, 0] * grid[:, 1]).sum()) // 4, 48)
        torch.testing.assert_close(feats, ref, atol=2e-4, rtol=2e-4)
        out = m(input_ids=ids, pixel_values=pix, image_grid_hws=grid)
        emb = m.embed_text(ids).clone()
        emb[ids == IMG] = ref
        want = m.language_model(inputs_embeds=emb)
        torch.testing.assert_close(out.logits, want.logits, atol=2e-4, rtol=2e-4)
        # one image alone gives the same rows as inside the packed batch (attention stays inside an image)
        solo = m.get_image_features(pix[24:60], image_grid_hws=grid[1:2])
        torch.testing.assert_close(solo, feats[6:15], atol=2e-4, rtol=2e-4)


def test_trains_decodes_and_round_trips_names():
    cfg, m = _model()
    grid, pix, ids = _inputs()
    m.train()
    _, met = m.compute_loss(input_ids=ids, labels=ids, pixel_values=pix, image_grid_hws=grid)
    loss = met.loss
    loss.backward()
    assert torch.isfinite(loss)
    assert m.vision_tower.encoder.blocks[0].wqkv.weight.grad.abs().sum() > 0
    assert m.multi_modal_projector.linear_1.weight.grad.abs().sum() > 0
    m.eval()
    with torch.no_grad():
        full = m(input_ids=ids, pixel_values=pix, image_grid_hws=grid).logits
        cache = m.init_cache(1, 64)
        m(input_ids=ids[:, :-2], pixel_values=pix, image_grid_hws=grid, past_key_values=cache)
        cache.advance(ids.shape[1] - 2)
        nxt = m(input_ids=ids[:, -2:], past_key_values=cache).logits
        torch.testing.assert_close(nxt, full[:, -2:], atol=3e-4, rtol=3e-4)
    hf = internal_to_hf(m)
    assert "vision_tower.encoder.blocks.0.wqkv.weight" in hf and "vision_tower.patch_embed.pos_emb.weight" in hf
    assert "multi_modal_projector.linear_1.weight" in hf and "language_model.lm_head.weight" in hf
    assert any(k.startswith("language_model.model.layers.1.mlp.experts.") for k in hf)
    torch.manual_seed(1)
    m2 = KimiVLForConditionalGeneration(cfg, dtype=torch.float32).eval()
    m2.load_state_dict(hf_to_internal(m2, hf))
    with torch.no_grad():
        torch.testing.assert_close(m2(input_ids=ids, pixel_values=pix, image_grid_hws=grid).logits, full)
