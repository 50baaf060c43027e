"""Qwen3-VL (easydel/modules/qwen3_vl): the Qwen2-VL recipe with a learned, bilinearly interpolated position table
in the vision tower, DeepStack (features of intermediate vision layers, merged by their own small MLPs, are added to
the hidden states of the first decoder layers at the image positions), a Qwen3 language model (per-head QK norm) and
interleaved three-stream rotary positions.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from ...layers.attention import Attention
from ...layers.linears import ColumnParallelLinear
from ...layers.norms import LayerNorm
from .._base.vlm import VLMConfig
from ..qwen2_vl.modeling_qwen2_vl import Qwen2VLForConditionalGeneration, _GridRotary, mrope_positions


@register_config("qwen3_vl_vision")
class Qwen3VLVisionConfig(EasyDeLBaseConfig):
    model_type = "qwen3_vl_vision"
    hf_config_keys = ("depth", "hidden_size", "hidden_act", "intermediate_size", "num_heads", "in_channels",
                      "patch_size", "spatial_merge_size", "temporal_patch_size", "out_hidden_size",
                      "num_position_embeddings", "deepstack_visual_indexes")

    def __init__(self, depth=27, hidden_size=1152, hidden_act="gelu_pytorch_tanh", intermediate_size=4304,
                 num_heads=16, in_channels=3, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
                 out_hidden_size=3584, num_position_embeddings=2304, deepstack_visual_indexes=(8, 16, 24),
                 initializer_range=0.02, **kw):
        self.depth, self.hidden_size, self.hidden_act, self.intermediate_size = depth, hidden_size, hidden_act, \
            intermediate_size
        self.num_heads, self.in_channels, self.patch_size = num_heads, in_channels, patch_size
        self.spatial_merge_size, self.temporal_patch_size = spatial_merge_size, temporal_patch_size
        self.out_hidden_size, self.num_position_embeddings = out_hidden_size, num_position_embeddings
        self.deepstack_visual_indexes = list(deepstack_visual_indexes)
        self.initializer_range = initializer_range
        super().__init__(**kw)


@register_config("qwen3_vl")
class Qwen3VLConfig(VLMConfig):
    model_type = "qwen3_vl"
    vision_default, text_default = "qwen3_vl_vision", "qwen3"

    def __init__(self, vision_config=None, text_config=None, image_token_id=151655, video_token_id=151656,
                 vision_start_token_id=151652, vision_end_token_id=151653, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="qwen3_vl_vision")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type=self.text_default)
            inner = text_config.get("rope_parameters") or text_config.get("rope_scaling") or {}
            text_config.setdefault("rope_theta", inner.get("rope_theta", 5000000.0))
            if self.text_default == "qwen3_moe":
                text_config.setdefault("norm_topk_prob", True)
        kw = self._init_parts(vision_config, text_config, image_token_id, kw)
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.vision_start_token_id, self.vision_end_token_id = vision_start_token_id, vision_end_token_id
        super().__init__(**kw)


class _MLP(nn.Module):
    def __init__(self, d, inner, act, dtype):
        super().__init__()
        from ...ops.reference import ACT2FN

        self.linear_fc1 = ColumnParallelLinear(d, inner, bias=True, dtype=dtype)
        self.linear_fc2 = ColumnParallelLinear(inner, d, bias=True, dtype=dtype)
        self.act = ACT2FN[act]

    def forward(self, x):
        return self.linear_fc2(self.act(self.linear_fc1(x)))


class _Block(nn.Module):
    def __init__(self, c: Qwen3VLVisionConfig, idx, dtype):
        super().__init__()
        d = c.hidden_size
        self.norm1, self.norm2 = LayerNorm(d, 1e-6, dtype=dtype), LayerNorm(d, 1e-6, dtype=dtype)
        self.attn = Attention(d, c.num_heads, c.num_heads, d // c.num_heads, layer_idx=idx, bias=True, o_bias=True,
                              rope=None, causal=False, dtype=dtype, init_std=c.initializer_range)
        self.mlp = _MLP(d, c.intermediate_size, c.hidden_act, dtype)

    def forward(self, x, pos, seg):
        x = x + self.attn(self.norm1(x), pos, segment_ids=seg)
        return x + self.mlp(self.norm2(x))


class _Merger(nn.Module):
    """LayerNorm (before or after folding the 2x2 neighbourhood into the channels) + two-layer GELU MLP."""

    def __init__(self, c: Qwen3VLVisionConfig, postshuffle: bool, dtype):
        super().__init__()
        self.m = c.hidden_size * c.spatial_merge_size ** 2
        self.post = postshuffle
        self.norm = LayerNorm(self.m if postshuffle else c.hidden_size, 1e-6, dtype=dtype)
        self.linear_fc1 = ColumnParallelLinear(self.m, self.m, bias=True, dtype=dtype)
        self.linear_fc2 = ColumnParallelLinear(self.m, c.out_hidden_size, bias=True, dtype=dtype)

    def forward(self, x):
        x = self.norm(x.reshape(-1, self.m)) if self.post else self.norm(x).reshape(-1, self.m)
        return self.linear_fc2(torch.nn.functional.gelu(self.linear_fc1(x)))


class Qwen3VLVisionTransformer(nn.Module):
    def __init__(self, c: Qwen3VLVisionConfig, dtype):
        super().__init__()
        self.cfg = c
        self.patch_embed = nn.Module()
        k = (c.temporal_patch_size, c.patch_size, c.patch_size)
        self.patch_embed.proj = nn.Conv3d(c.in_channels, c.hidden_size, k, stride=k, bias=True, dtype=dtype)
        self.pos_embed = nn.Embedding(c.num_position_embeddings, c.hidden_size, dtype=dtype)
        self.side = int(c.num_position_embeddings ** 0.5)
        hd = c.hidden_size // c.num_heads
        self.rotary = _GridRotary(hd, hd // 2, 4096, 10000.0, is_neox_style=True)
        self.blocks = nn.ModuleList([_Block(c, i, dtype) for i in range(c.depth)])
        for b in self.blocks:
            b.attn.rotary = self.rotary
        self.merger = _Merger(c, False, dtype)
        self.deepstack_merger_list = nn.ModuleList([_Merger(c, True, dtype) for _ in c.deepstack_visual_indexes])

    def grid_positions(self, grid_thw):
        s = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            q = torch.arange(w)[None, :].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            out.append(torch.stack([r, q]).repeat(1, t))
        return torch.cat(out, 1)

    def interpolated_positions(self, grid_thw):
        """Bilinear read of the ``side x side`` learned table at every patch centre, in merge-block order."""
        s, n, w_tab = self.cfg.spatial_merge_size, self.side, self.pos_embed.weight
        out = []
        for t, h, w in grid_thw.tolist():
            hi = torch.linspace(0, n - 1, h, device=w_tab.device)
            wi = torch.linspace(0, n - 1, w, device=w_tab.device)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clamp(max=n - 1), (w0 + 1).clamp(max=n - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            tab = w_tab.view(n, n, -1)
            e = (tab[h0.long()][:, w0.long()] * ((1 - dh) * (1 - dw))[..., None].to(w_tab.dtype)
                 + tab[h0.long()][:, w1.long()] * ((1 - dh) * dw)[..., None].to(w_tab.dtype)
                 + tab[h1.long()][:, w0.long()] * (dh * (1 - dw))[..., None].to(w_tab.dtype)
                 + tab[h1.long()][:, w1.long()] * (dh * dw)[..., None].to(w_tab.dtype))          # [h, w, D]
            e = e.view(h // s, s, w // s, s, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out)

    def forward(self, pixel_values, grid_thw):
        """-> (merged features ``[tokens, out]``, one merged feature tensor per DeepStack layer)."""
        c = self.cfg
        w = self.patch_embed.proj.weight
        x = torch.nn.functional.linear(pixel_values.to(w.dtype), w.view(c.hidden_size, -1), self.patch_embed.proj.bias)
        x = (x + self.interpolated_positions(grid_thw))[None]
        pos = self.grid_positions(grid_thw).to(x.device)[:, None]
        lens = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        seg = torch.repeat_interleave(torch.arange(1, lens.numel() + 1, dtype=torch.int32), lens)[None].to(x.device)
        if lens.numel() == 1:
            seg = None
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, pos, seg)
            if i in c.deepstack_visual_indexes:
                deep.append(self.deepstack_merger_list[c.deepstack_visual_indexes.index(i)](x[0]))
        return self.merger(x[0]), deep


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen3VLConfig, model_type="qwen3_vl")
class Qwen3VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super(Qwen2VLForConditionalGeneration, self).__init__(config, dtype, param_dtype, precision, rngs)
        self.visual = Qwen3VLVisionTransformer(config.vision_config, self.param_dtype)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)
        self.rope_deltas = None

    def get_image_features(self, pixel_values, image_grid_thw=None, **_):
        return self.visual(pixel_values, image_grid_thw)[0]

    def _merge(self, input_ids, pixel_values, image_grid_thw, pixel_values_videos=None, video_grid_thw=None):
        emb = self.embed_text(input_ids)
        if pixel_values is None and pixel_values_videos is None:
            return emb, None
        emb = emb.clone()
        stacks = None
        for px, grid, tok, what in ((pixel_values, image_grid_thw, self.config.image_token_id, "image"),
                                    (pixel_values_videos, video_grid_thw, self.config.video_token_id, "video")):
            if px is None:
                continue
            feats, deep = self.visual(px, grid)
            mask = input_ids == tok
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} {what} placeholder tokens for {feats.shape[0]} feature rows")
            emb[mask] = feats.to(emb.dtype)
            if stacks is None:
                stacks = [torch.zeros_like(emb) for _ in deep]
            for z, d in zip(stacks, deep):
                z[mask] = d.to(emb.dtype)
        return emb, stacks

    @staticmethod
    def _frame_grids(video_grid_thw):
        """Every frame group of a video is its own placeholder run (timestamps sit between them): one ``(1, h, w)``
        grid per temporal patch."""
        if video_grid_thw is None:
            return None
        g = torch.repeat_interleave(video_grid_thw, video_grid_thw[:, 0], dim=0).clone()
        g[:, 0] = 1
        return g

    def _positions(self, input_ids, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw,
                   attention_mask):
        return mrope_positions(
            input_ids, self.config.image_token_id, image_grid_thw if pixel_values is not None else None,
            self.config.vision_config.spatial_merge_size, attention_mask, self.config.video_token_id,
            self._frame_grids(video_grid_thw) if pixel_values_videos is not None else None)

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, **kw):
        first = past_key_values is None or past_key_values.seq_len() == 0
        if inputs_embeds is None:
            inputs_embeds, stacks = self._merge(input_ids, pixel_values if first else None, image_grid_thw,
                                                pixel_values_videos if first else None, video_grid_thw)
            if stacks:
                kw["deepstack_embeds"] = stacks
        if position_ids is None and input_ids is not None:
            if first:
                position_ids, self.rope_deltas = self._positions(input_ids, pixel_values, image_grid_thw,
                                                                 pixel_values_videos, video_grid_thw, attention_mask)
            else:
                B, T = input_ids.shape
                start = past_key_values.seq_len()
                base = torch.arange(start, start + T, device=input_ids.device)[None].expand(B, T)
                if self.rope_deltas is not None:
                    base = base + self.rope_deltas[:, None]
                position_ids = base[None].expand(3, B, T)
        return self.language_model(inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                                   position_ids=position_ids, past_key_values=past_key_values, **kw)

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        call = dict(call)
        ids = call.pop("input_ids")
        grid, pix = call.pop("image_grid_thw", None), call.pop("pixel_values", None)
        vgrid, vpix = call.pop("video_grid_thw", None), call.pop("pixel_values_videos", None)
        if call.get("position_ids") is None:
            call["position_ids"], _ = self._positions(ids, pix, grid, vpix, vgrid, call.get("attention_mask"))
        emb, stacks = self._merge(ids, pix, grid, vpix, vgrid)
        if stacks:
            call["deepstack_embeds"] = stacks
        call["inputs_embeds"] = emb
        labels = labels.masked_fill((ids == self.config.image_token_id) | (ids == self.config.video_token_id),
                                    loss_config.ignore_index)
        return self.language_model._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)


@register_config("qwen3_vl_moe")
class Qwen3VLMoeConfig(Qwen3VLConfig):
    """Qwen3-VL with the Qwen3-MoE language model (easydel/modules/qwen3_vl_moe)."""

    model_type = "qwen3_vl_moe"
    vision_default, text_default = "qwen3_vl_vision", "qwen3_moe"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen3VLMoeConfig, model_type="qwen3_vl_moe")
class Qwen3VLMoeForConditionalGeneration(Qwen3VLForConditionalGeneration):
    pass


# ---------------------------------------------------------------------------------------------------------------------
# Qwen3.5 (easydel/modules/qwen3_5, easydel/modules/qwen3_5_moe): the same vision tower without DeepStack in front
# of the hybrid gated-DeltaNet / attention language models; attention layers rotate a quarter of each head with the
# interleaved three-stream positions, DeltaNet layers take no positions.
# ---------------------------------------------------------------------------------------------------------------------
@register_config("qwen3_5_vision")
class Qwen3_5VisionConfig(Qwen3VLVisionConfig):
    model_type = "qwen3_5_vision"

    def __init__(self, **kw):
        kw.setdefault("deepstack_visual_indexes", ())
        super().__init__(**kw)


def _qwen3_5_text_dict(text_config, model_type):
    text_config = dict(text_config, model_type=model_type)
    rp = text_config.pop("rope_parameters", None)
    if rp:      # one dict in the published configs: base, rotated fraction and the three-stream sections
        rp = dict(rp)
        text_config.setdefault("rope_theta", rp.pop("rope_theta", 10000000.0))
        text_config.setdefault("partial_rotary_factor", rp.pop("partial_rotary_factor", 0.25))
        text_config.setdefault("rope_scaling", rp)
    return text_config


@register_config("qwen3_5")
class Qwen3_5Config(Qwen3VLConfig):
    model_type = "qwen3_5"
    vision_default, text_default = "qwen3_5_vision", "qwen3_5_text"

    def __init__(self, vision_config=None, text_config=None, image_token_id=248056, video_token_id=248057,
                 vision_start_token_id=248053, vision_end_token_id=248054, **kw):
        if isinstance(vision_config, dict):
            vision_config = Qwen3_5VisionConfig(**{k: v for k, v in vision_config.items() if k != "model_type"})
        if isinstance(text_config, dict):
            from ...infra.factory import registry

            text_config = registry.get_config(self.text_default)(
                **{k: v for k, v in _qwen3_5_text_dict(text_config, self.text_default).items() if k != "model_type"})
        super().__init__(vision_config=vision_config, text_config=text_config, image_token_id=image_token_id,
                         video_token_id=video_token_id, vision_start_token_id=vision_start_token_id,
                         vision_end_token_id=vision_end_token_id, **kw)


@register_config("qwen3_5_moe")
class Qwen3_5MoeConfig(Qwen3_5Config):
    model_type = "qwen3_5_moe"
    vision_default, text_default = "qwen3_5_vision", "qwen3_5_moe_text"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen3_5Config, model_type="qwen3_5")
class Qwen3_5ForConditionalGeneration(Qwen3VLForConditionalGeneration):
    pass


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen3_5MoeConfig, model_type="qwen3_5_moe")
class Qwen3_5MoeForConditionalGeneration(Qwen3VLForConditionalGeneration):
    pass
