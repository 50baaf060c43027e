"""GLM-4V / GLM-4.6V / GLM-4V-MoE (easydel/modules/glm4v, glm46v, glm4v_moe): the Qwen2-VL input convention
(flattened pixel blocks + ``image_grid_thw``, three-stream rotary positions in the language model) with GLM's vision
tower: RMSNorm blocks with gated MLPs, a learned position table read by bicubic interpolation at every patch centre,
rotary positions on the patch grid, a strided-convolution 2x2 downsample and a gated-MLP merger.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from ...layers.attention import Attention
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import GatedMLP
from ...layers.norms import LayerNorm, RMSNorm
from .._base.vlm import VLMConfig
from ..qwen2_vl.modeling_qwen2_vl import Qwen2VLForConditionalGeneration, _GridRotary


@register_config("glm4v_vision")
class Glm4vVisionConfig(EasyDeLBaseConfig):
    model_type = "glm4v_vision"
    hf_config_keys = ("depth", "hidden_size", "hidden_act", "attention_bias", "num_heads", "in_channels", "image_size",
                      "patch_size", "rms_norm_eps", "spatial_merge_size", "temporal_patch_size", "out_hidden_size",
                      "intermediate_size")

    def __init__(self, depth=24, hidden_size=1536, hidden_act="silu", attention_bias=False, num_heads=12,
                 in_channels=3, image_size=336, patch_size=14, rms_norm_eps=1e-5, spatial_merge_size=2,
                 temporal_patch_size=2, out_hidden_size=4096, intermediate_size=13696, initializer_range=0.02, **kw):
        self.depth, self.hidden_size, self.hidden_act, self.attention_bias = depth, hidden_size, hidden_act, \
            attention_bias
        self.num_heads, self.in_channels, self.image_size, self.patch_size = num_heads, in_channels, image_size, \
            patch_size
        self.rms_norm_eps, self.spatial_merge_size, self.temporal_patch_size = rms_norm_eps, spatial_merge_size, \
            temporal_patch_size
        self.out_hidden_size, self.intermediate_size, self.initializer_range = out_hidden_size, intermediate_size, \
            initializer_range
        super().__init__(**kw)


class _Glm4vConfigBase(VLMConfig):
    vision_default, text_default = "glm4v_vision", "glm4v_text"

    def __init__(self, vision_config=None, text_config=None, image_token_id=151343, video_token_id=151344,
                 image_start_token_id=151339, image_end_token_id=151340, video_start_token_id=151341,
                 video_end_token_id=151342, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="glm4v_vision")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type=self.text_default)
        kw = self._init_parts(vision_config, text_config, image_token_id, kw)
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.image_start_token_id, self.image_end_token_id = image_start_token_id, image_end_token_id
        self.video_start_token_id, self.video_end_token_id = video_start_token_id, video_end_token_id
        super().__init__(**kw)


@register_config("glm4v")
class Glm4vConfig(_Glm4vConfigBase):
    model_type = "glm4v"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_config("glm46v")
class Glm46VConfig(_Glm4vConfigBase):
    model_type = "glm46v"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_config("glm4v_moe")
class Glm4vMoeConfig(_Glm4vConfigBase):
    model_type = "glm4v_moe"
    text_default = "glm4_moe"

    def __init__(self, **kw):
        super().__init__(**kw)


class _Block(nn.Module):
    def __init__(self, c: Glm4vVisionConfig, idx, dtype):
        super().__init__()
        d = c.hidden_size
        self.norm1, self.norm2 = RMSNorm(d, c.rms_norm_eps, dtype), RMSNorm(d, c.rms_norm_eps, dtype)
        self.attn = Attention(d, c.num_heads, c.num_heads, d // c.num_heads, layer_idx=idx, bias=c.attention_bias,
                              o_bias=False, rope=None, causal=False, dtype=dtype, init_std=c.initializer_range)
        self.mlp = GatedMLP(d, c.out_hidden_size, c.hidden_act, False, dtype, c.initializer_range)

    def forward(self, x, pos, seg):
        x = x + self.attn(self.norm1(x), pos, segment_ids=seg)
        return x + self.mlp(self.norm2(x))


class _Merger(nn.Module):
    def __init__(self, dim, context_dim, act, dtype):
        super().__init__()
        self.proj = ColumnParallelLinear(dim, dim, bias=False, dtype=dtype)
        self.post_projection_norm = LayerNorm(dim, 1e-5, dtype=dtype)
        self.mlp = GatedMLP(dim, context_dim, act, False, dtype, 0.02)

    def forward(self, x):
        return self.mlp(torch.nn.functional.gelu(self.post_projection_norm(self.proj(x))))


class Glm4vVisionTransformer(nn.Module):
    def __init__(self, c: Glm4vVisionConfig, dtype):
        super().__init__()
        self.cfg = c
        k = (c.temporal_patch_size, c.patch_size, c.patch_size)
        self.patch_embed = nn.Module()
        self.patch_embed.proj = nn.Conv3d(c.in_channels, c.hidden_size, k, stride=k, bias=True, dtype=dtype)
        self.embeddings = nn.Module()
        self.embeddings.position_embedding = nn.Embedding((c.image_size // c.patch_size) ** 2, c.hidden_size,
                                                          dtype=dtype)
        self.post_conv_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype)
        hd = c.hidden_size // c.num_heads
        self.rotary = _GridRotary(hd, hd // 2, 4096, 10000.0, is_neox_style=True)
        self.blocks = nn.ModuleList([_Block(c, i, dtype) for i in range(c.depth)])
        for b in self.blocks:
            b.attn.rotary = self.rotary
        self.post_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype)
        self.downsample = nn.Conv2d(c.hidden_size, c.out_hidden_size, c.spatial_merge_size, c.spatial_merge_size,
                                    dtype=dtype)
        self.merger = _Merger(c.out_hidden_size, c.intermediate_size, c.hidden_act, dtype)

    def grid_positions(self, grid_thw):
        s = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            q = torch.arange(w)[None, :].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            out.append(torch.stack([r, q]).repeat(1, t))
        return torch.cat(out, 1)

    def position_embeddings(self, pos, grid_thw):
        """Bicubic read of the learned ``side x side`` table at ``((col + 0.5) / w, (row + 0.5) / h)`` of each patch."""
        tab = self.embeddings.position_embedding.weight
        side = int(tab.shape[0] ** 0.5)
        img = tab.view(side, side, -1).permute(2, 0, 1)[None].float()
        lens = (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).tolist()
        th = torch.cat([grid_thw[i, 1].repeat(n) for i, n in enumerate(lens)]).float().to(tab.device)
        tw = torch.cat([grid_thw[i, 2].repeat(n) for i, n in enumerate(lens)]).float().to(tab.device)
        ny = ((pos[0].float() + 0.5) / th) * 2 - 1
        nx = ((pos[1].float() + 0.5) / tw) * 2 - 1
        grid = torch.stack([nx, ny], -1)[None, :, None]
        e = torch.nn.functional.grid_sample(img, grid, mode="bicubic", align_corners=False, padding_mode="border")
        return e[0, :, :, 0].t().to(tab.dtype)

    def forward(self, pixel_values, grid_thw):
        c = self.cfg
        w = self.patch_embed.proj.weight
        x = torch.nn.functional.linear(pixel_values.to(w.dtype), w.view(c.hidden_size, -1), self.patch_embed.proj.bias)
        x = self.post_conv_layernorm(x)
        pos = self.grid_positions(grid_thw).to(x.device)
        x = (x + self.position_embeddings(pos, grid_thw))[None]
        lens = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        seg = torch.repeat_interleave(torch.arange(1, lens.numel() + 1, dtype=torch.int32), lens)[None].to(x.device)
        if lens.numel() == 1:
            seg = None
        for blk in self.blocks:
            x = blk(x, pos[:, None], seg)
        x = self.post_layernorm(x[0])
        s = c.spatial_merge_size
        x = x.view(-1, s, s, x.shape[-1]).permute(0, 3, 1, 2)
        return self.merger(self.downsample(x).view(-1, c.out_hidden_size))


class _Glm4vBase(Qwen2VLForConditionalGeneration):
    # checkpoints keep the tower's QKV matrix and the language model's gate / up matrix fused
    hf_keeps_fused = ("visual.:qkv_proj", "language_model.:gate_up_proj")

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super(Qwen2VLForConditionalGeneration, self).__init__(config, dtype, param_dtype, precision, rngs)
        self.visual = Glm4vVisionTransformer(config.vision_config, self.param_dtype)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)
        self.rope_deltas = None

    def hf_rename_in(self, sd):
        sd = {(k.replace(".merger.gate_proj.", ".merger.mlp.gate_proj.").replace(".merger.up_proj.",
               ".merger.mlp.up_proj.").replace(".merger.down_proj.", ".merger.mlp.down_proj.")
               if ".visual." in k or k.startswith("visual.") else k): v for k, v in sd.items()}
        return super().hf_rename_in(sd)

    def hf_rename_out(self, sd):
        out = super().hf_rename_out(sd)
        return {(k.replace(".merger.mlp.", ".merger.") if ".visual." in k else k): v for k, v in out.items()}


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Glm4vConfig, model_type="glm4v")
class Glm4vForConditionalGeneration(_Glm4vBase):
    pass


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Glm46VConfig, model_type="glm46v")
class Glm46VForConditionalGeneration(_Glm4vBase):
    pass


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Glm4vMoeConfig, model_type="glm4v_moe")
class Glm4vMoeForConditionalGeneration(_Glm4vBase):
    hf_keeps_fused = ("visual.:qkv_proj",)
