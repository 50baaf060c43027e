"""Kimi-VL (easydel/modules/kimi_vl/modeling_kimi_vl.py): the MoonViT native-resolution vision encoder, a two-layer
projector over 2x2 merged patches, and a DeepSeek-V3 language model.

MoonViT packs the patches of every image into one sequence ``[total_patches, hidden]``:

* patch embedding = a ``patch x patch`` convolution plus a learned ``64 x 64`` position table that is resized
  (bicubic, anti-aliased) to each image's ``h x w`` patch grid;
* pre-LayerNorm blocks whose attention stays inside an image (one segment per image) and rotates query / key channel
  pairs ``(2j, 2j+1)`` by the patch column for even ``j`` and by the patch row for odd ``j``, both with the frequency
  ``theta ** (-4 * (j // 2) / head_dim)``;
* a final LayerNorm, then the ``merge_h x merge_w`` neighbours of the grid are gathered into one row.

The projector normalises every patch, concatenates the merged neighbours and applies ``Linear - GELU - Linear``. The
rows replace the ``media_placeholder_token_id`` embeddings of the language model. Parameter names follow the
published checkpoints (``vision_tower.encoder.blocks.N.wqkv`` ...), so no vision rename table is needed.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from ...ops import functional as F
from ...ops import reference as R
from .._base.vlm import VLMConfig, VLMForConditionalGeneration


@register_config("moonvit")
class MoonViTConfig(EasyDeLBaseConfig):
    model_type = "moonvit"
    hf_config_keys = ("patch_size", "init_pos_emb_height", "init_pos_emb_width", "num_attention_heads",
                      "num_hidden_layers", "hidden_size", "intermediate_size", "merge_kernel_size")

    def __init__(self, patch_size=14, init_pos_emb_height=64, init_pos_emb_width=64, num_attention_heads=16,
                 num_hidden_layers=27, hidden_size=1152, intermediate_size=4304, merge_kernel_size=(2, 2), **kw):
        self.patch_size = patch_size
        self.init_pos_emb_height, self.init_pos_emb_width = init_pos_emb_height, init_pos_emb_width
        self.num_attention_heads, self.num_hidden_layers = num_attention_heads, num_hidden_layers
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.merge_kernel_size = tuple(merge_kernel_size)
        super().__init__(**kw)


@register_config("kimi_vl")
class KimiVLConfig(VLMConfig):
    model_type = "kimi_vl"
    vision_default, text_default = "moonvit", "deepseek_v3"

    def __init__(self, vision_config=None, text_config=None, ignore_index=-100, media_placeholder_token_id=163605,
                 pad_token_id=0, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="moonvit")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type="deepseek_v3")
        kw = self._init_parts(vision_config, text_config, media_placeholder_token_id, kw)
        self.ignore_index, self.media_placeholder_token_id = ignore_index, media_placeholder_token_id
        super().__init__(pad_token_id=pad_token_id, **kw)


class _PatchEmbed(nn.Module):
    def __init__(self, c: MoonViTConfig, dtype):
        super().__init__()
        self.proj = nn.Conv2d(3, c.hidden_size, c.patch_size, c.patch_size, dtype=dtype)
        self.pos_emb = nn.Module()
        self.pos_emb.weight = nn.Parameter(torch.randn(c.init_pos_emb_height, c.init_pos_emb_width, c.hidden_size,
                                                       dtype=dtype) * 0.02)

    def position_table(self, h: int, w: int) -> torch.Tensor:
        tab = self.pos_emb.weight
        if (h, w) == tuple(tab.shape[:2]):
            return tab.reshape(h * w, -1)
        img = tab.permute(2, 0, 1)[None].float()
        out = torch.nn.functional.interpolate(img, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
        return out[0].permute(1, 2, 0).reshape(h * w, -1).to(tab.dtype)

    def forward(self, pixel_values, grid_hws):
        w = self.proj.weight
        if pixel_values.ndim == 4 and pixel_values.shape[1] != w.shape[1]:      # channels-last patches
            pixel_values = pixel_values.permute(0, 3, 1, 2)
        x = torch.nn.functional.linear(pixel_values.reshape(pixel_values.shape[0], -1).to(w.dtype),
                                       w.view(w.shape[0], -1), self.proj.bias)
        pos = torch.cat([self.position_table(int(h), int(w_)) for h, w_ in grid_hws.tolist()], 0)
        return x + pos


def grid_rope_angles(grid_hws: torch.Tensor, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """``[total_patches, head_dim / 2]`` rotation angles: pair ``2i`` follows the column, pair ``2i + 1`` the row."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 4, dtype=torch.float32)[: head_dim // 4] / head_dim))
    out = []
    for h, w in grid_hws.tolist():
        ys = torch.arange(h, dtype=torch.float32)[:, None].expand(h, w).reshape(-1)
        xs = torch.arange(w, dtype=torch.float32)[None, :].expand(h, w).reshape(-1)
        out.append(torch.stack([xs[:, None] * freqs, ys[:, None] * freqs], -1).reshape(h * w, -1))
    return torch.cat(out, 0)


class _MLP2(nn.Module):
    def __init__(self, d, inner, dtype):
        super().__init__()
        self.fc0 = nn.Linear(d, inner, dtype=dtype)
        self.fc1 = nn.Linear(inner, d, dtype=dtype)

    def forward(self, x):
        return F.linear(torch.nn.functional.gelu(F.linear(x, self.fc0.weight, self.fc0.bias), approximate="tanh"),
                        self.fc1.weight, self.fc1.bias)


class _MoonBlock(nn.Module):
    def __init__(self, c: MoonViTConfig, dtype):
        super().__init__()
        d = c.hidden_size
        self.heads = c.num_attention_heads
        self.norm0 = nn.LayerNorm(d, eps=1e-5, dtype=dtype)
        self.norm1 = nn.LayerNorm(d, eps=1e-5, dtype=dtype)
        self.wqkv = nn.Linear(d, 3 * d, dtype=dtype)
        self.wo = nn.Linear(d, d, dtype=dtype)
        self.mlp = _MLP2(d, c.intermediate_size, dtype)

    def forward(self, x, cos, sin, seg):
        T, d = x.shape
        qkv = F.linear(self.norm0(x), self.wqkv.weight, self.wqkv.bias).view(T, 3, self.heads, d // self.heads)
        q = R.rotate(qkv[:, 0].float(), cos, sin, True).to(x.dtype)
        k = R.rotate(qkv[:, 1].float(), cos, sin, True).to(x.dtype)
        o = F.attention(q[None], k[None], qkv[:, 2][None].contiguous(), causal=False, segment_ids=seg)
        x = x + F.linear(o.reshape(T, d), self.wo.weight, self.wo.bias)
        return x + self.mlp(self.norm1(x))


class MoonVitPretrainedModel(nn.Module):
    """``pixel_values`` ``[total_patches, 3, P, P]`` + ``grid_hws`` ``[n_images, 2]`` -> per-image merged features
    ``[h/mh * w/mw, mh * mw, hidden]``."""

    def __init__(self, c: MoonViTConfig, dtype):
        super().__init__()
        self.cfg = c
        self.patch_embed = _PatchEmbed(c, dtype)
        self.encoder = nn.Module()
        self.encoder.blocks = nn.ModuleList([_MoonBlock(c, dtype) for _ in range(c.num_hidden_layers)])
        self.encoder.final_layernorm = nn.LayerNorm(c.hidden_size, eps=1e-5, dtype=dtype)

    def forward(self, pixel_values, grid_hws):
        c = self.cfg
        grid_hws = grid_hws.cpu()
        x = self.patch_embed(pixel_values, grid_hws)
        ang = grid_rope_angles(grid_hws, c.hidden_size // c.num_attention_heads).to(x.device)
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]
        lens = grid_hws[:, 0] * grid_hws[:, 1]
        seg = None
        if lens.numel() > 1:
            seg = torch.repeat_interleave(torch.arange(1, lens.numel() + 1, dtype=torch.int32), lens)[None].to(x.device)
        for blk in self.encoder.blocks:
            x = blk(x, cos, sin, seg)
        x = self.encoder.final_layernorm(x)
        mh, mw = c.merge_kernel_size
        out, at = [], 0
        for h, w in grid_hws.tolist():
            piece = x[at:at + h * w].view(h // mh, mh, w // mw, mw, -1).permute(0, 2, 1, 3, 4)
            out.append(piece.reshape((h // mh) * (w // mw), mh * mw, -1))
            at += h * w
        return out


class KimiVLMultiModalProjector(nn.Module):
    def __init__(self, config: KimiVLConfig, dtype):
        super().__init__()
        v = config.vision_config
        self.inner = v.hidden_size * v.merge_kernel_size[0] * v.merge_kernel_size[1]
        self.pre_norm = nn.LayerNorm(v.hidden_size, eps=1e-5, dtype=dtype)
        self.linear_1 = nn.Linear(self.inner, self.inner, dtype=dtype)
        self.linear_2 = nn.Linear(self.inner, config.text_config.hidden_size, dtype=dtype)

    def forward(self, image_features):
        x = self.pre_norm(torch.cat(image_features, 0)).view(-1, self.inner)
        x = torch.nn.functional.gelu(F.linear(x, self.linear_1.weight, self.linear_1.bias))
        return F.linear(x, self.linear_2.weight, self.linear_2.bias)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=KimiVLConfig, model_type="kimi_vl")
class KimiVLForConditionalGeneration(VLMForConditionalGeneration):
    """Checkpoints store ``vision_tower.*``, ``multi_modal_projector.*`` and ``language_model.{model,lm_head}.*`` at
    the top level, which are this module's own names: only the language model's table applies."""

    outer_rules = []
    ignored_prefixes = ()
    image_kwargs = ("image_grid_hws",)

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.vision_tower = MoonVitPretrainedModel(config.vision_config, self.param_dtype)
        self.multi_modal_projector = KimiVLMultiModalProjector(config, self.param_dtype)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)

    def _vision_renamer(self):
        from .._base.families import _Renamer

        return _Renamer([])

    def get_image_features(self, pixel_values, image_grid_hws=None, **kw):
        if image_grid_hws is None:
            raise ValueError("Kimi-VL needs image_grid_hws ([n_images, 2] patch-grid sizes) with pixel_values")
        w = self.vision_tower.patch_embed.proj.weight
        return self.multi_modal_projector(self.vision_tower(pixel_values.to(w.dtype), image_grid_hws))

    def get_vision_tower(self):
        return self.vision_tower

    def get_projector(self):
        return self.multi_modal_projector

    def get_language_model(self):
        return self.language_model
