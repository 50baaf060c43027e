"""Qwen2-VL (easydel/modules/qwen2_vl): a window-free ViT over flattened ``[temporal x patch x patch]`` pixel blocks
with rotary positions on the patch grid and a 2x2 patch merger, and a Qwen2 language model whose rotary embedding
takes three position streams (temporal, height, width: mRoPE).

Inputs follow the Hugging Face processor: ``pixel_values`` ``[total_patches, C * T * P * P]`` with the patches of
every image ordered merge-block by merge-block, and ``image_grid_thw`` ``[n_images, 3]``. Text tokens advance all
three streams together; the tokens of an image keep the temporal index and spread over the merged grid's rows and
columns, and the text after it resumes at ``max(position) + 1``.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from ...layers.attention import Attention
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import PlainMLP
from ...layers.norms import LayerNorm
from ...layers.rotary import RotaryEmbedding
from .._base.families import _Renamer
from .._base.vlm import VLMConfig, VLMForConditionalGeneration


@register_config("qwen2_vl_vision")
class Qwen2VLVisionConfig(EasyDeLBaseConfig):
    model_type = "qwen2_vl_vision"
    hf_config_keys = ("depth", "embed_dim", "hidden_size", "hidden_act", "mlp_ratio", "num_heads", "in_channels",
                      "patch_size", "spatial_merge_size", "temporal_patch_size")

    def __init__(self, depth=32, embed_dim=1280, hidden_size=3584, hidden_act="quick_gelu", mlp_ratio=4, num_heads=16,
                 in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2, initializer_range=0.02,
                 **kw):
        self.depth, self.embed_dim, self.hidden_size, self.hidden_act = depth, embed_dim, hidden_size, hidden_act
        self.mlp_ratio, self.num_heads, self.in_channels, self.patch_size = mlp_ratio, num_heads, in_channels, \
            patch_size
        self.spatial_merge_size, self.temporal_patch_size = spatial_merge_size, temporal_patch_size
        self.initializer_range = initializer_range
        super().__init__(**kw)


@register_config("qwen2_vl")
class Qwen2VLConfig(VLMConfig):
    model_type = "qwen2_vl"
    vision_default, text_default = "qwen2_vl_vision", "qwen2"

    def __init__(self, vision_config=None, text_config=None, image_token_id=151655, video_token_id=151656,
                 vision_start_token_id=151652, vision_end_token_id=151653, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="qwen2_vl_vision")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type="qwen2")
            text_config.setdefault("rms_norm_eps", 1e-5)       # defaults of the multimodal text config
            text_config.setdefault("rope_theta", 1000000.0)
        kw = self._init_parts(vision_config, text_config, image_token_id, kw)
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.vision_start_token_id, self.vision_end_token_id = vision_start_token_id, vision_end_token_id
        super().__init__(**kw)


class _VisionBlock(nn.Module):
    def __init__(self, c: Qwen2VLVisionConfig, idx: int, dtype):
        super().__init__()
        d = c.embed_dim
        self.norm1 = LayerNorm(d, 1e-6, dtype=dtype)
        self.norm2 = LayerNorm(d, 1e-6, dtype=dtype)
        self.attn = Attention(d, c.num_heads, c.num_heads, d // c.num_heads, layer_idx=idx, bias=True, o_bias=True,
                              rope=None, causal=False, dtype=dtype, init_std=c.initializer_range)
        self.mlp = PlainMLP(d, int(d * c.mlp_ratio), c.hidden_act, True, dtype, c.initializer_range)

    def forward(self, x, pos, seg):
        x = x + self.attn(self.norm1(x), pos, segment_ids=seg)
        return x + self.mlp(self.norm2(x))


class _GridRotary(RotaryEmbedding):
    """Half of the rotary channels turn with the patch row, half with the column; ``positions`` ``[2, 1, T]``."""

    def forward(self, positions, q, k):
        from ...ops import reference as R

        cos, sin = self.tables(q.device)
        p = positions.reshape(2, -1)
        c = torch.cat([cos[p[0]], cos[p[1]]], -1)[:, None]
        s = torch.cat([sin[p[0]], sin[p[1]]], -1)[:, None]

        def rot(x):
            x3 = x.reshape(-1, x.shape[-2], x.shape[-1])
            return R.rotate(x3.float(), c, s, False).to(x.dtype).view(x.shape)

        return rot(q), rot(k)


class Qwen2VLVisionTransformer(nn.Module):
    def __init__(self, c: Qwen2VLVisionConfig, dtype):
        super().__init__()
        self.cfg = c
        self.patch_embed = nn.Module()
        self.patch_embed.proj = nn.Conv3d(c.in_channels, c.embed_dim, (c.temporal_patch_size, c.patch_size,
                                                                      c.patch_size),
                                          stride=(c.temporal_patch_size, c.patch_size, c.patch_size), bias=False,
                                          dtype=dtype)
        hd = c.embed_dim // c.num_heads
        # a table over hd/2 rotary channels: each of the two position streams indexes its own half of it
        self.rotary = _GridRotary(hd, hd // 2, 4096, 10000.0, is_neox_style=True)
        self.blocks = nn.ModuleList([_VisionBlock(c, i, dtype) for i in range(c.depth)])
        for b in self.blocks:
            b.attn.rotary = self.rotary
        m = c.embed_dim * c.spatial_merge_size ** 2
        self.merger = nn.Module()
        self.merger.ln_q = LayerNorm(c.embed_dim, 1e-6, dtype=dtype)
        self.merger.mlp = nn.ModuleList([ColumnParallelLinear(m, m, bias=True, dtype=dtype), nn.GELU(),
                                         ColumnParallelLinear(m, c.hidden_size, bias=True, dtype=dtype)])

    def grid_positions(self, grid_thw):
        """Row / column index of every patch, in the processor's merge-block order."""
        s = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            q = torch.arange(w)[None, :].expand(h, w).reshape(h // s, s, w // s, s).permute(0, 2, 1, 3).reshape(-1)
            out.append(torch.stack([r, q]).repeat(1, t))
        return torch.cat(out, 1)

    def forward(self, pixel_values, grid_thw):
        c = self.cfg
        w = self.patch_embed.proj.weight
        x = torch.nn.functional.linear(pixel_values.to(w.dtype), w.view(c.embed_dim, -1))[None]
        pos = self.grid_positions(grid_thw).to(x.device)[:, None]           # [2, 1, T]
        lens = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        seg = torch.repeat_interleave(torch.arange(1, lens.numel() + 1, dtype=torch.int32), lens)[None].to(x.device)
        if lens.numel() == 1:
            seg = None
        for blk in self.blocks:
            x = blk(x, pos, seg)
        m = self.merger
        y = m.ln_q(x[0]).view(-1, c.embed_dim * c.spatial_merge_size ** 2)
        for layer in m.mlp:
            y = layer(y)
        return y


def mrope_positions(input_ids, image_token_id, grid_thw, merge: int, attention_mask=None, video_token_id=None,
                    video_grid_thw=None):
    """-> ``[3, B, T]`` positions and the per-row offset ``max(position) + 1 - length`` decoding continues from.

    Image and video placeholder runs take their grids from ``grid_thw`` / ``video_grid_thw`` in order of appearance;
    a video's temporal index advances once per temporal patch."""
    B, T = input_ids.shape
    pos = torch.zeros(3, B, T, dtype=torch.long, device=input_ids.device)
    deltas = []
    grids = {image_token_id: iter(grid_thw.tolist()) if grid_thw is not None else iter(())}
    if video_token_id is not None and video_grid_thw is not None:
        grids[video_token_id] = iter(video_grid_thw.tolist())
    for b in range(B):
        keep = attention_mask[b].bool() if attention_mask is not None else torch.ones(T, dtype=torch.bool,
                                                                                        device=input_ids.device)
        ids = input_ids[b][keep].tolist()
        chunks, cur, i, n = [], 0, 0, len(ids)
        while i < n:
            if ids[i] not in grids:
                j = i
                while j < n and ids[j] not in grids:
                    j += 1
                chunks.append(torch.arange(cur, cur + j - i)[None].expand(3, -1))
                cur += j - i
                i = j
            else:
                t, h, w = next(grids[ids[i]])
                gh, gw = h // merge, w // merge
                ti = torch.arange(t)[:, None, None].expand(t, gh, gw).reshape(-1)
                hi = torch.arange(gh)[None, :, None].expand(t, gh, gw).reshape(-1)
                wi = torch.arange(gw)[None, None, :].expand(t, gh, gw).reshape(-1)
                chunks.append(torch.stack([ti, hi, wi]) + cur)
                cur += max(t, gh, gw)
                i += t * gh * gw
        p = torch.cat(chunks, 1).to(input_ids.device)
        pos[:, b, keep] = p
        deltas.append(int(p.max()) + 1 - len(ids))
    return pos, torch.tensor(deltas, device=input_ids.device)


@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen2VLConfig, model_type="qwen2_vl")
class Qwen2VLForConditionalGeneration(VLMForConditionalGeneration):
    ignored_prefixes = ()
    outer_rules = [("model.visual.", "visual."), ("model.language_model.", "language_model.model."),
                   ("lm_head.", "language_model.lm_head.")]

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.visual = Qwen2VLVisionTransformer(config.vision_config, self.param_dtype)
        self.language_model = self.build_language_model(config, dtype, param_dtype, precision, rngs)
        self.rope_deltas = None

    def _vision_renamer(self):
        return _Renamer([])

    def hf_rename_in(self, sd):
        sd = {k.replace(".attn.qkv.", ".attn.qkv_proj.").replace(".attn.proj.", ".attn.o_proj.")
              if ".visual." in k or k.startswith("visual.") else k: v for k, v in sd.items()}
        return super().hf_rename_in(sd)

    def hf_rename_out(self, sd):
        out = super().hf_rename_out(sd)
        return {k.replace(".attn.qkv_proj.", ".attn.qkv.").replace(".attn.o_proj.", ".attn.proj.")
                if ".visual." in k else k: v for k, v in out.items()}

    hf_keeps_fused = ("visual.",)

    def get_image_features(self, pixel_values, image_grid_thw=None, **_):
        return self.visual(pixel_values, image_grid_thw)

    def get_video_features(self, pixel_values_videos, video_grid_thw=None, **_):
        """Videos go through the same tower: a grid with more than one temporal patch."""
        return self.get_image_features(pixel_values_videos, image_grid_thw=video_grid_thw)

    def merge_embeddings(self, input_ids, pixel_values=None, image_features=None, pixel_values_videos=None,
                         video_grid_thw=None, **kw):
        emb = super().merge_embeddings(input_ids, pixel_values, image_features, **kw)
        if pixel_values_videos is not None:
            feats = self.get_video_features(pixel_values_videos, video_grid_thw)
            mask = input_ids == self.config.video_token_id
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} video placeholder tokens for {feats.shape[0]} video feature rows")
            emb = emb.clone()
            emb[mask] = feats.to(emb.dtype)
        return emb

    image_kwargs = ("image_grid_thw", "pixel_values_videos", "video_grid_thw")

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_grid_thw=None, pixel_values_videos=None, video_grid_thw=None, **kw):
        first = past_key_values is None or past_key_values.seq_len() == 0
        if first and pixel_values_videos is not None:
            kw.update(pixel_values_videos=pixel_values_videos, video_grid_thw=video_grid_thw)
        if position_ids is None and input_ids is not None:
            if first:
                position_ids, self.rope_deltas = mrope_positions(
                    input_ids, self.config.image_token_id, image_grid_thw if pixel_values is not None else None,
                    self.config.vision_config.spatial_merge_size, attention_mask, self.config.video_token_id,
                    video_grid_thw if pixel_values_videos is not None else None)
            else:       # decoding: all three streams continue from the prompt's last position
                B, T = input_ids.shape
                start = past_key_values.seq_len()
                base = torch.arange(start, start + T, device=input_ids.device)[None].expand(B, T)
                if self.rope_deltas is not None:
                    base = base + self.rope_deltas[:, None]
                position_ids = base[None].expand(3, B, T)
        return super().forward(input_ids=input_ids, pixel_values=pixel_values, attention_mask=attention_mask,
                               position_ids=position_ids, inputs_embeds=inputs_embeds,
                               past_key_values=past_key_values, image_grid_thw=image_grid_thw, **kw)

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        call = dict(call)
        if call.get("position_ids") is None:
            call["position_ids"], _ = mrope_positions(
                call["input_ids"], self.config.image_token_id,
                call.get("image_grid_thw") if call.get("pixel_values") is not None else None,
                self.config.vision_config.spatial_merge_size, call.get("attention_mask"), self.config.video_token_id,
                call.get("video_grid_thw") if call.get("pixel_values_videos") is not None else None)
        labels = labels.masked_fill(call["input_ids"] == self.config.video_token_id, loss_config.ignore_index)
        return super()._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)
