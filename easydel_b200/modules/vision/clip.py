"""Contrastive image-text models: CLIP and SigLIP (easydel/modules/clip, easydel/modules/siglip).

Two towers (the vision transformers of ``vit.py`` and a text transformer of the same block), pooled and projected
into a shared space. CLIP: causal text tower pooled at the end-of-text token, linear projections without bias,
softmax contrastive loss over ``exp(logit_scale) * cos``. SigLIP: bidirectional text tower pooled at the last
position through a linear head, vision tower pooled by a one-query attention head, pairwise sigmoid loss over
``exp(logit_scale) * cos + logit_bias``.
"""

from __future__ import annotations

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, LossMetrics
from ...infra.modeling_outputs import BaseModelOutputWithPooling, CLIPOutput
from ...layers.linears import ColumnParallelLinear
from ...layers.mlp import PlainMLP
from ...layers.norms import LayerNorm
from .._base.families import _Renamer
from .._base.vlm import build_sub_config
from .vit import VisionTransformer, _EncoderLayer


class _TextConfigBase(EasyDeLBaseConfig):
    hf_config_keys = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                      "max_position_embeddings", "hidden_act", "layer_norm_eps", "projection_dim", "projection_size")

    def __init__(self, vocab_size=49408, hidden_size=512, intermediate_size=2048, num_hidden_layers=12,
                 num_attention_heads=8, max_position_embeddings=77, hidden_act="quick_gelu", layer_norm_eps=1e-5,
                 initializer_range=0.02, projection_dim=512, projection_size=None, pad_token_id=1, bos_token_id=49406,
                 eos_token_id=49407, **kw):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.max_position_embeddings, self.hidden_act, self.layer_norm_eps = max_position_embeddings, hidden_act, \
            layer_norm_eps
        self.initializer_range, self.projection_dim = initializer_range, projection_dim
        self.projection_size = projection_size if projection_size is not None else hidden_size
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id, **kw)


@register_config("clip_text_model")
class CLIPTextConfig(_TextConfigBase):
    model_type = "clip_text_model"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_config("siglip_text_model")
class SiglipTextConfig(_TextConfigBase):
    model_type = "siglip_text_model"

    def __init__(self, vocab_size=32000, hidden_size=768, intermediate_size=3072, max_position_embeddings=64,
                 hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6, pad_token_id=1, bos_token_id=49406,
                 eos_token_id=49407, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, intermediate_size=intermediate_size,
                         max_position_embeddings=max_position_embeddings, hidden_act=hidden_act,
                         layer_norm_eps=layer_norm_eps, pad_token_id=pad_token_id, bos_token_id=bos_token_id,
                         eos_token_id=eos_token_id, **kw)


class TextTransformer(nn.Module):
    def __init__(self, c, dtype, causal: bool, head: bool):
        super().__init__()
        self.cfg, self.causal = c, causal
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype)
        self.position_embedding = nn.Embedding(c.max_position_embeddings, c.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([_EncoderLayer(c, i, dtype, causal=causal) for i in range(c.num_hidden_layers)])
        self.final_layer_norm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.head = ColumnParallelLinear(c.hidden_size, c.projection_size, bias=True, dtype=dtype) if head else None

    def forward(self, input_ids, attention_mask=None, output_hidden_states: bool = False):
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device)[None].expand(B, T)
        x = self.token_embedding(input_ids) + self.position_embedding(pos)
        seg = None
        if attention_mask is not None and not bool(attention_mask.all()):
            seg = attention_mask.to(torch.int32)
        hs = [x] if output_hidden_states else None
        for layer in self.layers:
            x = layer(x, pos, seg)
            if hs is not None:
                hs.append(x)
        x = self.final_layer_norm(x)
        if self.head is not None:                       # SigLIP: the last position, through a linear head
            pooled = self.head(x[:, -1])
        else:                                           # CLIP: the (first) end-of-text token
            eos = self.cfg.eos_token_id
            idx = input_ids.argmax(-1) if eos == 2 else (input_ids == eos).int().argmax(-1)
            pooled = x[torch.arange(B, device=x.device), idx]
        return BaseModelOutputWithPooling(last_hidden_state=x, pooler_output=pooled,
                                          hidden_states=tuple(hs) if hs else None)


class SiglipPoolingHead(nn.Module):
    """One learned query attends over the patch tokens; LayerNorm + MLP residual on the result."""

    def __init__(self, c, dtype):
        super().__init__()
        self.heads = c.num_attention_heads
        self.probe = nn.Parameter(torch.randn(1, 1, c.hidden_size, dtype=dtype) * 0.02)
        self.attention = nn.Module()
        self.attention.in_proj_weight = nn.Parameter(torch.randn(3 * c.hidden_size, c.hidden_size, dtype=dtype) * 0.02)
        self.attention.in_proj_bias = nn.Parameter(torch.zeros(3 * c.hidden_size, dtype=dtype))
        self.attention.out_proj = ColumnParallelLinear(c.hidden_size, c.hidden_size, bias=True, dtype=dtype)
        self.layernorm = LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype)
        self.mlp = PlainMLP(c.hidden_size, c.intermediate_size, c.hidden_act, True, dtype, 0.02)

    def forward(self, x):
        B, T, D = x.shape
        h, hd = self.heads, D // self.heads
        wq, wk, wv = self.attention.in_proj_weight.chunk(3, 0)
        bq, bk, bv = self.attention.in_proj_bias.chunk(3, 0)
        q = torch.nn.functional.linear(self.probe.expand(B, 1, D), wq, bq).view(B, 1, h, hd)
        k = torch.nn.functional.linear(x, wk, bk).view(B, T, h, hd)
        v = torch.nn.functional.linear(x, wv, bv).view(B, T, h, hd)
        from ...ops import reference as R

        o = R.attention(q, k, v, causal=False).reshape(B, 1, D)      # a single query row: not a kernel-sized problem
        o = self.attention.out_proj(o)
        o = o + self.mlp(self.layernorm(o))
        return o[:, 0]


class _VisionWithPool(nn.Module):
    def __init__(self, c, dtype, pool_head: bool):
        super().__init__()
        self.body = VisionTransformer(c, dtype)
        self.head = SiglipPoolingHead(c, dtype) if pool_head else None
        self.use_cls = c.use_class_token

    def forward(self, pixel_values, output_hidden_states=False):
        out = self.body(pixel_values, output_hidden_states)
        x = out.last_hidden_state
        if self.head is not None:
            pooled = self.head(x)
        else:       # CLIP pools the class token (the tower's final LayerNorm applies to every token here)
            pooled = x[:, 0]
        return BaseModelOutputWithPooling(last_hidden_state=x, pooler_output=pooled, hidden_states=out.hidden_states)


class _DualConfig(EasyDeLBaseConfig):
    text_default, vision_default = "clip_text_model", "clip_vision_model"

    def __init__(self, text_config=None, vision_config=None, projection_dim=512, logit_scale_init_value=2.6592,
                 **kw):
        self.text_config = build_sub_config(text_config, self.text_default)
        self.vision_config = build_sub_config(vision_config, self.vision_default)
        self.projection_dim, self.logit_scale_init_value = projection_dim, logit_scale_init_value
        super().__init__(**kw)

    def to_dict(self):
        d = super().to_dict()
        d["text_config"], d["vision_config"] = self.text_config.to_dict(), self.vision_config.to_dict()
        return d


@register_config("clip")
class CLIPConfig(_DualConfig):
    model_type = "clip"

    def __init__(self, **kw):
        super().__init__(**kw)


@register_config("siglip")
class SiglipConfig(_DualConfig):
    model_type = "siglip"
    text_default, vision_default = "siglip_text_model", "siglip_vision_model"

    def __init__(self, **kw):
        super().__init__(**kw)


_CLIP_REN = _Renamer([
    ("vision_model.head.", "vision_model.head."),
    ("vision_model.encoder.layers.", "vision_model.body.layers."),
    ("vision_model.embeddings.class_embedding", "vision_model.body.class_embedding"),
    ("vision_model.embeddings.patch_embedding.", "vision_model.body.patch_embedding."),
    ("vision_model.embeddings.position_embedding.", "vision_model.body.position_embedding."),
    ("vision_model.pre_layrnorm.", "vision_model.body.pre_layrnorm."),
    ("vision_model.post_layernorm.", "vision_model.body.post_layernorm."),
    ("text_model.encoder.layers.", "text_model.layers."),
    ("text_model.embeddings.token_embedding.", "text_model.token_embedding."),
    ("text_model.embeddings.position_embedding.", "text_model.position_embedding."),
    (".self_attn.out_proj.", ".self_attn.o_proj."),
])


class _DualBase(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def hf_rename_in(self, sd):
        return _CLIP_REN.to_internal(self, {k: v for k, v in sd.items() if not k.endswith("position_ids")})

    def hf_rename_out(self, sd):
        return _CLIP_REN.to_hf(self, sd)

    def get_text_features(self, input_ids, attention_mask=None):
        return self._project_text(self.text_model(input_ids, attention_mask).pooler_output)

    def get_image_features(self, pixel_values):
        return self._project_image(self.vision_model(pixel_values).pooler_output)

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, return_loss: bool = False, **_):
        t_out = self.text_model(input_ids, attention_mask)
        v_out = self.vision_model(pixel_values)
        te = self._project_text(t_out.pooler_output)
        ie = self._project_image(v_out.pooler_output)
        te = te / te.norm(dim=-1, keepdim=True)
        ie = ie / ie.norm(dim=-1, keepdim=True)
        lt = self._logits(te, ie)
        loss = self.contrastive_loss(lt) if return_loss else None
        return CLIPOutput(loss=loss, logits_per_image=lt.t(), logits_per_text=lt, text_embeds=te, image_embeds=ie,
                          text_model_output=t_out, vision_model_output=v_out)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        out = self(return_loss=True, **{k: v for k, v in call.items() if k in ("input_ids", "pixel_values",
                                                                                 "attention_mask")})
        return out, LossMetrics(loss=out.loss * loss_scale)


@register_module(TaskType.ZERO_SHOT_IMAGE_CLASSIFICATION, config=CLIPConfig, model_type="clip")
class CLIPModel(_DualBase):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.text_model = TextTransformer(config.text_config, pd, causal=True, head=False)
        self.vision_model = _VisionWithPool(config.vision_config, pd, pool_head=False)
        self.visual_projection = ColumnParallelLinear(config.vision_config.hidden_size, config.projection_dim,
                                                      bias=False, dtype=pd)
        self.text_projection = ColumnParallelLinear(config.text_config.hidden_size, config.projection_dim, bias=False,
                                                    dtype=pd)
        self.logit_scale = nn.Parameter(torch.tensor(config.logit_scale_init_value, dtype=pd))

    def _project_text(self, x):
        return self.text_projection(x)

    def _project_image(self, x):
        return self.visual_projection(x)

    def _logits(self, te, ie):
        return te @ ie.t() * self.logit_scale.exp()

    @staticmethod
    def contrastive_loss(logits_per_text):
        n = logits_per_text.shape[0]
        tgt = torch.arange(n, device=logits_per_text.device)
        ce = torch.nn.functional.cross_entropy
        return 0.5 * (ce(logits_per_text.float(), tgt) + ce(logits_per_text.t().float(), tgt))


@register_module(TaskType.ZERO_SHOT_IMAGE_CLASSIFICATION, config=SiglipConfig, model_type="siglip")
class SiglipModel(_DualBase):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.text_model = TextTransformer(config.text_config, pd, causal=False, head=True)
        self.vision_model = _VisionWithPool(config.vision_config, pd, pool_head=True)
        self.logit_scale = nn.Parameter(torch.zeros(1, dtype=pd))
        self.logit_bias = nn.Parameter(torch.zeros(1, dtype=pd))

    def _project_text(self, x):
        return x

    def _project_image(self, x):
        return x

    def _logits(self, te, ie):
        return te @ ie.t() * self.logit_scale.exp() + self.logit_bias

    @staticmethod
    def contrastive_loss(logits_per_text):
        n = logits_per_text.shape[0]
        sign = 2 * torch.eye(n, device=logits_per_text.device) - 1
        return -torch.nn.functional.logsigmoid(sign * logits_per_text.float()).sum(-1).mean()
