"""Table-driven construction of decoder-only model families.

``define_family`` creates, registers and returns the config class and the ``Model`` /
``ForCausalLM`` / ``ForSequenceClassification`` classes of one family from:

* the Hugging Face style config defaults of that family,
* a function mapping a config to an :class:`ArchSpec`,
* optional weight-name rules translating between Hugging Face checkpoint names and this
  framework's module tree (plain string substitutions applied to every key, plus optional
  tensor-level hooks for fused / re-ordered projections).

The reference writes one ``modeling_<family>.py`` per family (easydel/modules/*, 75 directories);
here the shared structure lives in ``decoder.py`` and a family is a page of declarative data.
"""

from __future__ import annotations

import re
import typing as tp

import torch

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from .decoder import ArchSpec, DecoderForCausalLM, DecoderForSequenceClassification, DecoderModel, MoESpec

_HF_KEYS = ("pad_token_id", "bos_token_id", "eos_token_id", "tie_word_embeddings")


def make_config(model_type: str, defaults: dict, post: tp.Callable | None = None, name: str | None = None,
                attribute_map: dict | None = None):
    defaults = dict(defaults)

    class _Config(EasyDeLBaseConfig):
        def __init__(self, **kw):
            rp = kw.get("rope_parameters")
            if isinstance(rp, dict) and "rope_type" in rp or isinstance(rp, dict) and "rope_theta" in rp:
                # newer checkpoints keep the base frequency, the rotated fraction and the scaling recipe in one
                # dict; spread it over the fields the specs read unless those were given explicitly
                rest = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
                if "rope_theta" in rp:
                    kw.setdefault("rope_theta", rp["rope_theta"])
                if "partial_rotary_factor" in rp and "partial_rotary_factor" in defaults:
                    kw.setdefault("partial_rotary_factor", rp["partial_rotary_factor"])
                if kw.get("rope_scaling") is None and (rest.get("rope_type", "default") != "default"
                                                       or rest.get("mrope_section")):
                    kw["rope_scaling"] = rest
            for k, v in defaults.items():
                if k in _HF_KEYS:
                    kw.setdefault(k, v)
                    continue
                setattr(self, k, kw.pop(k, v))
            if getattr(self, "num_key_value_heads", 0) is None:
                self.num_key_value_heads = self.num_attention_heads
            if hasattr(self, "head_dim") and self.head_dim is None:
                self.head_dim = self.hidden_size // self.num_attention_heads
            if post is not None:
                post(self)
            super().__init__(**kw)

    _Config.model_type = model_type
    if attribute_map:
        _Config.attribute_map = dict(attribute_map)
    _Config.hf_config_keys = tuple(defaults)
    _Config.__name__ = _Config.__qualname__ = name or (model_type.title().replace("_", "") + "Config")
    return register_config(model_type)(_Config)


def rope_args(c, head_dim: int, partial: float = 1.0, neox: bool = True, theta_attr: str = "rope_theta",
              scaling_attr: str = "rope_scaling") -> dict:
    scaling = getattr(c, scaling_attr, None)
    params = getattr(c, "rope_parameters", None)
    theta = getattr(c, theta_attr, None)
    if isinstance(params, dict):
        theta = theta or params.get("rope_theta")
        if scaling is None and params.get("rope_type", "default") != "default":
            scaling = {k: v for k, v in params.items() if k != "rope_theta"}
    if isinstance(scaling, dict) and (scaling.get("rope_type") or scaling.get("type")) in (None, "default") \
            and not scaling.get("mrope_section"):
        scaling = None
    return dict(rotary_dim=head_dim, max_position=c.max_position_embeddings, base=theta or 10000.0,
                is_neox_style=neox, rope_scaling=scaling, partial_rotary_factor=partial)


def base_spec(c, **over) -> ArchSpec:
    """Reads the field names shared by the Llama-like configs."""
    hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
    kw = dict(
        hidden_size=c.hidden_size, num_layers=c.num_hidden_layers, num_heads=c.num_attention_heads,
        num_kv_heads=getattr(c, "num_key_value_heads", None) or c.num_attention_heads, head_dim=hd,
        intermediate_size=getattr(c, "intermediate_size", 4 * c.hidden_size), vocab_size=c.vocab_size,
        max_position=c.max_position_embeddings, norm="rms", norm_eps=getattr(c, "rms_norm_eps", 1e-6),
        act=getattr(c, "hidden_act", "silu"), mlp="gated", mlp_bias=getattr(c, "mlp_bias", False),
        attn_bias=getattr(c, "attention_bias", False), o_bias=getattr(c, "attention_bias", False),
        rope=rope_args(c, hd), tie_embeddings=getattr(c, "tie_word_embeddings", False),
        init_std=getattr(c, "initializer_range", 0.02))
    kw.update(over)
    return ArchSpec(**kw)


class _Renamer:
    """Bidirectional key substitutions: ``rules`` is a list of (hf_fragment, internal_fragment), or a
    function of the model returning one.

    A key is rewritten in one left-to-right pass; where several fragments match at the same position the
    one listed first wins, and replaced text is never rescanned, so a specific rule placed before a general
    one (``model.decoder.final_layer_norm.`` before ``model.decoder.``) behaves the same in both directions.
    """

    def __init__(self, rules, tensor_in=None, tensor_out=None):
        self.rules, self.tensor_in, self.tensor_out = rules, tensor_in, tensor_out

    def _table(self, model, inverse: bool):
        rules = self.rules(model) if callable(self.rules) else self.rules
        pairs = [(b, a) if inverse else (a, b) for a, b in rules]
        if not pairs:
            return None, {}
        return re.compile("|".join(re.escape(a) for a, _ in pairs)), dict(pairs)

    @staticmethod
    def _apply(sd, pattern, table):
        if pattern is None:
            return dict(sd)
        return {pattern.sub(lambda m: table[m.group(0)], k): v for k, v in sd.items()}

    def to_internal(self, model, sd: dict) -> dict:
        if self.tensor_in is not None:
            sd = self.tensor_in(model, sd)
        return self._apply(sd, *self._table(model, False))

    def to_hf(self, model, sd: dict) -> dict:
        out = self._apply(sd, *self._table(model, True))
        if self.tensor_out is not None:
            out = self.tensor_out(model, out)
        return out


def define_family(model_type: str, defaults: dict, spec_fn: tp.Callable[[tp.Any], ArchSpec], *,
                  class_prefix: str | None = None, rules: tp.Sequence[tuple[str, str]] = (), tensor_in=None,
                  tensor_out=None, config_post=None, hf_keeps_fused: tuple[str, ...] = (),
                  layernorm_names: list[str] | None = None, with_classifier: bool = True,
                  attribute_map: dict | None = None):
    prefix = class_prefix or model_type.title().replace("_", "")
    cfg = make_config(model_type, defaults, config_post, prefix + "Config", attribute_map)
    ren = _Renamer(rules, tensor_in, tensor_out) if (rules or tensor_in or tensor_out) else None

    def hooks(ns: dict) -> dict:
        ns["hf_keeps_fused"] = tuple(hf_keeps_fused)
        if ren is not None:
            ns["hf_rename_in"] = lambda self, sd: ren.to_internal(self, sd)
            ns["hf_rename_out"] = lambda self, sd: ren.to_hf(self, sd)
        return ns

    model = type(prefix + "Model", (DecoderModel,), hooks({"spec_fn": staticmethod(spec_fn)}))
    model = register_module(TaskType.BASE_MODULE, config=cfg, model_type=model_type,
                            layernorm_names=layernorm_names)(model)
    lm = type(prefix + "ForCausalLM", (DecoderForCausalLM,), hooks({"backbone_cls": model}))
    lm = register_module(TaskType.CAUSAL_LM, config=cfg, model_type=model_type, layernorm_names=layernorm_names)(lm)
    out = {prefix + "Config": cfg, prefix + "Model": model, prefix + "ForCausalLM": lm}
    if with_classifier:
        cl = type(prefix + "ForSequenceClassification", (DecoderForSequenceClassification,),
                  hooks({"backbone_cls": model}))
        cl = register_module(TaskType.SEQUENCE_CLASSIFICATION, config=cfg, model_type=model_type,
                             layernorm_names=layernorm_names)(cl)
        out[prefix + "ForSequenceClassification"] = cl
    return out


def moe_spec(c, *, num_experts, top_k, intermediate, norm_topk=True, shared=0, shared_gate=False, layers=None,
             aux_coef=0.0, **kw) -> MoESpec:
    return MoESpec(num_experts=num_experts, top_k=top_k, intermediate_size=intermediate, norm_topk_prob=norm_topk,
                   shared_intermediate_size=shared, shared_gate=shared_gate, layers=layers, aux_loss_coef=aux_coef,
                   **kw)
