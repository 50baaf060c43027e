"""String enums and literal sets shared across the framework.

Value sets follow easydel/infra/etils.py:79-469 so configs written for the
reference parse unchanged. Platform / backend enums are accepted for API
compatibility; this framework has exactly one device backend (sm_100a).
"""

from __future__ import annotations

import argparse
import typing as tp
from enum import Enum


class StrEnum(str, Enum):
    def __str__(self) -> str:  # noqa: D105
        return str(self.value)


class EasyDeLOptimizers(StrEnum):
    ADAFACTOR = "adafactor"
    ADAMW = "adamw"
    MARS = "mars"
    MUON = "muon"
    RMSPROP = "rmsprop"
    LION = "lion"
    SKEW = "skew"
    QUAD = "quad"


class EasyDeLSchedulers(StrEnum):
    NONE = "none"
    LINEAR = "linear"
    COSINE = "cosine"


class EasyDeLGradientCheckPointers(StrEnum):
    EVERYTHING_SAVEABLE = "everything_saveable"
    NOTHING_SAVEABLE = "nothing_saveable"
    CHECKPOINT_DOTS = "checkpoint_dots"
    CHECKPOINT_DOTS_WITH_NO_BATCH_DMIS = "checkpoint_dots_with_no_batch_dims"
    NONE = ""
    DOTS_SAVEABLE = "dots_saveable"
    DOTS_WITH_NO_BATCH_DIMS_AVAILABLE = "dots_with_no_batch_dims_saveable"
    SAVE_ANYTHING_EXCEPT_THESE_NAMES = "save_anything_except_these_names"
    SAVE_ANY_NAMES_BUT_THESE = "save_any_names_but_these"
    SAVE_ONLY_THESE_NAMES = "save_only_these_names"
    MLP_NOTSAVEABLE = "mlp_notsaveable"
    ATTN_NOTSAVEABLE = "attn_notsaveable"
    MLP_ATTN_NOTSAVEABLE = "mlp_attn_notsaveable"
    SAVE_FROM_BOTH_POLICIES = "save_from_both_policies"


class EasyDeLPlatforms(StrEnum):
    JAX = "jax"
    TRITON = "triton"
    PALLAS = "pallas"
    CUDA = "cuda"


class EasyDeLBackends(StrEnum):
    CPU = "cpu"
    GPU = "gpu"
    TPU = "tpu"
    TT = "tt"


AVAILABLE_GRADIENT_CHECKPOINTS = tp.Literal[
    "everything_saveable", "nothing_saveable", "checkpoint_dots", "checkpoint_dots_with_no_batch_dims", "",
    "dots_saveable", "dots_with_no_batch_dims_saveable", "save_anything_except_these_names",
    "save_any_names_but_these", "save_only_these_names", "mlp_notsaveable", "attn_notsaveable",
    "mlp_attn_notsaveable", "save_from_both_policies",
]
AVAILABLE_SCHEDULERS = tp.Literal["linear", "cosine", "none"]
AVAILABLE_OPTIMIZERS = tp.Literal["adafactor", "adamw", "mars", "muon", "rmsprop", "lion", "skew", "quad"]
AVAILABLE_MOE_METHODS = tp.Literal["fused_moe", "standard_moe", "dense_moe"]
AVAILABLE_ATTENTION_MECHANISMS = tp.Literal[
    "auto", "vanilla", "flash_attn2", "blocksparse", "ring", "cudnn", "blockwise", "sdpa",
    "autoregressive_decodeattn", "ragged_page_attention_v2", "ragged_page_attention_v3",
    "multi_latent_ragged_page_attention_v1", "page_attention", "unified_attention", "paged_flash_attention",
]
DEFAULT_ATTENTION_MECHANISM = "vanilla"
DEFAULT_MLA_ATTENTION_MECHANISM = "auto"
AVAILABLE_SPARSE_MODULE_TYPES = tp.Literal["bcoo", "bcsr", "coo", "csr"]

# Names a model may tag intermediate activations with; the selective
# activation-checkpoint policies refer to them (easydel/infra/etils.py:365-469).
GRADIENT_CHECKPOINT_TARGETS: tuple[str, ...] = (
    "attn_dense", "attn_key", "attn_output", "attn_qk_product", "attn_query", "attn_receptance", "attn_value",
    "attn_weights", "embeddings", "layer_output", "lm_head_output", "mlp_down", "mlp_gate", "mlp_output", "mlp_up",
    "moe_expert_output", "moe_router_logits", "normed_input", "residual", "model_output", "router_logits",
    "moe_gate", "moe_up", "moe_down", "ssm_output", "ssm_state", "conv_output", "vision_embeddings",
)


class MoEMethods(StrEnum):
    FUSED_MOE = "fused_moe"
    STANDARD_MOE = "standard_moe"
    DENSE_MOE = "dense_moe"


class AttentionMechanisms(StrEnum):
    AUTO = "auto"
    VANILLA = "vanilla"
    FLASH_ATTN2 = "flash_attn2"
    BLOCKSPARSE = "blocksparse"
    RING = "ring"
    CUDNN = "cudnn"
    BLOCKWISE = "blockwise"
    SDPA = "sdpa"
    AUTOREGRESSIVE_DECODE = "autoregressive_decodeattn"
    RAGGED_PAGE_ATTENTION_V2 = "ragged_page_attention_v2"
    RAGGED_PAGE_ATTENTION_V3 = "ragged_page_attention_v3"
    MLA_RAGGED_PAGE_ATTENTION_V1 = "multi_latent_ragged_page_attention_v1"
    PAGE_ATTENTION = "page_attention"
    UNIFIED_ATTENTION = "unified_attention"
    PAGED_FLASH_ATTENTION = "paged_flash_attention"


class StoreTupleAction(argparse.Action):
    """argparse action that parses ``1,-1,1,1,1`` into a tuple of ints."""

    def __call__(self, parser, namespace, values, option_string=None):
        try:
            setattr(namespace, self.dest, tuple(int(v) for v in str(values).split(",")))
        except ValueError as e:
            raise argparse.ArgumentTypeError(f"invalid tuple {values!r} for {option_string}") from e


def define_flags_with_default(_required_fields: list[str] | None = None, **kwargs):
    """Builds an argparse namespace from keyword defaults (mirrors easydel/infra/etils.py:472-640).

    Returns ``(args, defaults)``; tuple defaults are parsed from comma-separated strings.
    """
    parser = argparse.ArgumentParser()
    for name, default in kwargs.items():
        if isinstance(default, tuple):
            parser.add_argument(f"--{name}", action=StoreTupleAction, default=default)
        elif isinstance(default, bool):
            parser.add_argument(f"--{name}", type=lambda s: str(s).lower() in ("1", "true", "yes"), default=default)
        else:
            parser.add_argument(f"--{name}", type=type(default) if default is not None else str, default=default)
    args, _ = parser.parse_known_args()
    for f in _required_fields or []:
        if getattr(args, f) in (None, ""):
            raise ValueError(f"required flag --{f} is missing")
    return args, kwargs
