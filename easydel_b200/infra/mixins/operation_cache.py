"""Which cache every layer of a model needs, discovered from the built module tree.

Role of easydel/infra/mixins/operation_cache.py:58-1150 (``LayerOperationInfo``, ``OperationsCacheInfo``,
``OperationCacheMixin``). The reference asks its operation registry which cache types each attention operation
can run on; here an operation is one of this library's kernels, and what a layer needs follows from what the
layer *is*: softmax attention keeps keys / values (dense cache for ``generate``, 128-token pages for the
engine), latent attention keeps one compressed row per token, recurrent mixers keep a fixed-size state, and a
sliding-window or chunked-local layer only ever needs the pages inside its window.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field


class CacheType(enum.Flag):
    TRANSFORMER = enum.auto()     # dense [B, T, Hkv, D] keys / values (model.generate)
    RAGGED_PAGES = enum.auto()    # 128-token pages addressed through page tables (eSurge)
    LATENT_PAGES = enum.auto()    # pages of [latent | rotary key] rows (multi-head latent attention)
    RECURRENT = enum.auto()       # fixed-size state per sequence (SSM, delta rule, lightning attention)
    HYBRID = enum.auto()          # pages for the attention layers plus per-slot states for the recurrent ones

    @classmethod
    def any(cls) -> "CacheType":
        return cls.TRANSFORMER | cls.RAGGED_PAGES | cls.LATENT_PAGES | cls.RECURRENT | cls.HYBRID


class ExecutionMode(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    MIXED = "mixed"


@dataclass
class LayerOperationInfo:
    layer_index: int
    layer_type: str                       # full_attention | sliding_attention | chunked_attention | latent_attention |
    operation_name: str                   # linear_attention | ssm | lightning_attention | parallel_hybrid
    decode_operation_name: str | None = None
    slot: int | None = None               # distinguishes several cache-bearing operations of one layer
    supported_cache_types: CacheType = field(default_factory=CacheType.any)
    requires_kv_cache: bool = True
    requires_state_cache: bool = False
    sliding_window: int | None = None
    chunk_size: int | None = None
    num_kv_heads: int = 0
    head_dim: int = 0

    @property
    def is_attention_layer(self) -> bool:
        return self.requires_kv_cache

    @property
    def is_recurrent_layer(self) -> bool:
        return self.requires_state_cache and not self.requires_kv_cache

    @property
    def has_separate_decode(self) -> bool:
        return self.decode_operation_name is not None and self.decode_operation_name != self.operation_name

    def tokens_kept(self, context: int) -> int:
        """How many tokens of a ``context``-token sequence this layer has to keep keys / values for."""
        if not self.requires_kv_cache:
            return 0
        if self.sliding_window:
            return min(context, self.sliding_window)
        if self.chunk_size:
            return min(context, self.chunk_size)
        return context


@dataclass
class OperationsCacheInfo:
    layers: list[LayerOperationInfo] = field(default_factory=list)
    prefill_operation: str = ""
    decode_operation: str = ""
    combined_cache_types: CacheType = field(default_factory=CacheType.any)
    is_hybrid_model: bool = False
    supports_ragged_pages: bool = False
    supports_transformer_cache: bool = False
    requires_hybrid_cache: bool = False
    requires_state_management: bool = False
    has_separate_decode_ops: bool = False

    @property
    def requires_ragged_pages(self) -> bool:
        return self.supports_ragged_pages

    @property
    def requires_transformer_cache(self) -> bool:
        return self.supports_transformer_cache

    @property
    def num_attention_layers(self) -> int:
        return sum(1 for l in self.layers if l.is_attention_layer)

    @property
    def num_recurrent_layers(self) -> int:
        return sum(1 for l in self.layers if l.requires_state_cache)

    @property
    def attention_ratio(self) -> float:
        return self.num_attention_layers / len(self.layers) if self.layers else 0.0

    def get_recommended_cache_type(self) -> str:
        if self.requires_hybrid_cache or self.requires_state_management:
            return "hybrid"
        if self.supports_transformer_cache:
            return "transformer"
        if self.supports_ragged_pages:
            return "ragged"
        return "transformer"

    def get_layer_by_index(self, index: int) -> LayerOperationInfo | None:
        return next((l for l in self.layers if l.layer_index == index), None)

    def get_layers_by_index(self, index: int) -> list[LayerOperationInfo]:
        return [l for l in self.layers if l.layer_index == index]

    def page_groups(self) -> list[dict]:
        """Layers that can share one page table: same retention rule (full context, a window, a chunk).
        ``[{"kind", "window", "layers"}]``, the full-attention group first."""
        groups: dict[tuple, dict] = {}
        for l in self.layers:
            if not l.requires_kv_cache:
                continue
            if l.sliding_window:
                key = ("sliding", int(l.sliding_window))
            elif l.chunk_size:
                key = ("chunked", int(l.chunk_size))
            else:
                key = ("full", 0)
            g = groups.setdefault(key, {"kind": key[0], "window": key[1], "layers": []})
            g["layers"].append(l.layer_index)
        return sorted(groups.values(), key=lambda g: (g["kind"] != "full", g["window"]))

    def kv_bytes_per_token(self, context: int, element_size: int = 2) -> float:
        """Average bytes of keys + values kept per token of a ``context``-token sequence, over all layers."""
        total = 0
        for l in self.layers:
            total += 2 * l.tokens_kept(context) * l.num_kv_heads * l.head_dim * element_size
        return total / max(1, context)


class OperationCacheMixin:
    """``get_operations_cache_info`` and friends for every model built from decoder layers."""

    def _decoder_layers(self):
        backbone = getattr(self, "language_model", self)
        backbone = getattr(backbone, "model", backbone)
        return list(getattr(backbone, "layers", ()))

    def get_operations_cache_info(self, mode: ExecutionMode = ExecutionMode.MIXED) -> OperationsCacheInfo:
        infos: list[LayerOperationInfo] = []
        for i, layer in enumerate(self._decoder_layers()):
            infos.extend(_describe_layer(i, layer))
        return _combine(infos)

    def get_operations_cache_info_dynamic(self, mode: ExecutionMode = ExecutionMode.MIXED) -> OperationsCacheInfo:
        return self.get_operations_cache_info(mode)

    def get_layer_cache_requirements(self, layer_index: int) -> LayerOperationInfo | None:
        return self.get_operations_cache_info().get_layer_by_index(layer_index)

    def get_required_cache_class(self) -> type:
        """The cache class ``generate`` should build (the engine always builds the paged one)."""
        from ...caching import transformer as T

        return T.TransformerCache

    def get_operations_cache_view(self) -> dict[int, type]:
        """Layer index -> class of the per-layer view the paged engine cache hands that layer."""
        from ...caching import paged as P

        out = {}
        for l in self.get_operations_cache_info().layers:
            if l.layer_type == "latent_attention":
                out[l.layer_index] = P.PagedLatentView
            elif l.requires_kv_cache:
                out[l.layer_index] = P.PagedLayerView
            else:
                out[l.layer_index] = P.PagedLinearState
        return out

    def get_operations_cache_info_by_slot(self) -> dict[int, dict[int, LayerOperationInfo]]:
        out: dict[int, dict[int, LayerOperationInfo]] = {}
        for l in self.get_operations_cache_info().layers:
            out.setdefault(l.layer_index, {})[l.slot or 0] = l
        return out

    def get_unique_cache_view_classes(self) -> set[type]:
        return set(self.get_operations_cache_view().values())


def _describe_layer(i: int, layer) -> list[LayerOperationInfo]:
    out: list[LayerOperationInfo] = []
    ltype = getattr(layer, "ltype", "full")
    spec = getattr(layer, "spec", None)
    attn = getattr(layer, "self_attn", None)
    paged = CacheType.TRANSFORMER | CacheType.RAGGED_PAGES | CacheType.HYBRID
    if ltype == "lightning":
        out.append(LayerOperationInfo(i, "lightning_attention", "lightning_attention", None, None,
                                      CacheType.RECURRENT | CacheType.HYBRID, False, True))
        return out
    if getattr(layer, "is_linear", False):
        name = "kimi_delta_attention" if ltype == "kda" else "gated_delta_rule"
        out.append(LayerOperationInfo(i, "linear_attention", name, None, None, CacheType.RECURRENT | CacheType.HYBRID,
                                      False, True))
        return out
    if spec is not None and getattr(spec, "mla", None) is not None:
        out.append(LayerOperationInfo(i, "latent_attention", "flash_attention", "latent_paged_attention", None,
                                      CacheType.TRANSFORMER | CacheType.LATENT_PAGES | CacheType.HYBRID, True, False,
                                      num_kv_heads=1, head_dim=spec.mla["kv_lora_rank"] + spec.mla["qk_rope_head_dim"]))
        return out
    if attn is not None:
        window = getattr(attn, "sliding_window", None) or None
        chunk = getattr(attn, "chunk_size", None) or None
        kind = "sliding_attention" if window else ("chunked_attention" if chunk else "full_attention")
        out.append(LayerOperationInfo(i, kind, "flash_attention", "paged_decode_attention",
                                      0 if hasattr(layer, "mamba") else None, paged, True, False, window, chunk,
                                      getattr(attn, "num_kv_heads", 0), getattr(attn, "head_dim", 0)))
    if hasattr(layer, "mamba"):
        out.append(LayerOperationInfo(i, "ssm", "ssd_scan", None, 1, CacheType.RECURRENT | CacheType.HYBRID, False,
                                      True))
    return out


def _combine(infos: list[LayerOperationInfo]) -> OperationsCacheInfo:
    combined = CacheType.any()
    for l in infos:
        combined &= l.supported_cache_types
    any_state = any(l.requires_state_cache for l in infos)
    any_kv = any(l.requires_kv_cache for l in infos)
    first_attn = next((l for l in infos if l.requires_kv_cache), None)
    return OperationsCacheInfo(
        layers=infos,
        prefill_operation=first_attn.operation_name if first_attn else (infos[0].operation_name if infos else ""),
        decode_operation=(first_attn.decode_operation_name or first_attn.operation_name) if first_attn else "",
        combined_cache_types=combined, is_hybrid_model=any_state and any_kv,
        supports_ragged_pages=bool(combined & CacheType.RAGGED_PAGES) and not any_state,
        supports_transformer_cache=bool(combined & CacheType.TRANSFORMER) and not any_state,
        requires_hybrid_cache=any_state, requires_state_management=any_state,
        has_separate_decode_ops=any(l.has_separate_decode for l in infos))
