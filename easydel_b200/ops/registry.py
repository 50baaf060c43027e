"""Named attention operations and their registry (easydel/operations/_operation_impl.py:96,
easydel/operations/_operation_meta.py, easydel/operations/kernels/*.py, easydel/layers/attention/_flexible.py).

Each operation is a small object (metadata + configuration) whose ``forward`` calls one of this package's attention
entry points; models select one by the name in ``config.attn_mechanism`` through :class:`FlexibleAttentionModule`.
There is one implementation per name (this package targets one device type), so the registry maps names to classes
rather than (name, backend) pairs:

    flash_attn2, blocksparse, blockwise, cudnn, auto   the tcgen05 flash kernels (``ops.functional.attention``)
    vanilla                                             dense fp32 softmax attention (``ops.reference.attention``)
    sdpa                                                ``torch.nn.functional.scaled_dot_product_attention``
    ring                                                sequence-parallel attention over a process group
    ragged_page_attention_v2 / _v3, page_attention,
    unified_attention, paged_flash_attention            mixed prefill / decode over the paged cache
    autoregressive_decodeattn                           one query token per sequence over the paged cache
"""

from __future__ import annotations

import dataclasses
import typing as tp

import torch


@dataclasses.dataclass
class OperationMetadata:
    """What an operation needs to know about the model it runs in."""

    runtime_dtype: torch.dtype = torch.bfloat16
    runtime_softmax_dtype: torch.dtype = torch.float32
    sequence_axis_name: str = "sp"
    mesh: tp.Any = None                     # a ``parallel.mesh.DeviceMesh`` (ring attention takes its ``sp`` group)
    platform: str = "cuda"
    backend: str = "sm_100a"

    @classmethod
    def from_config(cls, config) -> "OperationMetadata":
        dt = getattr(config, "attn_dtype", None) or getattr(config, "dtype", None) or torch.bfloat16
        return cls(runtime_dtype=dt, mesh=getattr(config, "mesh", None))


@dataclasses.dataclass
class BaseOperationConfig:
    """Options shared by every attention operation; subclasses add their own."""

    causal: bool = True
    softmax_scale: float | None = None
    sliding_window: int | None = None
    logits_soft_cap: float = 0.0


@dataclasses.dataclass
class FlashAttentionConfig(BaseOperationConfig):
    pass


@dataclasses.dataclass
class BlockSparseAttentionConfig(BaseOperationConfig):
    chunk_size: int | None = None           # block-diagonal causal attention inside chunks of this many tokens


@dataclasses.dataclass
class ScaledDotProductAttentionConfig(BaseOperationConfig):
    pass


@dataclasses.dataclass
class RingAttentionConfig(BaseOperationConfig):
    layout: str = "zigzag"                  # how the sequence is cut over the ranks: zigzag | contiguous
    impl: str = "auto"                      # gather | peer | auto


@dataclasses.dataclass
class RaggedPageAttentionv2Config(BaseOperationConfig):
    pass


@dataclasses.dataclass
class RaggedPageAttentionv3Config(BaseOperationConfig):
    pass


AttentionConfig = BaseOperationConfig


@dataclasses.dataclass
class AttentionOutput:
    attention_outputs: torch.Tensor | None = None
    attention_weights: torch.Tensor | None = None
    cache_view: tp.Any = None


class OperationRegistry:
    _table: dict[str, type["OperationImpl"]] = {}

    @classmethod
    def register(cls, impl: type["OperationImpl"]) -> type["OperationImpl"]:
        names = impl.get_impl_name()
        for n in ((names,) if isinstance(names, str) else names):
            cls._table[str(n)] = impl
        return impl

    @classmethod
    def get(cls, name: str) -> type["OperationImpl"]:
        try:
            return cls._table[str(name)]
        except KeyError:
            raise KeyError(f"no operation named {name!r}; known: {sorted(cls._table)}") from None

    @classmethod
    def create(cls, name: str, metadata: OperationMetadata | None = None, config=None) -> "OperationImpl":
        return cls.get(name)(metadata, config)

    @classmethod
    def list_implementations(cls) -> list[str]:
        return sorted(cls._table)


class OperationImpl:
    """Base class: ``get_impl_name`` (one name or a tuple of names), ``forward``; calling the object runs it."""

    config_class: type = BaseOperationConfig

    def __init__(self, metadata: OperationMetadata | None = None, config=None):
        self.metadata = metadata or OperationMetadata()
        self.config = config if config is not None else self.config_class()

    @classmethod
    def get_impl_name(cls) -> str | tuple[str, ...]:
        raise NotImplementedError

    def get_impl_metadata(self) -> OperationMetadata:
        return self.metadata

    def forward(self, *args, **kw) -> AttentionOutput:
        raise NotImplementedError

    def __call__(self, *args, **kw) -> AttentionOutput:
        return self.forward(*args, **kw)

    def _opts(self, kw: dict) -> dict:
        c = self.config
        return dict(causal=kw.pop("causal", c.causal), scale=kw.pop("softmax_scale", kw.pop("scale", c.softmax_scale)),
                    sliding_window=kw.pop("sliding_window", c.sliding_window),
                    softcap=kw.pop("logits_soft_cap", kw.pop("softcap", c.logits_soft_cap)) or 0.0)


@OperationRegistry.register
class FlashAttn(OperationImpl):
    """q ``[B, T, Hq, D]``, k / v ``[B, T, Hkv, D]``: the flash kernels on CUDA bf16, the dense form elsewhere."""

    config_class = FlashAttentionConfig

    @classmethod
    def get_impl_name(cls):
        return ("flash_attn2", "flash", "cudnn", "blockwise", "auto")

    def forward(self, query, key, value, *, segment_ids=None, sinks=None, cu_seqlens=None, **kw) -> AttentionOutput:
        from . import functional as F

        o = F.attention(query, key, value, segment_ids=segment_ids, sinks=sinks, cu_seqlens=cu_seqlens,
                        **self._opts(kw))
        return AttentionOutput(attention_outputs=o)


@OperationRegistry.register
class BlockSparseAttn(FlashAttn):
    """Causal attention restricted to blocks: a ``chunk_size`` makes the mask block-diagonal (expressed as segment
    ids, which the flash kernels take), a sliding window limits the look-back; both skip whole key blocks."""

    config_class = BlockSparseAttentionConfig

    @classmethod
    def get_impl_name(cls):
        return "blocksparse"

    def forward(self, query, key, value, *, segment_ids=None, positions=None, **kw) -> AttentionOutput:
        chunk = kw.pop("chunk_size", getattr(self.config, "chunk_size", None))
        if chunk:
            B, T = query.shape[:2]
            pos = positions if positions is not None else torch.arange(T, device=query.device)[None].expand(B, T)
            blocks = pos // int(chunk)
            base = segment_ids.long() if segment_ids is not None else torch.ones_like(blocks)
            segment_ids = ((base * (int(blocks.max()) + 1) + blocks) * (base != 0)).to(torch.int32)
        return super().forward(query, key, value, segment_ids=segment_ids, **kw)


@OperationRegistry.register
class VanillaAttn(OperationImpl):
    """Dense softmax attention in fp32; also returns the probabilities when asked (``output_attentions``)."""

    @classmethod
    def get_impl_name(cls):
        return "vanilla"

    def forward(self, query, key, value, *, segment_ids=None, sinks=None, bias=None, output_attentions=False,
                **kw) -> AttentionOutput:
        from . import reference as R

        c = self._opts(kw)
        o = R.attention(query, key, value, segment_ids=segment_ids, sinks=sinks, bias=bias, **c)
        w = None
        if output_attentions:
            G = query.shape[2] // key.shape[2]
            s = torch.einsum("bqhd,bkhd->bhqk", query.float(), key.float().repeat_interleave(G, 2))
            s = s * (c["scale"] if c["scale"] is not None else query.shape[-1] ** -0.5)
            if c["causal"]:
                Tq, Tk = s.shape[-2:]
                s = s.masked_fill(~torch.ones(Tq, Tk, dtype=torch.bool, device=s.device).tril(Tk - Tq), float("-inf"))
            w = s.softmax(-1)
        return AttentionOutput(attention_outputs=o.to(query.dtype), attention_weights=w)


@OperationRegistry.register
class ScaledDotProductAttn(OperationImpl):
    config_class = ScaledDotProductAttentionConfig

    @classmethod
    def get_impl_name(cls):
        return "sdpa"

    def forward(self, query, key, value, *, attention_mask=None, **kw) -> AttentionOutput:
        c = self._opts(kw)
        if c["softcap"] or c["sliding_window"]:
            raise NotImplementedError("sdpa takes neither a soft cap nor a sliding window; use flash_attn2")
        q, k, v = (t.transpose(1, 2) for t in (query, key, value))
        o = torch.nn.functional.scaled_dot_product_attention(
            q, k, v, attn_mask=attention_mask, is_causal=c["causal"] and attention_mask is None, scale=c["scale"],
            enable_gqa=q.shape[1] != k.shape[1])
        return AttentionOutput(attention_outputs=o.transpose(1, 2))


@OperationRegistry.register
class RingAttn(OperationImpl):
    """Every rank holds a slice of the sequence; ``group`` (or the mesh's ``sp`` group) names the ranks."""

    config_class = RingAttentionConfig

    @classmethod
    def get_impl_name(cls):
        return "ring"

    def forward(self, query, key, value, *, group=None, **kw) -> AttentionOutput:
        from ..parallel import context_parallel as CP

        if group is None and self.metadata.mesh is not None:
            group = self.metadata.mesh.get_group(self.metadata.sequence_axis_name)
        if group is None:
            raise ValueError("ring attention needs the process group of the sequence-parallel ranks")
        c = self._opts(kw)
        if c["sliding_window"]:
            raise NotImplementedError("ring attention covers causal / full attention without a window")
        o = CP.ring_attention(query.contiguous(), key.contiguous(), value.contiguous(), group,
                              layout=kw.pop("layout", self.config.layout), causal=c["causal"], scale=c["scale"],
                              softcap=c["softcap"], impl=kw.pop("impl", self.config.impl))
        return AttentionOutput(attention_outputs=o)


class _PagedBase(OperationImpl):
    """q ``[T, Hq, D]`` of all scheduled sequences; ``cache_view`` exposes the layer's key / value page pools and
    ``cache_metadata`` the batch (``cu_q``, ``kv_lens``, ``page_table``, ``max_q``)."""

    def forward(self, query, key=None, value=None, *, cache_view=None, cache_metadata=None, k_pages=None,
                v_pages=None, cu_q=None, kv_lens=None, page_table=None, max_q=None, sinks=None,
                **kw) -> AttentionOutput:
        from . import serving as S

        m = cache_metadata
        if cache_view is not None and k_pages is None:
            k_pages, v_pages = cache_view.k_pages, cache_view.v_pages
        cu_q = cu_q if cu_q is not None else m.cu_q
        kv_lens = kv_lens if kv_lens is not None else m.kv_lens
        page_table = page_table if page_table is not None else m.page_table
        max_q = max_q if max_q is not None else getattr(m, "max_q", None) or int((cu_q[1:] - cu_q[:-1]).max())
        c = self._opts(kw)
        o = S.paged_attention(query, k_pages, v_pages, cu_q, kv_lens, page_table, int(max_q), scale=c["scale"],
                              causal=c["causal"], window=int(c["sliding_window"] or 0), softcap=c["softcap"],
                              sinks=sinks)
        return AttentionOutput(attention_outputs=o, cache_view=cache_view)


@OperationRegistry.register
class RaggedPageAttnV2(_PagedBase):
    config_class = RaggedPageAttentionv2Config

    @classmethod
    def get_impl_name(cls):
        return "ragged_page_attention_v2"


@OperationRegistry.register
class RaggedPageAttnV3(_PagedBase):
    config_class = RaggedPageAttentionv3Config

    @classmethod
    def get_impl_name(cls):
        return ("ragged_page_attention_v3", "page_attention", "unified_attention")


@OperationRegistry.register
class PagedFlashAttn(_PagedBase):
    @classmethod
    def get_impl_name(cls):
        return "paged_flash_attention"


@OperationRegistry.register
class AutoRegressiveDecodeAttn(OperationImpl):
    """One query token per sequence, q ``[B, Hq, D]``, over the paged cache (the split-K streaming kernel)."""

    @classmethod
    def get_impl_name(cls):
        return "autoregressive_decodeattn"

    def forward(self, query, k_pages, v_pages, kv_lens, page_table, *, sinks=None, num_splits: int = 1,
                **kw) -> AttentionOutput:
        from . import serving as S

        c = self._opts(kw)
        if S.decode_kernel_supports(query, k_pages, c["softcap"]):
            o = S.decode_attention(query, k_pages, v_pages, kv_lens, page_table, scale=c["scale"],
                                   window=int(c["sliding_window"] or 0), sinks=sinks, num_splits=num_splits)
        else:
            cu = torch.arange(query.shape[0] + 1, dtype=torch.int32, device=query.device)
            o = S.paged_attention(query, k_pages, v_pages, cu, kv_lens, page_table, 1, scale=c["scale"],
                                  window=int(c["sliding_window"] or 0), softcap=c["softcap"], sinks=sinks)
        return AttentionOutput(attention_outputs=o)


class FlexibleAttentionModule(torch.nn.Module):
    """The operation a model's ``attn_mechanism`` names, behind one call signature."""

    def __init__(self, base_config=None, softmax_scale: float | None = None, attn_mechanism: str | None = None,
                 causal: bool = True, sliding_window: int | None = None, logits_soft_cap: float = 0.0):
        super().__init__()
        name = str(attn_mechanism or getattr(base_config, "attn_mechanism", None) or "auto")
        cls = OperationRegistry.get(name)
        cfg = cls.config_class(causal=causal, softmax_scale=softmax_scale, sliding_window=sliding_window,
                               logits_soft_cap=logits_soft_cap)
        meta = OperationMetadata.from_config(base_config) if base_config is not None else OperationMetadata()
        self.impl, self.mechanism = cls(meta, cfg), name

    def forward(self, query_states, key_states, value_states, **kw) -> AttentionOutput:
        return self.impl(query_states, key_states, value_states, **kw)


__all__ = ["OperationMetadata", "BaseOperationConfig", "AttentionConfig", "FlashAttentionConfig",
           "BlockSparseAttentionConfig", "ScaledDotProductAttentionConfig", "RingAttentionConfig",
           "RaggedPageAttentionv2Config", "RaggedPageAttentionv3Config", "AttentionOutput", "OperationRegistry",
           "OperationImpl", "FlashAttn", "BlockSparseAttn", "VanillaAttn", "ScaledDotProductAttn", "RingAttn",
           "RaggedPageAttnV2", "RaggedPageAttnV3", "PagedFlashAttn", "AutoRegressiveDecodeAttn",
           "FlexibleAttentionModule"]
