"""Dense per-layer KV cache used by ``model.generate()`` (easydel/caching/transformer/cache.py:329-1039).

Keys / values are stored ``[B, S, Hkv, D]`` per layer with one shared write cursor; the attention
kernel aligns queries to the end of the keys, so a decode step is a length-1 query over ``S`` keys.
Left-padded prompts are handled with per-row start offsets turned into segment masks on prefill.
"""

from __future__ import annotations

import torch

from ..ops import functional as F


class TransformerCache:
    def __init__(self, num_layers: int, batch: int, max_len: int, num_kv_heads: int, head_dim: int,
                 dtype=torch.bfloat16, device=None):
        self.k = torch.zeros(num_layers, batch, max_len, num_kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.length = 0
        self.max_len = max_len
        self.linear: dict[int, object] = {}     # layer -> recurrent state of a linear-attention layer (hybrids)

    @classmethod
    def init_for_model(cls, model, batch_size: int, max_length: int, dtype=None, device=None):
        spec = model.spec
        tp_size = getattr(model.config.mesh, "tp", 1)
        cache = cls(spec.num_layers, batch_size, max_length, max(1, spec.num_kv_heads // tp_size), spec.head_dim,
                    dtype or model.dtype, device or model.device)
        layers = getattr(getattr(model, "model", model), "layers", ())
        for i, layer in enumerate(layers):
            mixer = getattr(layer, "linear_attn", None) or getattr(layer, "mamba", None)
            if mixer is None and hasattr(getattr(layer, "self_attn", None), "make_state"):
                mixer = layer.self_attn
            if mixer is not None:
                cache.linear[i] = mixer.make_state(batch_size, dtype or model.dtype, device or model.device)
        return cache

    def seq_len(self) -> int:
        return self.length

    def view(self, layer: int) -> "TransformerCacheView":
        return TransformerCacheView(self, layer)

    def advance(self, n: int) -> None:
        self.length += n

    def reorder(self, index: torch.Tensor) -> None:
        """Beam search: re-gathers the batch rows."""
        self.k = self.k.index_select(1, index)
        self.v = self.v.index_select(1, index)
        for st in self.linear.values():
            st.reorder(index)


class TransformerCacheView:
    def __init__(self, cache: TransformerCache, layer: int):
        self.cache, self.layer = cache, layer

    @property
    def linear_state(self):
        return self.cache.linear.get(self.layer)

    def attend(self, attn, q, k, v, positions=None, attn_meta=None):
        c = self.cache
        T = q.shape[1]
        s, e = c.length, c.length + T
        if e > c.max_len:
            raise ValueError(f"KV cache overflow: {e} > {c.max_len}")
        hk = k.shape[2]          # layers may use fewer KV heads than the widest one the cache was sized for
        c.k[self.layer, :, s:e, :hk] = k
        c.v[self.layer, :, s:e, :hk] = v
        kk, vv = c.k[self.layer, :, :e, :hk], c.v[self.layer, :, :e, :hk]
        if hk != c.k.shape[3]:
            kk, vv = kk.contiguous(), vv.contiguous()
        seg = None
        if attn_meta is not None and attn_meta.get("kv_segment_ids") is not None:
            # left padding: padded positions carry segment 0
            seg_k = attn_meta["kv_segment_ids"][:, :e]
            from ..ops import reference as R

            return R.attention(q, kk, vv, causal=True, scale=attn.scale, segment_ids=seg_k[:, s:e],
                               kv_segment_ids=seg_k, sliding_window=attn.sliding_window, softcap=attn.softcap,
                               sinks=attn.sinks)
        chunk = getattr(attn, "chunk_size", None)
        if chunk and e > chunk:
            # block-diagonal causal attention over the cache: keys outside the query's block are masked out
            from ..ops import reference as R

            qpos = torch.arange(s, e, device=q.device)
            kpos = torch.arange(e, device=q.device)
            bias = torch.where((qpos[:, None] // chunk) == (kpos[None, :] // chunk), 0.0, float("-inf"))
            return R.attention(q, kk, vv, causal=True, scale=attn.scale, softcap=attn.softcap, sinks=attn.sinks,
                               bias=bias[None, None])
        if kk.shape[0] > 1 and e < c.max_len:
            kk, vv = kk.contiguous(), vv.contiguous()  # the kernels want equally spaced token rows
        return F.attention(q, kk, vv, causal=True, scale=attn.scale, sliding_window=attn.sliding_window,
                           softcap=attn.softcap, sinks=attn.sinks)
