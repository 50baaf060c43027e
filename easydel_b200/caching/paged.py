"""Paged KV cache for the eSurge engine.

Layout follows the reference's GPU cache (``UnifiedAttentionCache``: separate key and value page
arrays ``[P, page, Hkv, D]``, easydel/caching/unified_attention/cache.py:465-466); the number of
pages comes from free HBM x ``hbm_utilization`` like easydel/caching/ragged_page/cache.py:557-559.
Page size is 128 tokens: one page is exactly one key tile of the paged attention kernel, so a
tile is fetched with a single TMA load addressed through the page table.

``PagedBatchMeta`` is the per-step device metadata (the reference's ``RaggedPagesMetadata``,
ragged_page/cache.py:1157-1250): query start offsets, context lengths, page tables, slot mapping.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass

import torch

from ..ops import serving as S

PAGE_SIZE = S.PAGE_SIZE


@dataclass
class PagedBatchMeta:
    cu_q: torch.Tensor           # int32 [B+1] offsets of each sequence's new tokens in the flat token axis
    kv_lens: torch.Tensor        # int32 [B]   keys per sequence after this step's append
    page_table: torch.Tensor     # int32 [B, maxP]
    slot_mapping: torch.Tensor   # int32 [T]   flat page slot of every new token (-1 = padding)
    max_q: int                   # largest number of new tokens of any sequence
    num_seqs: int
    last_token_index: torch.Tensor | None = None  # int32 [B] row of each sequence's last new token
    request_distribution: tuple[int, int, int] | None = None  # (#decode, #decode+#prefill, #total)
    num_splits: int = 1          # decode-only steps: cut every sequence's keys into this many page ranges
    seq_slots: torch.Tensor | None = None   # int64 [B] engine slot of every sequence (recurrent-state pools)
    # cache groups beyond the first (sliding-window / chunked-local layers with their own pools): per group the page
    # table [B, maxP] and the slot mapping [T]; entry g - 1 belongs to group g
    group_tables: list | None = None
    group_slots: list | None = None

    def table_of(self, group: int) -> torch.Tensor:
        return self.page_table if group == 0 or not self.group_tables else self.group_tables[group - 1]

    def slots_of(self, group: int) -> torch.Tensor:
        return self.slot_mapping if group == 0 or not self.group_slots else self.group_slots[group - 1]


class PagedKVCache:
    """Key / value pages of every layer. Layers that retain keys under the same rule (full context, a sliding window,
    a block of chunked-local attention) form a *group* with its own page count and page tables
    (:mod:`easydel_b200.caching.specs`); one group of all layers is the plain case."""

    def __init__(self, num_layers: int, num_pages: int, num_kv_heads: int, head_dim: int, dtype=torch.bfloat16,
                 device=None, page_size: int = PAGE_SIZE, latent: bool = False, groups=None):
        if page_size != PAGE_SIZE:
            raise ValueError(f"the paged attention kernels use pages of {PAGE_SIZE} tokens, got {page_size}")
        from .specs import FullAttentionSpec, KVCacheGroup, MLAAttentionSpec

        self.num_layers, self.page_size = num_layers, page_size
        self.num_kv_heads, self.head_dim, self.dtype = num_kv_heads, head_dim, dtype
        # latent attention stores one row per token (compressed keys/values + the shared rotary key): no value pool
        self.latent = latent
        if groups is None:
            es = torch.empty(0, dtype=dtype).element_size()
            spec_cls = MLAAttentionSpec if latent else FullAttentionSpec
            groups = [KVCacheGroup(spec_cls(page_size=page_size, num_kv_heads=num_kv_heads, head_dim=head_dim,
                                            element_size=es), list(range(num_layers)), int(num_pages))]
        self.groups = list(groups)
        self.layer_slot: dict[int, tuple[int, int]] = {}
        self._k, self._v = [], []
        for g, grp in enumerate(self.groups):
            shape = (len(grp.layers), int(grp.num_pages), page_size, grp.spec.num_kv_heads, grp.spec.head_dim)
            k = torch.zeros(shape, dtype=dtype, device=device)      # zeros: the null page must hold finite numbers
            self._k.append(k)
            self._v.append(k if grp.kind == "latent" else torch.zeros(shape, dtype=dtype, device=device))
            for j, layer in enumerate(grp.layers):
                self.layer_slot[layer] = (g, j)
        # hybrids: layer -> recurrent state with one row per engine slot; ``step_meta`` is the running step's batch
        self.linear: dict[int, object] = {}
        self.step_meta: PagedBatchMeta | None = None

    @property
    def k(self) -> torch.Tensor:
        return self._k[0]

    @property
    def v(self) -> torch.Tensor:
        return self._v[0]

    @property
    def num_pages(self) -> int:
        return int(self.groups[0].num_pages)

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    def memory_bytes(self) -> int:
        seen, n = set(), 0
        for t in (*self._k, *self._v):
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n

    def add_state_pools(self, model, num_slots: int) -> None:
        layers = getattr(getattr(model, "model", model), "layers", ())
        for i, layer in enumerate(layers):
            mixer = getattr(layer, "linear_attn", None) or getattr(layer, "mamba", None)
            if mixer is None and hasattr(getattr(layer, "self_attn", None), "make_state"):
                mixer = layer.self_attn
            if mixer is not None:
                self.linear[i] = mixer.make_state(num_slots, self.dtype, self.k.device)

    def reset_slot_state(self, slot: int) -> None:
        for st in self.linear.values():
            for v in vars(st).values():
                if isinstance(v, torch.Tensor):
                    v[slot].zero_()

    @staticmethod
    def bytes_per_page(num_layers: int, num_kv_heads: int, head_dim: int, dtype=torch.bfloat16,
                       page_size: int = PAGE_SIZE) -> int:
        return 2 * num_layers * page_size * num_kv_heads * head_dim * torch.empty(0, dtype=dtype).element_size()

    @classmethod
    def init_for_model(cls, model, num_pages: int | None = None, page_size: int = PAGE_SIZE,
                       hbm_utilization: float = 0.85, max_model_length: int | None = None, dtype=None, device=None,
                       max_pages: int | None = None, max_num_seqs: int | None = None,
                       max_num_batched_tokens: int | None = None):
        """Groups the model's layers by retention rule and sizes every group's pool. ``num_pages`` fixes the page
        count of every group; otherwise free HBM x ``hbm_utilization`` is divided by
        :func:`easydel_b200.caching.specs.plan_pages` (window-bounded groups get what ``max_num_seqs`` sequences can
        hold, the rest goes to the full-attention layers)."""
        from . import specs as SP

        spec = model.spec
        device = device or model.device
        dtype = dtype or getattr(model.config, "kvdtype", None) or model.dtype
        es = torch.empty(0, dtype=dtype).element_size()
        latent = getattr(spec, "mla", None) is not None
        lm = getattr(model, "language_model", model)
        groups = SP.build_groups(lm, element_size=es, page_size=page_size) \
            if hasattr(lm, "get_operations_cache_info") else []
        if not groups:      # a model of recurrent layers only still gets a (tiny) pool: the scheduler counts pages
            tp_size = getattr(model.config.mesh, "tp", 1)
            groups = [SP.KVCacheGroup(SP.FullAttentionSpec(page_size=page_size,
                                                           num_kv_heads=max(1, spec.num_kv_heads // tp_size),
                                                           head_dim=spec.head_dim, element_size=es), [], 2)]
        if num_pages is not None:
            counts = [int(num_pages)] * len(groups)
        else:
            if torch.device(device).type == "cuda":
                free, total = torch.cuda.mem_get_info(device)
                budget = max(0, int(free - (1.0 - hbm_utilization) * total))
            else:
                budget = 256 << 20
            seqs = max_num_seqs or 256
            mlen = max_model_length or spec.max_position
            counts = SP.plan_pages(groups, budget, seqs, mlen, max_num_batched_tokens or 2048)
            if max_pages is not None:
                # never more than max_num_seqs * pages-per-sequence would need
                counts = [min(int(c), int(max_pages)) for c in counts]
        for g, n in zip(groups, counts):
            g.num_pages = max(2, int(n))
        head = groups[0].spec
        return cls(spec.num_layers, groups[0].num_pages, head.num_kv_heads, head.head_dim, dtype, device, page_size,
                   latent=latent, groups=groups)

    def view(self, layer: int):
        slot = self.layer_slot.get(layer)
        if slot is None:
            view = PagedLayerView(None, None)        # a layer without keys / values (recurrent mixer only)
        else:
            g, j = slot
            view = PagedLatentView(self._k[g][j]) if self.groups[g].kind == "latent" else \
                PagedLayerView(self._k[g][j], self._v[g][j], group=g)
        pool = self.linear.get(layer)
        view.linear_state = None if pool is None else PagedLinearState(pool, self.step_meta)
        return view

    def seq_len(self) -> int:  # the engine passes explicit positions
        return 0


class PagedLinearState:
    """The recurrent state rows of the sequences scheduled in this step, gathered from the per-slot pool; ``cu`` gives
    the layers the ragged sequence bounds on the flat token axis. ``commit`` scatters the rows back."""

    def __init__(self, pool, meta: PagedBatchMeta):
        if meta is None or meta.seq_slots is None:
            raise RuntimeError("recurrent layers need the step's slot ids (PagedKVCache.step_meta.seq_slots)")
        self._pool, self._slots = pool, meta.seq_slots
        self.cu = meta.cu_q
        for name, v in vars(pool).items():
            if isinstance(v, torch.Tensor):
                setattr(self, name, v.index_select(0, self._slots))

    def commit(self) -> None:
        for name, v in vars(self._pool).items():
            if isinstance(v, torch.Tensor):
                v.index_copy_(0, self._slots, getattr(self, name).to(v.dtype))


class PagedLayerView:
    linear_state = None

    def __init__(self, k_pages: torch.Tensor, v_pages: torch.Tensor, group: int = 0):
        self.k_pages, self.v_pages, self.group = k_pages, v_pages, group

    def attend(self, attn, q, k, v, positions=None, attn_meta: PagedBatchMeta | None = None):
        """Appends this step's keys/values to their pages, then runs paged attention.

        q ``[1, T, Hq, D]`` / k, v ``[1, T, Hkv, D]`` (all sequences flattened on the token axis)."""
        meta = attn_meta
        T = q.shape[1]
        q3, k3, v3 = q[0], k[0], v[0]
        table = meta.table_of(self.group)
        S.kv_append(k3, v3, self.k_pages, self.v_pages, meta.slots_of(self.group))
        if getattr(attn, "chunk_size", None) or (q3.is_cuda and q3.shape[-1] not in (64, 128)):
            # block-diagonal attention, or a head size outside the paged kernel's (64 / 128)
            return self._attend_gathered(attn, q3, meta)[None]
        if meta.max_q == 1 and q3.shape[0] == meta.num_seqs and S.decode_kernel_supports(q3, self.k_pages,
                                                                                           attn.softcap):
            # a pure decode step: the streaming kernel (one CTA per sequence, KV head and key split)
            o = S.decode_attention(q3, self.k_pages, self.v_pages, meta.kv_lens, table, scale=attn.scale,
                                   window=attn.sliding_window or 0, sinks=attn.sinks, num_splits=meta.num_splits)
            return o[None]
        if meta.num_splits > 1 and meta.max_q == 1 and not attn.sliding_window and q3.is_cuda:
            o = S.paged_attention_splitkv(q3, self.k_pages, self.v_pages, meta.kv_lens, table,
                                          meta.num_splits, scale=attn.scale, softcap=attn.softcap, sinks=attn.sinks)
            return o[None]
        o = S.paged_attention(q3, self.k_pages, self.v_pages, meta.cu_q, meta.kv_lens, table, meta.max_q,
                              scale=attn.scale, causal=True, window=attn.sliding_window or 0, softcap=attn.softcap,
                              sinks=attn.sinks)
        return o[None]


def _pad_queries(q, meta: PagedBatchMeta):
    """Flat ``[T, H, D]`` queries -> (``[B, max_q, H, D]``, query positions ``[B, max_q]``, row lengths or None)."""
    B, T = meta.num_seqs, q.shape[0]
    kv_lens = meta.kv_lens[:B].long()
    if meta.max_q == 1 and T >= B:
        return q[:B, None], (kv_lens - 1)[:, None], None, None
    cu = meta.cu_q.tolist()
    lens = [cu[b + 1] - cu[b] for b in range(B)]
    qb = q.new_zeros(B, meta.max_q, *q.shape[1:])
    for b, n in enumerate(lens):
        qb[b, :n] = q[cu[b]:cu[b + 1]]
    qpos = kv_lens[:, None] - torch.tensor(lens, device=q.device)[:, None] + \
        torch.arange(meta.max_q, device=q.device)[None]
    return qb, qpos, lens, cu


def _attend_gathered(self, attn, q3, meta: PagedBatchMeta):
    """Causal attention over the gathered pages of the scheduled sequences in the dense form, one padded row per
    sequence: block-diagonal masks (keys outside the query's block of ``chunk_size`` positions), sliding windows and
    head sizes the paged kernel does not cover."""
    from ..ops import reference as R

    B = meta.num_seqs
    table = meta.table_of(getattr(self, "group", 0))[:B].long().clamp_min(0)
    kk = self.k_pages[table].reshape(B, -1, *self.k_pages.shape[2:])
    vv = self.v_pages[table].reshape(B, -1, *self.v_pages.shape[2:])
    qb, qpos, lens, cu = _pad_queries(q3, meta)
    kpos = torch.arange(kk.shape[1], device=q3.device)
    ok = (kpos[None, None, :] <= qpos[:, :, None]) & (kpos[None, None, :] < meta.kv_lens[:B].long()[:, None, None])
    if getattr(attn, "chunk_size", None):
        ok = ok & ((kpos[None, None, :] // attn.chunk_size) == (qpos[:, :, None] // attn.chunk_size))
    if attn.sliding_window:
        ok = ok & (kpos[None, None, :] > qpos[:, :, None] - attn.sliding_window)
    bias = torch.where(ok, 0.0, float("-inf"))[:, None]
    o = R.attention(qb, kk, vv, causal=False, scale=attn.scale, softcap=attn.softcap, sinks=attn.sinks, bias=bias)
    out = q3.new_zeros(q3.shape[0], *o.shape[2:])
    if lens is None:
        out[:B] = o[:, 0]
    else:
        for b, n in enumerate(lens):
            out[cu[b]:cu[b + 1]] = o[b, :n]
    return out


PagedLayerView._attend_gathered = _attend_gathered


class PagedLatentView:
    """Pages of latent-attention rows ``[compressed kv | rotary key]`` (one per token, shared by all heads).

    Attention runs in the absorbed form: the key up-projection is folded into the query and the value up-projection
    is applied after the weighted sum, so the cache is read as it is stored and never expanded per head. The pages
    of the scheduled sequences are gathered through the page table; the products are batched matrix multiplies.
    """

    linear_state = None

    def __init__(self, pages: torch.Tensor):
        self.pages = pages                  # [P, page, 1, kv_lora_rank + rope_dim]

    def attend_latent(self, mla, q_nope, q_rope, latent, k_rope, meta: PagedBatchMeta):
        """q_nope ``[1,T,H,nope]``, q_rope ``[1,T,H,rope]`` (rotated), latent ``[1,T,L]`` (normalised), k_rope
        ``[1,T,rope]`` (rotated) -> ``[1,T,H,v_head_dim]``."""
        T, H, L = q_nope.shape[1], q_nope.shape[2], latent.shape[-1]
        new = torch.cat([latent[0], k_rope[0]], -1).to(self.pages.dtype)[:, None, :].contiguous()
        S.kv_append(new, new, self.pages, self.pages, meta.slot_mapping)
        w = mla.kv_b_proj.weight.view(H, mla.nope + mla.vd, L)
        w_uk, w_uv = w[:, : mla.nope], w[:, mla.nope:]
        q = torch.cat([torch.einsum("thn,hnl->thl", q_nope[0], w_uk.to(q_nope.dtype)), q_rope[0]], -1)   # [T,H,L+R]
        B = meta.num_seqs
        if meta.max_q == 1 and T == B and mla.rope_dim == 64 and L == 512 and S.mla_decode_kernel_supports(q, self.pages):
            # a pure decode step of the 512 + 64 layout: the streaming kernel walks the page table itself
            o_lat = S.mla_decode_attention(q.contiguous(), self.pages, meta.kv_lens, meta.page_table, scale=mla.scale,
                                           num_splits=meta.num_splits)
            return torch.einsum("bhl,hvl->bhv", o_lat, w_uv.to(o_lat.dtype))[None]
        table = meta.page_table[:B].long().clamp_min(0)
        kv = self.pages[table].reshape(B, -1, self.pages.shape[-1])                                       # [B,Tk,L+R]
        Tk = kv.shape[1]
        kv_lens = meta.kv_lens[:B].long()
        if meta.max_q == 1 and T >= B:        # decode: row b is sequence b (rows past B are padding)
            qb = q[:B, None]
            qpos = (kv_lens - 1)[:, None]
            lens = None
        else:
            cu = meta.cu_q.tolist()
            lens = [cu[b + 1] - cu[b] for b in range(B)]
            qb = q.new_zeros(B, meta.max_q, H, q.shape[-1])
            for b, n in enumerate(lens):
                qb[b, :n] = q[cu[b]:cu[b + 1]]
            qpos = kv_lens[:, None] - torch.tensor(lens, device=q.device)[:, None] + \
                torch.arange(meta.max_q, device=q.device)[None]
        kpos = torch.arange(Tk, device=q.device)
        mask = (kpos[None, None, :] <= qpos[:, :, None]) & (kpos[None, None, :] < kv_lens[:, None, None])
        s = torch.einsum("bqhw,bkw->bhqk", qb, kv.to(qb.dtype)).float() * mla.scale
        s = s.masked_fill(~mask[:, None], float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0).to(qb.dtype)
        o = torch.einsum("bhqk,bkl->bqhl", p, kv[..., :L].to(qb.dtype))
        o = torch.einsum("bqhl,hvl->bqhv", o, w_uv.to(qb.dtype))                                           # [B,Tq,H,vd]
        out = q.new_zeros(T, H, mla.vd)
        if lens is None:
            out[:B] = o[:, 0]
        else:
            for b, n in enumerate(lens):
                out[cu[b]:cu[b + 1]] = o[b, :n]
        return out[None]
