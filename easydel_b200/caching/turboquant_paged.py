"""Paged KV cache holding TurboQuant-compressed keys and values.

Five page pools per layer instead of two: key codes (Lloyd-Max indices of the rotated unit key, two 4-bit codes per
byte), key sign bits of the residual sketch (eight per byte), key norms (norm of the key, norm of its quantisation
residual), value codes and value norms. At the default 4 bits and a 128-bit sketch a 128-wide head costs 64 + 16 + 4
+ 64 + 2 = 150 bytes per token and KV head against 512 in bf16. Attention runs as tensor code over the pages of each
scheduled sequence: scores are the unbiased estimate of ``layers/turboquant.key_scores`` (codebook term + sign-sketch
correction), values are de-quantised after the softmax. There is no fused kernel for this cache; the engine runs it
eagerly (no decode graphs).

Counterpart of easydel/caching/turboquant_ragged_page/cache.py:65-430 (``TurboQuantRaggedPagesCache`` and its view).
"""

from __future__ import annotations

import torch

from ..layers import turboquant as TQ
from .paged import PAGE_SIZE, PagedBatchMeta, _pad_queries


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """uint8 values < 16, last dimension even -> two per byte."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    out = torch.stack([packed & 0xF, packed >> 4], dim=-1)
    return out.reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def pack_bits(bits: torch.Tensor) -> torch.Tensor:
    """bool ``[..., m]`` (m a multiple of 8) -> uint8 ``[..., m / 8]``."""
    b = bits.reshape(*bits.shape[:-1], -1, 8).to(torch.uint8)
    w = (1 << torch.arange(8, device=bits.device, dtype=torch.uint8))
    return (b * w).sum(-1).to(torch.uint8)


def unpack_bits(packed: torch.Tensor) -> torch.Tensor:
    w = (1 << torch.arange(8, device=packed.device, dtype=torch.uint8))
    return ((packed[..., None] & w) != 0).reshape(*packed.shape[:-1], packed.shape[-1] * 8)


class TurboQuantLayerView:
    """One layer's compressed pools; same ``attend`` contract as :class:`easydel_b200.caching.paged.PagedLayerView`."""

    linear_state = None
    group = 0

    def __init__(self, cache: "TurboQuantPagedKVCache", layer: int):
        self.cache, self.layer = cache, layer

    def attend(self, attn, q, k, v, positions=None, attn_meta: PagedBatchMeta | None = None):
        c, meta, L = self.cache, attn_meta, self.layer
        q3, k3, v3 = q[0], k[0], v[0]                         # [T, H, D]
        slots = meta.slots_of(0).long()
        kc, kn, ks, kr = TQ.quantize_keys(k3, c.constants)
        vc, vn = TQ.quantize_values(v3, c.constants)
        flat = lambda t: t.view(-1, *t.shape[2:])             # noqa: E731  pools are [pages, page, ...]
        flat(c.k_codes[L])[slots] = pack_nibbles(kc) if c.packed else kc
        flat(c.k_signs[L])[slots] = pack_bits(ks)
        flat(c.k_norms[L])[slots] = torch.stack([kn, kr], -1).to(c.k_norms.dtype)
        flat(c.v_codes[L])[slots] = pack_nibbles(vc) if c.packed else vc
        flat(c.v_norms[L])[slots] = vn.to(c.v_norms.dtype)
        # gather every scheduled sequence's pages and attend in the dense form, one padded row per sequence
        B = meta.num_seqs
        table = meta.table_of(0)[:B].long().clamp_min(0)
        take = lambda pool: pool[L][table].reshape(B, -1, *pool.shape[3:])     # noqa: E731  [B, Tk, Hkv, ...]
        un = unpack_nibbles if c.packed else (lambda t: t)
        kcodes, vcodes = un(take(c.k_codes)), un(take(c.v_codes))
        ksign, knorm = unpack_bits(take(c.k_signs)), take(c.k_norms).float()
        vnorm = take(c.v_norms).float()
        qb, qpos, lens, cu = _pad_queries(q3, meta)            # [B, max_q, Hq, D]
        Hq, Hkv = qb.shape[2], kcodes.shape[2]
        G = Hq // Hkv
        qh = qb.permute(0, 2, 1, 3).reshape(B, Hkv, G * qb.shape[1], -1)       # queries of a KV head's group together
        kq = (kcodes.permute(0, 2, 1, 3), knorm[..., 0].permute(0, 2, 1), ksign.permute(0, 2, 1, 3),
              knorm[..., 1].permute(0, 2, 1))
        s = TQ.key_scores(qh, *kq, c.constants) * (attn.scale if attn.scale is not None else qb.shape[-1] ** -0.5)
        s = s.view(B, Hkv, G, qb.shape[1], -1)
        if attn.softcap:
            s = attn.softcap * torch.tanh(s / attn.softcap)
        kpos = torch.arange(s.shape[-1], device=s.device)
        ok = (kpos[None, None, :] <= qpos[:, :, None]) & (kpos[None, None, :] < meta.kv_lens[:B].long()[:, None, None])
        if attn.sliding_window:
            ok = ok & (kpos[None, None, :] > qpos[:, :, None] - attn.sliding_window)
        s = s.masked_fill(~ok[:, None, None], float("-inf"))
        p = torch.softmax(s, -1).nan_to_num(0.0)
        vals = TQ.dequantize_values(vcodes.permute(0, 2, 1, 3), vnorm.permute(0, 2, 1), c.constants)   # [B, Hkv, Tk, D]
        o = (p.reshape(B, Hkv, -1, s.shape[-1]) @ vals).view(B, Hkv, G, qb.shape[1], -1)
        o = o.permute(0, 3, 1, 2, 4).reshape(B, qb.shape[1], Hq, -1).to(q3.dtype)
        out = q3.new_zeros(q3.shape)
        if lens is None:
            out[:B] = o[:, 0]
        else:
            for b, n in enumerate(lens):
                out[cu[b]:cu[b + 1]] = o[b, :n]
        return out[None]


class TurboQuantPagedKVCache:
    """Compressed page pools for a model whose attention layers all keep the full context."""

    latent = False
    compressed = True

    def __init__(self, num_layers: int, num_pages: int, num_kv_heads: int, head_dim: int, config: TQ.TurboQuantConfig,
                 dtype=torch.bfloat16, device=None, page_size: int = PAGE_SIZE):
        from .specs import FullAttentionSpec, KVCacheGroup

        if page_size != PAGE_SIZE:
            raise ValueError(f"pages hold {PAGE_SIZE} tokens, got {page_size}")
        self.config, self.dtype, self.page_size = config, dtype, page_size
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.constants = TQ.TurboQuantConstants.create(config, head_dim, device=device)
        m = int(self.constants.qjl_dim)
        if m % 8 or head_dim % 2:
            raise ValueError("the sign sketch must be a multiple of 8 bits wide and the head size even")
        self.packed = config.bits <= 4        # value codes need `bits` bits, key codes one fewer
        cw = head_dim // 2 if self.packed else head_dim
        shape = (num_layers, int(num_pages), page_size, num_kv_heads)
        z = lambda last, dt: torch.zeros(*shape, *last, dtype=dt, device=device)   # noqa: E731
        self.k_codes, self.v_codes = z((cw,), torch.uint8), z((cw,), torch.uint8)
        self.k_signs = z((m // 8,), torch.uint8)
        self.k_norms, self.v_norms = z((2,), torch.bfloat16), z((), torch.bfloat16)
        per_token = cw * 2 + m // 8 + 4 + 2
        # the scheduler's page bookkeeping sees one full-attention group; its byte size is the compressed one
        spec = FullAttentionSpec(page_size=page_size, num_kv_heads=num_kv_heads, head_dim=head_dim, element_size=1)
        self.groups = [KVCacheGroup(spec, list(range(num_layers)), int(num_pages))]
        self.bytes_per_token_head = per_token
        self.linear: dict[int, object] = {}
        self.step_meta: PagedBatchMeta | None = None

    @property
    def num_pages(self) -> int:
        return int(self.groups[0].num_pages)

    @property
    def num_groups(self) -> int:
        return 1

    @property
    def k(self) -> torch.Tensor:
        return self.k_codes

    def memory_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.k_codes, self.v_codes, self.k_signs, self.k_norms,
                                                           self.v_norms))

    def compression_ratio(self) -> float:
        """bf16 bytes per token and KV head over the compressed bytes."""
        return 4.0 * self.head_dim / self.bytes_per_token_head

    def add_state_pools(self, model, num_slots: int) -> None:
        return None

    def reset_slot_state(self, slot: int) -> None:
        return None

    def view(self, layer: int) -> TurboQuantLayerView:
        return TurboQuantLayerView(self, layer)

    @classmethod
    def init_for_model(cls, model, config: TQ.TurboQuantConfig, num_pages: int | None = None,
                       hbm_utilization: float = 0.85, max_pages: int | None = None, device=None, **_):
        spec = model.spec
        if getattr(spec, "mla", None) is not None:
            raise ValueError("the compressed cache covers standard attention layers, not latent attention")
        device = device or model.device
        tp_size = getattr(getattr(model.config, "mesh", None), "tp", 1)
        hkv = max(1, spec.num_kv_heads // tp_size)
        probe = cls(1, 2, hkv, spec.head_dim, config, device="cpu")
        per_page = probe.bytes_per_token_head * hkv * PAGE_SIZE * spec.num_layers
        if num_pages is None:
            if torch.device(device).type == "cuda":
                free, total = torch.cuda.mem_get_info(device)
                budget = max(0, int(free - (1.0 - hbm_utilization) * total))
            else:
                budget = 64 << 20
            num_pages = max(2, budget // per_page)
            if max_pages is not None:
                num_pages = min(num_pages, int(max_pages))
        return cls(spec.num_layers, int(num_pages), hkv, spec.head_dim, config, dtype=model.dtype, device=device)


__all__ = ["TurboQuantPagedKVCache", "TurboQuantLayerView", "pack_nibbles", "unpack_nibbles", "pack_bits",
           "unpack_bits"]
