"""Multi-head latent attention (DeepSeek-V2 / V3; easydel/layers/attention MLA paths and modules/deepseek_v3).

Keys and values are generated from a low-rank latent ``c_kv`` (``kv_lora_rank`` wide) plus one rotary key shared by
all heads; queries optionally go through their own low-rank bottleneck. The generation cache stores only the
normalised latent and the rotary key per token (:class:`MLACache`), and the per-head keys / values are re-expanded
from it. Query / key heads are ``qk_nope + qk_rope`` wide while value heads are ``v_head_dim`` wide; the flash
kernels here handle equal widths of 64 or 128, so the score and value products of this layer run through the dense
attention reference (library matmuls) — an MLA kernel is open work.
"""

from __future__ import annotations

import torch
from torch import nn

from ..ops import functional as F
from ..ops import reference as R
from .linears import ColumnParallelLinear, RowParallelLinear
from .norms import RMSNorm
from .rotary import get_rope


class MLACache:
    def __init__(self, num_layers: int, batch: int, max_len: int, kv_lora_rank: int, rope_dim: int,
                 dtype=torch.bfloat16, device=None):
        self.latent = torch.zeros(num_layers, batch, max_len, kv_lora_rank, dtype=dtype, device=device)
        self.k_rope = torch.zeros(num_layers, batch, max_len, rope_dim, dtype=dtype, device=device)
        self.length, self.max_len = 0, max_len
        self.linear: dict[int, object] = {}     # layer -> recurrent state of a linear-attention layer (hybrids)
        self.index_keys: dict[int, torch.Tensor] = {}   # layer -> keys of the sparse-attention scorer seen so far

    def seq_len(self) -> int:
        return self.length

    def advance(self, n: int) -> None:
        self.length += n

    def view(self, layer: int):
        return _MLAView(self, layer)

    def reorder(self, index: torch.Tensor) -> None:
        self.latent = self.latent.index_select(1, index)
        self.k_rope = self.k_rope.index_select(1, index)
        for st in self.linear.values():
            st.reorder(index)


class _MLAView:
    def __init__(self, cache: MLACache, layer: int):
        self.cache, self.layer = cache, layer

    @property
    def linear_state(self):
        return self.cache.linear.get(self.layer)

    def update(self, latent: torch.Tensor, k_rope: torch.Tensor):
        c = self.cache
        T = latent.shape[1]
        s, e = c.length, c.length + T
        if e > c.max_len:
            raise ValueError(f"MLA cache overflow: {e} > {c.max_len}")
        c.latent[self.layer, :, s:e] = latent
        c.k_rope[self.layer, :, s:e] = k_rope
        return c.latent[self.layer, :, :e], c.k_rope[self.layer, :, :e]


class MLAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, *, q_lora_rank: int | None, kv_lora_rank: int,
                 qk_nope_head_dim: int, qk_rope_head_dim: int, v_head_dim: int, rope: dict, rope_interleave: bool = True,
                 norm_eps: float = 1e-6, bias: bool = False, scale: float | None = None, layer_idx: int = 0,
                 dtype=torch.bfloat16, init_std: float = 0.02, tp_size: int = 1, tp_rank: int = 0, tp_group=None,
                 use_rope: bool = True, indexer: dict | None = None):
        super().__init__()
        # DeepSeek sparse attention (GLM-MoE-DSA): a light scorer ranks the keys of every query and attention runs
        # over the ``topk`` best ones only; kwargs: n_heads, head_dim, topk
        self.indexer_cfg = indexer
        self.use_rope = use_rope        # Kimi-Linear's latent layers carry no positions (``mla_use_nope``)
        self.H, self.nope, self.rope_dim, self.vd = num_heads // tp_size, qk_nope_head_dim, qk_rope_head_dim, v_head_dim
        self.qk_dim = qk_nope_head_dim + qk_rope_head_dim
        self.kv_lora_rank, self.layer_idx, self.interleave = kv_lora_rank, layer_idx, rope_interleave
        self.scale = scale if scale is not None else self.qk_dim ** -0.5
        self.sliding_window, self.softcap, self.sinks = None, 0.0, None
        kw = dict(dtype=dtype, init_std=init_std)
        if q_lora_rank:
            self.q_a_proj = ColumnParallelLinear(hidden_size, q_lora_rank, bias=bias, **kw)
            self.q_a_layernorm = RMSNorm(q_lora_rank, norm_eps, dtype)
            self.q_b_proj = ColumnParallelLinear(q_lora_rank, num_heads * self.qk_dim, bias=False, tp_size=tp_size,
                                                 tp_rank=tp_rank, tp_group=tp_group, **kw)
            self.q_proj = None
        else:
            self.q_proj = ColumnParallelLinear(hidden_size, num_heads * self.qk_dim, bias=False, tp_size=tp_size,
                                               tp_rank=tp_rank, tp_group=tp_group, **kw)
        self.kv_a_proj_with_mqa = ColumnParallelLinear(hidden_size, kv_lora_rank + qk_rope_head_dim, bias=bias, **kw)
        self.kv_a_layernorm = RMSNorm(kv_lora_rank, norm_eps, dtype)
        self.kv_b_proj = ColumnParallelLinear(kv_lora_rank, num_heads * (qk_nope_head_dim + v_head_dim), bias=False,
                                              tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group, **kw)
        self.o_proj = RowParallelLinear(num_heads * v_head_dim, hidden_size, bias=bias, tp_size=tp_size,
                                        tp_rank=tp_rank, tp_group=tp_group, **kw)
        self.rotary = get_rope(head_size=qk_rope_head_dim, **rope)
        if indexer is not None:
            from .norms import LayerNorm

            ih, idim = indexer["n_heads"], indexer["head_dim"]
            self.indexer = nn.Module()
            self.indexer.wq_b = ColumnParallelLinear(q_lora_rank, ih * idim, bias=False, **kw)
            self.indexer.wk = ColumnParallelLinear(hidden_size, idim, bias=False, **kw)
            self.indexer.k_norm = LayerNorm(idim, 1e-6, dtype=dtype)
            self.indexer.weights_proj = ColumnParallelLinear(hidden_size, ih, bias=False, **kw)

    def _index_bias(self, hidden, q_resid, positions, cache_view, Tk):
        """Additive mask ``[B, 1, T, Tk]``: 0 at the ``topk`` keys the scorer ranks highest for each query (among
        the causally visible ones), -inf elsewhere. Score: ``sum_h w_h relu(q_h . k) / sqrt(d)`` with rotary
        (half-split layout) on the first ``rope_dim`` channels of the scorer's own q / k."""
        cfg = self.indexer_cfg
        B, T, _ = hidden.shape
        ih, idim, rd = cfg["n_heads"], cfg["head_dim"], self.rope_dim
        cos, sin = self.rotary.tables(hidden.device)
        pos = positions.reshape(-1) if positions.numel() == B * T else positions.expand(B, T).reshape(-1)

        def rot(x):       # x [B, T, h, idim]
            h = x.shape[2]
            xr = R.apply_rope(x[..., :rd].reshape(B * T, h, rd), pos, cos, sin, rd, False).view(B, T, h, rd)
            return torch.cat([xr, x[..., rd:]], -1)

        q = rot(self.indexer.wq_b(q_resid).view(B, T, ih, idim))
        k = rot(self.indexer.k_norm(self.indexer.wk(hidden))[:, :, None, :])[:, :, 0]
        if cache_view is not None:
            store = cache_view.cache.index_keys
            prev = store.get(cache_view.layer)
            k = k if prev is None or T > 1 and cache_view.cache.length == 0 else torch.cat([prev, k], 1)
            store[cache_view.layer] = k
        w = self.indexer.weights_proj(hidden).float() * ih ** -0.5
        sc = torch.relu(torch.einsum("bshd,btd->bsht", q.float(), k.float()) * idim ** -0.5)
        score = torch.einsum("bsht,bsh->bst", sc, w)
        qpos = torch.arange(Tk - T, Tk, device=hidden.device)[:, None]
        visible = torch.arange(Tk, device=hidden.device)[None, :] <= qpos
        score = score.masked_fill(~visible[None], float("-inf"))
        top = score.topk(min(cfg["topk"], Tk), dim=-1).indices
        bias = torch.full((B, T, Tk), float("-inf"), device=hidden.device)
        bias.scatter_(-1, top, 0.0)
        return bias[:, None]

    def _rope(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """x ``[B, T, h, rope_dim]``. Checkpoints with ``rope_interleave`` store pairs interleaved: de-interleave,
        then rotate in the half-split layout (what the Hugging Face implementation does)."""
        if not self.use_rope:
            return x
        if self.interleave:
            B, T, h, d = x.shape
            x = x.view(B, T, h, d // 2, 2).transpose(-1, -2).reshape(B, T, h, d)
        cos, sin = self.rotary.tables(x.device)
        B, T, h, d = x.shape
        pos = positions.reshape(-1) if positions.numel() == B * T else positions.expand(B, T).reshape(-1)
        return R.apply_rope(x.reshape(B * T, h, d), pos, cos, sin, d, False).view(B, T, h, d)

    def forward(self, hidden, positions, *, segment_ids=None, cache_view=None, attn_meta=None, **_):
        B, T, _ = hidden.shape
        q_resid = None
        if self.q_proj is None:
            q_resid = self.q_a_layernorm(self.q_a_proj(hidden))
            q = self.q_b_proj(q_resid)
        else:
            q = self.q_proj(hidden)
        q = q.view(B, T, self.H, self.qk_dim)
        q_nope, q_rope = q[..., : self.nope], q[..., self.nope:]
        ckv = self.kv_a_proj_with_mqa(hidden)
        latent = self.kv_a_layernorm(ckv[..., : self.kv_lora_rank].contiguous())
        k_rope = self._rope(ckv[..., self.kv_lora_rank:].reshape(B, T, 1, self.rope_dim), positions)[:, :, 0]
        q_rope = self._rope(q_rope, positions)
        kv_seg = None
        if cache_view is not None and hasattr(cache_view, "attend_latent"):      # paged serving cache
            if self.indexer_cfg is not None:
                raise NotImplementedError("sparse-index latent attention is not wired into the paged serving cache")
            o = cache_view.attend_latent(self, q_nope, q_rope, latent, k_rope, attn_meta)
            return self.o_proj(o.reshape(B, T, self.H * self.vd).to(hidden.dtype))
        if cache_view is not None:
            if not hasattr(cache_view, "update"):
                raise TypeError("latent attention needs an MLACache (model.init_cache builds one)")
            latent, k_rope = cache_view.update(latent, k_rope)
            if attn_meta is not None and attn_meta.get("kv_segment_ids") is not None:
                kv_seg = attn_meta["kv_segment_ids"][:, : latent.shape[1]]
        Tk = latent.shape[1]
        kv = self.kv_b_proj(latent).view(B, Tk, self.H, self.nope + self.vd)
        k = torch.cat([kv[..., : self.nope], k_rope[:, :, None, :].expand(B, Tk, self.H, self.rope_dim)], -1)
        v = kv[..., self.nope:]
        qf = torch.cat([q_nope, q_rope], -1)
        if self.indexer_cfg is not None:
            bias = self._index_bias(hidden, q_resid, positions, cache_view, Tk)
            o = R.attention(qf, k, v, causal=True, scale=self.scale, bias=bias)
            return self.o_proj(o.reshape(B, T, self.H * self.vd).to(hidden.dtype))
        if kv_seg is not None:
            o = R.attention(qf, k, v, causal=True, scale=self.scale, segment_ids=kv_seg[:, Tk - T:],
                            kv_segment_ids=kv_seg)
        else:
            # 192-wide keys with 128-wide values are outside the flash kernels: the dispatcher picks the fused
            # library attention for them on a GPU and the dense form on CPU
            o = F.attention(qf, k, v, causal=True, scale=self.scale, segment_ids=segment_ids)
        return self.o_proj(o.reshape(B, T, self.H * self.vd).to(hidden.dtype))
