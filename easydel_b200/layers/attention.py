"""Self-attention layer shared by every decoder family.

One class covers what the reference's ``UnifiedAttention`` does for standard attention
(easydel/layers/attention/_unified.py:290-340, forward at :1048-1174): fused QKV projection,
optional QK-norm, rotary embedding, GQA, sliding window, logit soft-cap, attention sinks, ALiBi,
then the attention operator chosen by the execution mode:

* training / full-sequence forward: flash attention kernels (``ops.functional.attention``);
* ``generate()`` with a dense cache: the same kernel over the cache contents (queries aligned
  to the end of the keys);
* eSurge serving: the paged cache view appends K/V into pages and runs the paged attention
  kernels (``caching.paged``).
"""

from __future__ import annotations

import math
import typing as tp

import torch
from torch import nn

from ..ops import functional as F
from .linears import ColumnParallelLinear, RowParallelLinear
from .norms import LayerNorm, RMSNorm
from .rotary import get_rope


def alibi_slopes(n_heads: int) -> torch.Tensor:
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]

    if math.log2(n_heads).is_integer():
        return torch.tensor(pow2(n_heads), dtype=torch.float32)
    c = 2 ** math.floor(math.log2(n_heads))
    return torch.tensor(pow2(c) + pow2(2 * c)[0::2][: n_heads - c], dtype=torch.float32)


class _PerHeadLayerNorm(nn.Module):
    """Bias-free LayerNorm over the last axis with a separate scale vector per head."""

    def __init__(self, heads: int, head_dim: int, eps: float, dtype, tp_size: int = 1, tp_rank: int = 0):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(heads, head_dim, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:   # [..., heads, head_dim]
        xf = x.float()
        mean = xf.mean(-1, keepdim=True)
        var = (xf - mean).pow(2).mean(-1, keepdim=True)
        return ((xf - mean) * torch.rsqrt(var + self.eps) * self.weight.float()).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, *, layer_idx: int = 0,
                 bias: bool = False, o_bias: bool = False, qk_norm: str | None = None, qk_norm_eps: float = 1e-6,
                 rope: dict | None = None, sliding_window: int | None = None, softcap: float = 0.0,
                 scale: float | None = None, use_sinks: bool = False, use_alibi: bool = False, causal: bool = True,
                 clip_qkv: float | None = None, dtype: torch.dtype = torch.float32, init_std: float = 0.02,
                 tp_size: int = 1, tp_rank: int = 0, tp_group=None, qk_norm_offset: float = 0.0,
                 output_gate: bool = False, chunk_size: int | None = None,
                 temp_tuning: tuple[float, float] | None = None, head_scale_init: float | None = None):
        super().__init__()
        # GIDD: one learned multiplier per query head on top of ``scale`` (with L2-normalised q / k it is the whole
        # temperature of the head)
        self.head_scale = None if head_scale_init is None else nn.Parameter(
            torch.full((num_heads // tp_size,), float(head_scale_init), dtype=dtype))
        self.layer_idx = layer_idx
        # Llama-4: attention restricted to blocks of ``chunk_size`` positions (rotary layers); position-dependent
        # query temperature ``log1p(floor((pos + 1) / floor_scale)) * attn_scale + 1`` (layers without rotary)
        self.chunk_size, self.temp_tuning = chunk_size, temp_tuning
        # Qwen3-Next: the query projection also emits a per-channel gate ([q (D) | gate (D)] per head); the
        # attention output is multiplied by sigmoid(gate) before the output projection
        self.output_gate = output_gate
        self.hidden_size = hidden_size
        self.num_heads_global, self.num_kv_heads_global = num_heads, num_kv_heads
        if num_heads % tp_size:
            raise ValueError(f"num_heads {num_heads} not divisible by tp {tp_size}")
        # KV heads are split when there are enough of them, replicated otherwise
        self.kv_replicated = num_kv_heads % tp_size != 0
        if self.kv_replicated and tp_size % num_kv_heads:
            raise ValueError(f"cannot place {num_kv_heads} KV heads on tp={tp_size}")
        self.num_heads = num_heads // tp_size
        self.num_kv_heads = max(1, num_kv_heads // tp_size)
        self.head_dim = head_dim
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.sliding_window = sliding_window
        self.softcap = softcap
        self.causal = causal
        self.clip_qkv = clip_qkv
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
        kv_out = num_kv_heads * head_dim if not self.kv_replicated else self.num_kv_heads * head_dim * tp_size
        self.qkv_proj = ColumnParallelLinear(hidden_size, (num_heads * head_dim * (2 if output_gate else 1), kv_out,
                                                           kv_out), bias=bias,
                                             dtype=dtype, init_std=init_std, tp_size=tp_size, tp_rank=tp_rank,
                                             tp_group=tp_group)
        self.o_proj = RowParallelLinear(num_heads * head_dim, hidden_size, bias=o_bias, dtype=dtype,
                                        init_std=init_std, tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group)
        self.qkv_proj.remat_name, self.o_proj.remat_name = "attn_qkv", "attn_output"
        self.qk_norm, self.qk_norm_eps = qk_norm, qk_norm_eps
        if qk_norm == "rms_head":      # per-head RMSNorm over head_dim (Qwen3, Gemma3, OLMo... per-head flavour)
            self.q_norm = RMSNorm(head_dim, qk_norm_eps, dtype, offset=qk_norm_offset)
            self.k_norm = RMSNorm(head_dim, qk_norm_eps, dtype, offset=qk_norm_offset)
        elif qk_norm == "rms_full":    # RMSNorm over the whole projection (OLMo2, Cohere-style full width)
            self.q_norm = RMSNorm(self.num_heads * head_dim, qk_norm_eps, dtype)
            self.k_norm = RMSNorm(self.num_kv_heads * head_dim, qk_norm_eps, dtype)
        elif qk_norm == "layer_head":  # per-head LayerNorm without bias (Cohere, StableLM per-head)
            self.q_norm = LayerNorm(head_dim, qk_norm_eps, bias=False, dtype=dtype)
            self.k_norm = LayerNorm(head_dim, qk_norm_eps, bias=False, dtype=dtype)
        elif qk_norm == "layer_perhead":  # LayerNorm over head_dim with one scale row per head (Cohere)
            self.q_norm = _PerHeadLayerNorm(self.num_heads, head_dim, qk_norm_eps, dtype, tp_size, tp_rank)
            self.k_norm = _PerHeadLayerNorm(self.num_kv_heads, head_dim, qk_norm_eps, dtype,
                                            1 if self.kv_replicated else tp_size, tp_rank)
        self.rotary = None
        if rope is not None:
            self.rotary = get_rope(head_size=head_dim, **rope)
        self.sinks = nn.Parameter(torch.zeros(self.num_heads, dtype=torch.float32)) if use_sinks else None
        if use_alibi:
            sl = alibi_slopes(num_heads)[tp_rank * self.num_heads:(tp_rank + 1) * self.num_heads]
            self.register_buffer("alibi", sl, persistent=False)
        else:
            self.alibi = None

    # ------------------------------------------------------------------
    #: set by the decoder when the sequence is sharded over the ``sp`` mesh axis (``attn_mechanism="ring"``)
    cp_group = None
    cp_layout = "zigzag"
    cp_impl = "auto"

    def _split(self, qkv: torch.Tensor):
        B, T, _ = qkv.shape
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        return F.split_qkv(qkv, Hq, Hkv, D)

    def _apply_qk_norm(self, qkv: torch.Tensor) -> torch.Tensor:
        B, T, W = qkv.shape
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        q, k, v = qkv[..., : Hq * D], qkv[..., Hq * D:(Hq + Hkv) * D], qkv[..., (Hq + Hkv) * D:]
        if self.qk_norm in ("rms_head", "layer_head", "layer_perhead"):
            q = self.q_norm(q.reshape(B, T, Hq, D)).reshape(B, T, Hq * D)
            k = self.k_norm(k.reshape(B, T, Hkv, D)).reshape(B, T, Hkv * D)
        else:
            q = self.q_norm(q.contiguous())
            k = self.k_norm(k.contiguous())
        return torch.cat([q, k, v], dim=-1)

    def forward(self, hidden: torch.Tensor, positions: torch.Tensor, *, segment_ids: torch.Tensor | None = None,
                cache_view=None, attn_meta=None, cu_seqlens=None, max_seqlen=None) -> torch.Tensor:
        """hidden ``[B,T,H]``; positions ``[B,T]``. Returns ``[B,T,H]``."""
        qkv = self.qkv_proj(hidden)
        B, T = qkv.shape[0], qkv.shape[1]   # a sequence-parallel block hands in row shards and gets [B, T] back
        if self.qk_norm == "l2_full":     # q and k are normalised over the whole projection (all heads together)
            Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
            q, k, v = qkv[..., : Hq * D].float(), qkv[..., Hq * D:(Hq + Hkv) * D].float(), qkv[..., (Hq + Hkv) * D:]
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + self.qk_norm_eps)
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + self.qk_norm_eps)
            qkv = torch.cat([q.to(v.dtype), k.to(v.dtype), v], dim=-1)
        gate = None
        if self.output_gate:
            Hq, D = self.num_heads, self.head_dim
            qg = qkv[..., : 2 * Hq * D].view(B, T, Hq, 2 * D)
            gate = qg[..., D:].reshape(B, T, Hq * D)
            qkv = torch.cat([qg[..., :D].reshape(B, T, Hq * D), qkv[..., 2 * Hq * D:]], dim=-1)
        if self.clip_qkv is not None:
            qkv = qkv.clamp(-self.clip_qkv, self.clip_qkv)
        if self.qk_norm is not None and self.qk_norm not in ("l2_post_rope", "l2_full"):
            qkv = self._apply_qk_norm(qkv)
        if self.rotary is not None and positions.dim() == 3:
            # three position streams (temporal, height, width) share the frequency axis by sections
            q, k, v = self._split(qkv)
            q, k = self.rotary(positions, q, k)
            positions = positions[0]
        else:
            if self.rotary is not None:
                # serving: the projection's output is consumed here only, so it is rotated where it lies
                qkv = self.rotary.rotate_packed(qkv, positions, self.num_heads + self.num_kv_heads,
                                                inplace=cache_view is not None and not torch.is_grad_enabled())
            q, k, v = self._split(qkv)
        if self.head_scale is not None:
            q = (q * self.head_scale.to(q.dtype)[None, None, :, None])
        if self.qk_norm == "l2_post_rope":      # weightless RMS normalisation of every head, after the rotation
            q = (q.float() * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + self.qk_norm_eps)).to(v.dtype)
            k = (k.float() * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + self.qk_norm_eps)).to(v.dtype)
        if self.temp_tuning is not None:
            a_scale, floor_scale = self.temp_tuning
            t = torch.log1p(torch.floor((positions.float() + 1.0) / floor_scale)) * a_scale + 1.0
            q = (q * t[..., None, None]).to(v.dtype)
        if self.chunk_size and cache_view is None and T > 1:
            # a block-diagonal causal mask is a segment mask: (document, position // chunk) names the segment
            blocks = positions // self.chunk_size
            base = segment_ids.long() if segment_ids is not None else torch.ones_like(blocks)
            if int(blocks.max()) > 0:
                segment_ids = (base * (int(blocks.max()) + 1) + blocks).to(torch.int32) * (base != 0)
        if cache_view is not None:
            o = cache_view.attend(self, q, k, v, positions=positions, attn_meta=attn_meta)
        elif self.cp_group is not None:
            if segment_ids is not None or self.sliding_window or self.sinks is not None or self.alibi is not None \
                    or self.chunk_size:
                raise NotImplementedError("sequence-parallel (ring) attention covers plain causal / full attention: "
                                          "no packed segments, windows, sinks or position biases")
            from ..parallel import context_parallel as CP

            o = CP.ring_attention(q.contiguous(), k.contiguous(), v.contiguous(), self.cp_group,
                                  layout=self.cp_layout, causal=self.causal, scale=self.scale,
                                  softcap=self.softcap or 0.0, impl=self.cp_impl)
        elif self.alibi is not None:
            o = self._alibi_attention(q, k, v, segment_ids)
        else:
            o = F.attention(q, k, v, causal=self.causal, scale=self.scale, segment_ids=segment_ids,
                            sliding_window=self.sliding_window, softcap=self.softcap, sinks=self.sinks,
                            cu_seqlens=cu_seqlens)
        o = o.reshape(B, T, self.num_heads * self.head_dim)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.o_proj(o)

    def _alibi_attention(self, q, k, v, segment_ids):
        # ALiBi families (Falcon-RW, MPT, BLOOM-style) are served by the dense oracle path: a
        # position-dependent bias has no slot in the flash kernels.
        from ..ops import reference as R

        Tq, Tk = q.shape[1], k.shape[1]
        rel = (torch.arange(Tk, device=q.device)[None, :] - torch.arange(Tq, device=q.device)[:, None] - (Tk - Tq))
        bias = self.alibi.to(q.device)[None, :, None, None] * rel[None, None].float()
        return R.attention(q, k, v, causal=self.causal, scale=self.scale, segment_ids=segment_ids, bias=bias)


AttentionModule = Attention      # the name model code uses for its attention base class
