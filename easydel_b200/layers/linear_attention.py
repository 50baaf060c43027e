"""Gated DeltaNet token mixer (Qwen3-Next, easydel/modules/qwen3_next; the recurrence is the gated delta rule of
easydel/layers/operations: ``S_t = e^{g_t} S_{t-1} + k_t beta_t (v_t - k_t^T e^{g_t} S_{t-1})^T``, ``o_t = q_t^T S_t``).

``x -> [q | k | v | z] , [b | a]`` projections (grouped by key head as in the checkpoints), a depth-wise causal
convolution + SiLU over ``[q | k | v]``, L2-normalised q / k, ``beta = sigmoid(b)``, ``g = -exp(A_log) softplus(a + dt_bias)``,
the delta rule, a per-head RMSNorm gated by ``silu(z)``, and the output projection. Sequence state for incremental
decoding: the last ``W-1`` convolution inputs and the ``[H, DK, DV]`` fp32 recurrent state per sequence.
"""

from __future__ import annotations

import torch
from torch import nn

from ..ops import ssm
from .linears import ColumnParallelLinear, RowParallelLinear


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x / sqrt(sum(x^2) + eps)`` in fp32: the epsilon sits inside the root, which matters for small activations."""
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)


class LinearAttentionState:
    """Per-layer state of one batch of sequences."""

    def __init__(self, batch: int, conv_dim: int, conv_width: int, heads: int, dk: int, dv: int, dtype, device):
        self.conv = torch.zeros(batch, conv_width - 1, conv_dim, dtype=dtype, device=device)
        self.recurrent = torch.zeros(batch, heads, dk, dv, dtype=torch.float32, device=device)

    def reorder(self, index):
        self.conv = self.conv.index_select(0, index)
        self.recurrent = self.recurrent.index_select(0, index)


class GatedDeltaNet(nn.Module):
    def __init__(self, hidden_size: int, num_k_heads: int, num_v_heads: int, head_k_dim: int, head_v_dim: int,
                 conv_kernel: int = 4, norm_eps: float = 1e-6, layer_idx: int = 0, dtype=torch.float32,
                 init_std: float = 0.02, layout: str = "grouped"):
        """``layout="grouped"``: two fused projections ordered per key head (Qwen3-Next checkpoints);
        ``"flat"``: four projections ``[q | k | v]``, ``z``, ``b``, ``a`` in plain head order (Qwen3.5)."""
        super().__init__()
        self.layout = layout
        self.hk, self.hv, self.dk, self.dv = num_k_heads, num_v_heads, head_k_dim, head_v_dim
        self.rep = num_v_heads // num_k_heads
        self.key_dim, self.value_dim = head_k_dim * num_k_heads, head_v_dim * num_v_heads
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_kernel, self.eps, self.layer_idx = conv_kernel, norm_eps, layer_idx
        lin = lambda o: ColumnParallelLinear(hidden_size, o, bias=False, dtype=dtype, init_std=init_std)  # noqa: E731
        if layout == "grouped":
            self.in_proj_qkvz = lin(2 * self.key_dim + 2 * self.value_dim)
            self.in_proj_ba = lin(2 * num_v_heads)
        else:
            self.in_proj_qkv, self.in_proj_z = lin(2 * self.key_dim + self.value_dim), lin(self.value_dim)
            self.in_proj_b, self.in_proj_a = lin(num_v_heads), lin(num_v_heads)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, conv_kernel, groups=self.conv_dim, bias=False,
                                padding=conv_kernel - 1, dtype=dtype)
        self.dt_bias = nn.Parameter(torch.ones(num_v_heads, dtype=dtype))
        self.A_log = nn.Parameter(torch.log(torch.empty(num_v_heads).uniform_(1e-3, 16)).to(dtype))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(head_v_dim, dtype=dtype))
        self.out_proj = RowParallelLinear(self.value_dim, hidden_size, bias=False, dtype=dtype, init_std=init_std)

    def make_state(self, batch: int, dtype, device) -> LinearAttentionState:
        return LinearAttentionState(batch, self.conv_dim, self.conv_kernel, self.hv, self.dk, self.dv, dtype, device)

    def _split(self, qkvz, ba):
        """Checkpoint layout: per key head ``[q (dk) | k (dk) | v (rep*dv) | z (rep*dv)]`` and ``[b (rep) | a (rep)]``."""
        lead = qkvz.shape[:-1]
        r = self.rep
        x = qkvz.view(*lead, self.hk, 2 * self.dk + 2 * r * self.dv)
        q, k, v, z = torch.split(x, [self.dk, self.dk, r * self.dv, r * self.dv], dim=-1)
        y = ba.view(*lead, self.hk, 2 * r)
        b, a = torch.split(y, [r, r], dim=-1)
        return (q.reshape(*lead, self.key_dim), k.reshape(*lead, self.key_dim), v.reshape(*lead, self.value_dim),
                z.reshape(*lead, self.hv, self.dv), b.reshape(*lead, self.hv), a.reshape(*lead, self.hv))

    def forward(self, hidden: torch.Tensor, segment_ids: torch.Tensor | None = None, state=None) -> torch.Tensor:
        """hidden ``[B, T, H]``. ``segment_ids`` ``[B, T]`` restart the recurrence at packed-document boundaries (0 =
        padding, which then forms its own segment). ``state``: a :class:`LinearAttentionState` for incremental use."""
        B, T, _ = hidden.shape
        if self.layout == "grouped":
            q, k, v, z, b, a = self._split(self.in_proj_qkvz(hidden), self.in_proj_ba(hidden))
        else:
            q, k, v = torch.split(self.in_proj_qkv(hidden), [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            z = self.in_proj_z(hidden).view(B, T, self.hv, self.dv)
            b, a = self.in_proj_b(hidden), self.in_proj_a(hidden)
        mixed = torch.cat([q, k, v], -1).reshape(B * T, self.conv_dim)
        if segment_ids is not None and state is None:
            from ..ops.attention import segment_ids_to_cu_seqlens

            cu, _ = segment_ids_to_cu_seqlens(segment_ids)
        else:
            cu = getattr(state, "cu", None)       # a serving state names its own (ragged) sequence bounds
            if cu is None:
                cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=hidden.device)
        w = self.conv1d.weight.squeeze(1)
        mixed = ssm.ragged_conv1d(mixed, w, None, cu, "silu", None if state is None else state.conv)
        q, k, v = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k = _l2norm(q.reshape(B * T, self.hk, self.dk)), _l2norm(k.reshape(B * T, self.hk, self.dk))
        if self.rep > 1:
            q, k = q.repeat_interleave(self.rep, 1), k.repeat_interleave(self.rep, 1)
        v = v.reshape(B * T, self.hv, self.dv)
        beta = torch.sigmoid(b.reshape(B * T, self.hv).float())
        g = -self.A_log.float().exp() * torch.nn.functional.softplus(a.reshape(B * T, self.hv).float()
                                                                     + self.dt_bias.float())
        o = ssm.gated_delta_rule(q.to(v.dtype), k.to(v.dtype), v, g, beta, None, cu,
                                 None if state is None else state.recurrent)
        # per-head RMSNorm, gated by silu(z)
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.eps)
        of = (self.norm.weight.float() * of).to(hidden.dtype).float() * torch.nn.functional.silu(
            z.reshape(B * T, self.hv, self.dv).float())
        return self.out_proj(of.to(hidden.dtype).reshape(B, T, self.value_dim))


class KDAState:
    """Convolution windows of q, k, v and the recurrent state of one batch of sequences."""

    def __init__(self, batch, key_dim, value_dim, conv_width, heads, dk, dv, dtype, device):
        z = lambda c: torch.zeros(batch, conv_width - 1, c, dtype=dtype, device=device)  # noqa: E731
        self.q_conv, self.k_conv, self.v_conv = z(key_dim), z(key_dim), z(value_dim)
        self.recurrent = torch.zeros(batch, heads, dk, dv, dtype=torch.float32, device=device)

    def reorder(self, index):
        for n in ("q_conv", "k_conv", "v_conv", "recurrent"):
            setattr(self, n, getattr(self, n).index_select(0, index))


class KimiDeltaAttention(nn.Module):
    """Kimi delta attention (easydel/modules/kimi_linear/modeling_kimi_linear.py:830-1150): separate q / k / v
    projections each followed by its own depth-wise causal convolution + SiLU, the gated delta rule with a per-head
    decay ``-exp(A_log) softplus(f_b(silu(f_a x)) + dt_bias)`` (easydel/operations/kernels/kda.py:78-98) and update
    gate ``sigmoid(b x)``, L2-normalised q / k, then a per-head RMSNorm gated by ``silu(g_b(silu(g_a x)))``."""

    def __init__(self, hidden_size: int, num_heads: int, head_k_dim: int = 128, head_v_dim: int = 128,
                 d_conv: int = 4, gate_low_rank_dim: int = 128, norm_eps: float = 1e-6, layer_idx: int = 0,
                 dtype=torch.float32, init_std: float = 0.02):
        super().__init__()
        self.h, self.dk, self.dv, self.W, self.eps = num_heads, head_k_dim, head_v_dim, d_conv, norm_eps
        self.key_dim, self.value_dim = num_heads * head_k_dim, num_heads * head_v_dim
        lin = lambda i, o: ColumnParallelLinear(i, o, bias=False, dtype=dtype, init_std=init_std)  # noqa: E731
        self.q_proj, self.k_proj, self.v_proj = lin(hidden_size, self.key_dim), lin(hidden_size, self.key_dim), \
            lin(hidden_size, self.value_dim)
        conv = lambda c: nn.Conv1d(c, c, d_conv, groups=c, bias=False, padding=d_conv - 1, dtype=dtype)  # noqa: E731
        self.q_conv1d, self.k_conv1d, self.v_conv1d = conv(self.key_dim), conv(self.key_dim), conv(self.value_dim)
        self.f_a_proj, self.f_b_proj = lin(hidden_size, gate_low_rank_dim), lin(gate_low_rank_dim, num_heads)
        self.b_proj = lin(hidden_size, num_heads)
        self.g_a_proj, self.g_b_proj = lin(hidden_size, gate_low_rank_dim), lin(gate_low_rank_dim, self.value_dim)
        self.A_log = nn.Parameter(torch.log(torch.empty(num_heads).uniform_(1.0, 16.0)).to(dtype))
        self.dt_bias = nn.Parameter(torch.zeros(num_heads, dtype=dtype))
        self.o_norm = nn.Module()
        self.o_norm.weight = nn.Parameter(torch.ones(head_v_dim, dtype=dtype))
        self.o_proj = RowParallelLinear(self.value_dim, hidden_size, bias=False, dtype=dtype, init_std=init_std)

    def make_state(self, batch, dtype, device) -> KDAState:
        return KDAState(batch, self.key_dim, self.value_dim, self.W, self.h, self.dk, self.dv, dtype, device)

    def forward(self, hidden, segment_ids=None, state: KDAState | None = None):
        B, T, _ = hidden.shape
        if segment_ids is not None and state is None:
            from ..ops.attention import segment_ids_to_cu_seqlens

            cu, _ = segment_ids_to_cu_seqlens(segment_ids)
        else:
            cu = getattr(state, "cu", None)       # a serving state names its own (ragged) sequence bounds
            if cu is None:
                cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=hidden.device)

        def conv(x, mod, st):
            return ssm.ragged_conv1d(x.reshape(B * T, -1), mod.weight.squeeze(1), None, cu, "silu", st)

        q = conv(self.q_proj(hidden), self.q_conv1d, None if state is None else state.q_conv)
        k = conv(self.k_proj(hidden), self.k_conv1d, None if state is None else state.k_conv)
        v = conv(self.v_proj(hidden), self.v_conv1d, None if state is None else state.v_conv)
        q, k = _l2norm(q.view(B * T, self.h, self.dk)), _l2norm(k.view(B * T, self.h, self.dk))
        v = v.view(B * T, self.h, self.dv)
        gate = self.f_b_proj(torch.nn.functional.silu(self.f_a_proj(hidden))).reshape(B * T, self.h)
        g = -self.A_log.float().exp() * torch.nn.functional.softplus(gate.float() + self.dt_bias.float())
        beta = torch.sigmoid(self.b_proj(hidden).reshape(B * T, self.h).float())
        o = ssm.gated_delta_rule(q.to(v.dtype), k.to(v.dtype), v, g, beta, None, cu,
                                 None if state is None else state.recurrent)
        og = self.g_b_proj(torch.nn.functional.silu(self.g_a_proj(hidden))).reshape(B * T, self.h, self.dv)
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.eps) * self.o_norm.weight.float()
        of = of * torch.nn.functional.silu(og.float())
        return self.o_proj(of.to(hidden.dtype).reshape(B, T, self.value_dim))
