"""Mamba-2 (SSD) mixer used beside attention in hybrid blocks (Falcon-H1, easydel/modules/falcon_h1).

``in_proj`` emits ``[gate z | x | B | C | dt]``; each section has its own fixed multiplier (a muP vector), the
``[x | B | C]`` part goes through a depth-wise causal convolution + SiLU, the SSD scan mixes along the sequence, and the
result is gated by ``silu(z)`` (optionally through a grouped RMSNorm) before ``out_proj``. The scan and the convolution
are the CUDA kernels of ``ops/ssm.py``.
"""

from __future__ import annotations

import torch
from torch import nn

from ..ops import ssm
from .linears import ColumnParallelLinear, RowParallelLinear


class SSMState:
    def __init__(self, batch, conv_dim, conv_width, heads, head_dim, state, dtype, device):
        self.conv = torch.zeros(batch, conv_width - 1, conv_dim, dtype=dtype, device=device)
        self.ssm = torch.zeros(batch, heads, head_dim, state, dtype=torch.float32, device=device)

    def reorder(self, index):
        self.conv, self.ssm = self.conv.index_select(0, index), self.ssm.index_select(0, index)


class SSDMixer(nn.Module):
    def __init__(self, hidden_size: int, d_ssm: int, num_heads: int, head_dim: int, n_groups: int, d_state: int,
                 d_conv: int = 4, conv_bias: bool = True, proj_bias: bool = False, rms_norm: bool = False,
                 norm_before_gate: bool = True, norm_eps: float = 1e-5, multipliers=(1.0,) * 5,
                 in_multiplier: float = 1.0, layer_idx: int = 0, dtype=torch.float32, init_std: float = 0.02):
        super().__init__()
        self.I, self.NH, self.P, self.G, self.N, self.W = d_ssm, num_heads, head_dim, n_groups, d_state, d_conv
        self.conv_dim = d_ssm + 2 * n_groups * d_state
        self.in_multiplier, self.eps = in_multiplier, norm_eps
        self.rms_norm, self.norm_before_gate = rms_norm, norm_before_gate
        self.in_proj = ColumnParallelLinear(hidden_size, d_ssm + self.conv_dim + num_heads, bias=proj_bias,
                                            dtype=dtype, init_std=init_std)
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, d_conv, groups=self.conv_dim, padding=d_conv - 1,
                                bias=conv_bias, dtype=dtype)
        self.dt_bias = nn.Parameter(torch.ones(num_heads, dtype=dtype))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, num_heads + 1, dtype=torch.float32)).to(dtype))
        self.D = nn.Parameter(torch.ones(num_heads, dtype=dtype))
        if rms_norm:
            self.norm = nn.Module()
            self.norm.weight = nn.Parameter(torch.ones(d_ssm, dtype=dtype))
        self.out_proj = RowParallelLinear(d_ssm, hidden_size, bias=proj_bias, dtype=dtype, init_std=init_std)
        gn = n_groups * d_state
        v = torch.ones(d_ssm + self.conv_dim + num_heads)
        for (a, b), m in zip(((0, d_ssm), (d_ssm, 2 * d_ssm), (2 * d_ssm, 2 * d_ssm + gn),
                              (2 * d_ssm + gn, 2 * d_ssm + 2 * gn), (2 * d_ssm + 2 * gn, v.numel())), multipliers):
            v[a:b] *= m
        self.register_buffer("mup_vector", v, persistent=False)

    def make_state(self, batch, dtype, device) -> SSMState:
        return SSMState(batch, self.conv_dim, self.W, self.NH, self.P, self.N, dtype, device)

    def _gated(self, y, z):
        if not self.rms_norm:
            return y * torch.nn.functional.silu(z.float()).to(y.dtype)
        yf, zf = y.float(), torch.nn.functional.silu(z.float())
        if not self.norm_before_gate:
            yf = yf * zf
        g = yf.view(*yf.shape[:-1], self.G, -1)
        g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + self.eps)
        yf = g.view(yf.shape) * self.norm.weight.float()
        if self.norm_before_gate:
            yf = yf * zf
        return yf.to(y.dtype)

    def forward(self, h, segment_ids=None, state: SSMState | None = None):
        B, T, _ = h.shape
        I, G, N, NH, P = self.I, self.G, self.N, self.NH, self.P
        proj = self.in_proj(h * self.in_multiplier) * self.mup_vector.to(h.dtype)
        z, xbc, dt = proj[..., :I], proj[..., I:I + self.conv_dim], proj[..., I + self.conv_dim:]
        if segment_ids is not None and state is None:
            from ..ops.attention import segment_ids_to_cu_seqlens

            cu, _ = segment_ids_to_cu_seqlens(segment_ids)
        else:
            cu = getattr(state, "cu", None)       # a serving state names its own (ragged) sequence bounds
            if cu is None:
                cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=h.device)
        xbc = ssm.ragged_conv1d(xbc.reshape(B * T, self.conv_dim), self.conv1d.weight[:, 0, :], self.conv1d.bias, cu,
                                "silu", None if state is None else state.conv)
        x, Bm, Cm = xbc[:, :I], xbc[:, I:I + G * N], xbc[:, I + G * N:]
        y = ssm.ssd_scan(x.reshape(B * T, NH, P).contiguous(), dt.reshape(B * T, NH).contiguous(),
                         -torch.exp(self.A_log.float()), Bm.reshape(B * T, G, N).contiguous(),
                         Cm.reshape(B * T, G, N).contiguous(), self.D, self.dt_bias, True, cu,
                         None if state is None else state.ssm)
        return self.out_proj(self._gated(y.reshape(B, T, I), z))
