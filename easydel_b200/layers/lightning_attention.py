"""Lightning attention (MiniMax, easydel/modules/minimax): linear attention with a fixed per-head exponential decay,
``o_t = sum_{s<=t} e^{-lambda_h (t - s)} (q_t . k_s) v_s`` with ``q, k, v = silu(qkv_proj(x))`` and no softmax; the
result goes through an RMSNorm over all heads and a sigmoid output gate.

The recurrence ``S_t = e^{-lambda} S_{t-1} + v_t k_t^T, o_t = S_t q_t`` is the Mamba-2 state-space scan with a unit
time step (``x = v``, ``B = k``, ``C = q``, ``A = -lambda``), so it runs on the SSD scan kernel of ``ops/ssm.py``.
The decay tables of the block-wise formulation that checkpoints carry as buffers are kept for checkpoint parity.
"""

from __future__ import annotations

import torch
from torch import nn

from ..ops import ssm
from .linears import ColumnParallelLinear, RowParallelLinear
from .norms import RMSNorm


class LightningState:
    def __init__(self, batch, heads, head_dim, device):
        self.kv = torch.zeros(batch, heads, head_dim, head_dim, dtype=torch.float32, device=device)

    def reorder(self, index):
        self.kv = self.kv.index_select(0, index)


class LightningAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, num_layers: int, block_size: int = 256,
                 act: str = "silu", norm_eps: float = 1e-6, layer_idx: int = 0, dtype=torch.float32,
                 init_std: float = 0.02):
        super().__init__()
        from ..ops.reference import ACT2FN

        self.h, self.d, self.act = num_heads, head_dim, ACT2FN[act]
        inner = num_heads * head_dim
        # named apart from the split-able ``qkv_proj`` of softmax layers: checkpoints keep this matrix fused, per head [q|k|v]
        self.lqkv = ColumnParallelLinear(hidden_size, 3 * inner, bias=False, dtype=dtype, init_std=init_std)
        self.out_proj = RowParallelLinear(inner, hidden_size, bias=False, dtype=dtype, init_std=init_std)
        self.output_gate = ColumnParallelLinear(hidden_size, inner, bias=False, dtype=dtype, init_std=init_std)
        self.norm = RMSNorm(inner, norm_eps, dtype)
        base = 1 / (2 ** (8 / num_heads))
        rate = base ** (torch.arange(num_heads) + 1.0) * (1 - layer_idx / (num_layers - 1 + 1e-5) + 1e-5)
        rate = rate[:, None, None].float()
        r = torch.arange(block_size) + 1.0
        diag = rate * (r[:, None] - r[None, :])[None, None]
        self.register_buffer("slope_rate", rate)
        self.register_buffer("query_decay", torch.exp(-rate * r[:, None]))
        self.register_buffer("key_decay", torch.exp(-rate * (block_size - r[:, None])))
        self.register_buffer("diagonal_decay", torch.exp(torch.where(diag >= 0, -diag, float("-inf"))))

    def make_state(self, batch, dtype, device) -> LightningState:
        return LightningState(batch, self.h, self.d, device)

    def forward(self, hidden, segment_ids=None, state: LightningState | None = None):
        B, T, _ = hidden.shape
        qkv = self.act(self.lqkv(hidden)).view(B * T, self.h, 3 * self.d)
        q, k, v = torch.split(qkv, self.d, dim=-1)
        if segment_ids is not None and state is None:
            from ..ops.attention import segment_ids_to_cu_seqlens

            cu, _ = segment_ids_to_cu_seqlens(segment_ids)
        else:
            cu = getattr(state, "cu", None)       # a serving state names its own (ragged) sequence bounds
            if cu is None:
                cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=hidden.device)
        ones = torch.ones(B * T, self.h, dtype=v.dtype, device=v.device)
        o = ssm.ssd_scan(v.contiguous(), ones, -self.slope_rate.view(-1).float(), k.contiguous(), q.contiguous(),
                         None, None, False, cu, None if state is None else state.kv)
        o = self.norm(o.reshape(B, T, self.h * self.d))
        return self.out_proj(torch.sigmoid(self.output_gate(hidden)) * o)
