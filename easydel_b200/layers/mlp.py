"""Feed-forward blocks: gated (SwiGLU / GeGLU) and plain two-layer MLPs."""

from __future__ import annotations

import torch
from torch import nn

from ..ops import functional as F
from ..ops.reference import ACT2FN
from .linears import ColumnParallelLinear, RowParallelLinear


class GatedMLP(nn.Module):
    """``down(act(gate(x)) * up(x))`` with gate and up fused into one column-parallel GEMM
    (the Llama MLP of easydel/modules/llama/modeling_llama.py:48-127)."""

    def __init__(self, hidden_size: int, intermediate_size: int, act: str = "silu", bias: bool = False,
                 dtype: torch.dtype = torch.float32, init_std: float = 0.02, tp_size: int = 1, tp_rank: int = 0,
                 tp_group=None):
        super().__init__()
        self.act = act
        self.gate_up_proj = ColumnParallelLinear(hidden_size, (intermediate_size, intermediate_size), bias=bias,
                                                 dtype=dtype, init_std=init_std, tp_size=tp_size, tp_rank=tp_rank,
                                                 tp_group=tp_group)
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias=bias, dtype=dtype, init_std=init_std,
                                           tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group)
        self.gate_up_proj.remat_name, self.down_proj.remat_name = "mlp_gate_up", "mlp_down"

    # fixed muP multipliers on the gate pre-activation and on the output (Falcon-H1); 1.0 elsewhere
    gate_multiplier: float = 1.0
    down_multiplier: float = 1.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up_proj(x)
        if self.gate_multiplier != 1.0:
            half = gu.shape[-1] // 2
            gu = torch.cat([gu[..., :half] * self.gate_multiplier, gu[..., half:]], dim=-1)
        y = self.down_proj(F.gated_act(gu, self.act))
        return y if self.down_multiplier == 1.0 else y * self.down_multiplier


class PlainMLP(nn.Module):
    """``fc2(act(fc1(x)))`` (GPT-2, OPT, Falcon, GPT-NeoX, Phi, StarCoder...)."""

    def __init__(self, hidden_size: int, intermediate_size: int, act: str = "gelu", bias: bool = True,
                 dtype: torch.dtype = torch.float32, init_std: float = 0.02, tp_size: int = 1, tp_rank: int = 0,
                 tp_group=None):
        super().__init__()
        self.act = act
        self.fc1 = ColumnParallelLinear(hidden_size, intermediate_size, bias=bias, dtype=dtype, init_std=init_std,
                                        tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group)
        self.fc2 = RowParallelLinear(intermediate_size, hidden_size, bias=bias, dtype=dtype, init_std=init_std,
                                     tp_size=tp_size, tp_rank=tp_rank, tp_group=tp_group)
        self.fc1.remat_name, self.fc2.remat_name = "mlp_gate_up", "mlp_down"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(ACT2FN[self.act](self.fc1(x)))
