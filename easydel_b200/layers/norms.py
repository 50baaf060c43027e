"""Normalisation layers (easydel/layers/norms/_norms.py:93-727).

``RMSNorm`` keeps its weight under the attribute ``weight`` (HF naming; the checkpoint
writer stores it as ``kernel`` like the reference). Math runs in fp32 inside the fused
kernel for bf16 inputs.
"""

from __future__ import annotations

import torch
from torch import nn

from ..ops import functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype: torch.dtype = torch.float32, *, offset: float = 0.0,
                 device=None):
        super().__init__()
        self.dim, self.eps, self.offset = dim, eps, offset
        # Gemma stores (w - 1): offset = 1.0 and zero init
        init = torch.zeros if offset != 0.0 else torch.ones
        self.weight = nn.Parameter(init(dim, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, self.weight, self.eps, self.offset)

    def forward_with_residual(self, x, residual: torch.Tensor):
        """Returns (norm(x + residual), x + residual) from one kernel. ``x`` may be a pending tensor-parallel
        reduction, in which case the sum over ranks happens in the same kernel."""
        if hasattr(x, "add_rms_norm"):
            return x.add_rms_norm(residual, self.weight, self.eps, self.offset)
        return F.add_rms_norm(x, residual, self.weight, self.eps, self.offset)

    def extra_repr(self) -> str:
        return f"dim={self.dim}, eps={self.eps}" + (f", offset={self.offset}" if self.offset else "")


class RMSNormGated(nn.Module):
    """``rmsnorm(x * silu(gate))`` (Mamba-2 / Qwen3-Next style, _norms.py:274)."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype: torch.dtype = torch.float32, norm_before_gate: bool = False,
                 device=None):
        super().__init__()
        self.eps, self.norm_before_gate = eps, norm_before_gate
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
        if gate is not None and not self.norm_before_gate:
            x = x * torch.nn.functional.silu(gate.float()).to(x.dtype)
        y = F.rms_norm(x, self.weight, self.eps)
        if gate is not None and self.norm_before_gate:
            y = y * torch.nn.functional.silu(gate.float()).to(y.dtype)
        return y


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, bias: bool = True, dtype: torch.dtype = torch.float32,
                 elementwise_affine: bool = True, device=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device)) if elementwise_affine else None
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if (bias and elementwise_affine) else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x, self.weight, self.bias, self.eps)


class BatchNorm(nn.BatchNorm1d):
    """Feature-last batch norm used by a few vision towers (_norms.py:343)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 3:
            return super().forward(x.transpose(1, 2)).transpose(1, 2)
        return super().forward(x)
