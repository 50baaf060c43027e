"""Linear layers with column / row / replicated parallel styles.

The reference's ``ParallelLinear`` family (easydel/layers/linears/_linear.py:78-510) is an
einsum plus a sharding annotation. Here the style is metadata the runtime acts on:

* ``column``: output features are split over the tensor-parallel group (each rank owns
  ``out/tp`` rows of the ``[out, in]`` weight). The input is replicated, or, while the model
  runs a sequence-parallel block (``parallel.tp.SequenceParallelState``), row-sharded: then the
  all-gather of the rows happens inside the GEMM (``csrc/gemm_collective.cu``, all-gather -> GEMM),
  and the backward data-gradient product reduce-scatters its rows inside its GEMM.
* ``row``: input features are split (each rank owns ``in/tp`` columns); partial outputs are
  summed across the group: an all-reduce (NCCL, or the one-shot peer kernel for decode-size
  messages), or, in a sequence-parallel block, a reduce-scatter fused into the GEMM epilogue.
* The data-parallel / FSDP axes shard the flat parameter storage, not the module:
  see ``parallel.flat`` and ``parallel.dist_optim``.

Weights use the torch layout ``[out, in]``; the checkpoint writer transposes them to the
reference's ``kernel (in, out)`` on disk.
"""

from __future__ import annotations

import math
import typing as tp

import torch
from torch import nn

from ..ops import functional as F


class ParallelLinear(nn.Module):
    parallel_style = "replicated"
    # set by a model that can run its layers on sequence-sharded activations (``parallel.tp.SequenceParallelState``)
    sp_state = None
    # activation-checkpoint name of this product (``ops.remat``): set by the block that owns the layer
    remat_name: str | None = None

    def __init__(self, in_features: int, out_features: int | tp.Sequence[int], bias: bool = False, *,
                 dtype: torch.dtype = torch.float32, init_std: float | None = 0.02, tp_size: int = 1,
                 tp_rank: int = 0, tp_group=None, scale: float | str | None = None, device=None):
        super().__init__()
        self.out_splits = tuple(out_features) if not isinstance(out_features, int) else None
        out_total = sum(self.out_splits) if self.out_splits else int(out_features)
        self.in_features_global, self.out_features_global = in_features, out_total
        self.tp_size, self.tp_rank, self.tp_group = tp_size, tp_rank, tp_group
        in_local, out_local = in_features, out_total
        if tp_size > 1 and self.parallel_style == "column":
            if self.out_splits:
                if any(s % tp_size for s in self.out_splits):
                    raise ValueError(f"merged column outputs {self.out_splits} not divisible by tp={tp_size}")
                out_local = sum(s // tp_size for s in self.out_splits)
            else:
                if out_total % tp_size:
                    raise ValueError(f"out_features {out_total} not divisible by tp={tp_size}")
                out_local = out_total // tp_size
        elif tp_size > 1 and self.parallel_style == "row":
            if in_features % tp_size:
                raise ValueError(f"in_features {in_features} not divisible by tp={tp_size}")
            in_local = in_features // tp_size
        self.in_features, self.out_features = in_local, out_local
        self.weight = nn.Parameter(torch.empty(out_local, in_local, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_local, dtype=dtype, device=device)) if bias else None
        self.init_std = init_std
        if scale == "fan_in":
            scale = 1.0 / math.sqrt(in_features)
        elif scale == "fan_out":
            scale = 1.0 / math.sqrt(out_total)
        self.scale = scale
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight.device.type == "meta":
            return
        if self.init_std is None:
            nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        else:
            nn.init.normal_(self.weight, mean=0.0, std=self.init_std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def local_out_splits(self) -> tuple[int, ...]:
        """Widths of the merged outputs on this rank (e.g. q / k / v of a fused projection)."""
        if not self.out_splits:
            return (self.out_features,)
        if self.parallel_style == "column" and self.tp_size > 1:
            return tuple(s // self.tp_size for s in self.out_splits)
        return self.out_splits

    def forward(self, x: torch.Tensor, w: torch.Tensor | None = None) -> torch.Tensor:
        """``w`` overrides the weight (tied embeddings pass the embedding table here)."""
        y = F.linear(x, self.weight if w is None else w, self.bias, name=self.remat_name)
        if self.scale is not None:
            y = y * self.scale
        return y

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, "
                f"style={self.parallel_style}, tp={self.tp_size}")


class ColumnParallelLinear(ParallelLinear):
    parallel_style = "column"

    def forward(self, x: torch.Tensor, w: torch.Tensor | None = None) -> torch.Tensor:
        if self.tp_size > 1:
            from ..parallel import tp as tpar

            sp = self.sp_state
            if sp is not None and sp.active:
                # sequence-parallel block: ``x`` holds this rank's rows; the all-gather happens inside the GEMM
                y = tpar.column_parallel_sp(sp, x, self.weight if w is None else w, self.bias)
                return y if self.scale is None else y * self.scale
            x = tpar.copy_to_tp(x, self.tp_group)
        return super().forward(x, w)


class RowParallelLinear(ParallelLinear):
    parallel_style = "row"
    # When set (by a decoder layer whose next operation is the fused residual-add + RMSNorm), small inference
    # products return a ``parallel.tp.PendingReduce`` so that the all-reduce is fused into that norm.
    defer_reduce = False

    def forward(self, x: torch.Tensor, w: torch.Tensor | None = None):
        if self.tp_size > 1:
            from ..parallel import tp as tpar

            sp = self.sp_state
            if sp is not None and sp.active:
                # sequence-parallel block: the reduce-scatter of the output rows happens inside the GEMM
                y = tpar.row_parallel_sp(sp, x, self.weight if w is None else w, self.bias)
                return y if self.scale is None else y * self.scale
            return tpar.row_parallel_linear(x, self.weight if w is None else w, self.bias, self.tp_group,
                                            scale=self.scale, defer=self.defer_reduce)
        return super().forward(x, w)


class eLoRA(nn.Module):
    """Low-rank adapter around a linear layer: ``y = base(x) + (alpha / r) * B(A(dropout(x)))``.

    Mirrors the wrapping behaviour of easydel/layers/linears/_lora.py:38-102; ``merge`` folds the
    adapter into the base weight, ``unwrap`` returns the untouched base.
    """

    def __init__(self, base: ParallelLinear, rank: int, alpha: float | None = None, dropout: float = 0.0,
                 dtype: torch.dtype | None = None):
        super().__init__()
        self.base = base
        self.rank = rank
        self.alpha = float(alpha if alpha is not None else rank)
        dt = dtype or base.weight.dtype
        dev = base.weight.device
        self.lora_a = nn.Parameter(torch.empty(rank, base.in_features, dtype=dt, device=dev))
        self.lora_b = nn.Parameter(torch.zeros(base.out_features, rank, dtype=dt, device=dev))
        nn.init.kaiming_uniform_(self.lora_a, a=math.sqrt(5))
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        for p in base.parameters():
            p.requires_grad_(False)

    @property
    def scaling(self) -> float:
        return self.alpha / self.rank

    @property
    def weight(self):
        return self.base.weight

    def forward(self, x: torch.Tensor, w: torch.Tensor | None = None) -> torch.Tensor:
        y = self.base(x, w)
        z = torch.nn.functional.linear(torch.nn.functional.linear(self.dropout(x), self.lora_a), self.lora_b)
        return y + z * self.scaling

    @torch.no_grad()
    def merge(self) -> ParallelLinear:
        delta = (self.lora_b.float() @ self.lora_a.float()) * self.scaling
        self.base.weight.add_(delta.to(self.base.weight.dtype))
        for p in self.base.parameters():
            p.requires_grad_(True)
        return self.base

    def unwrap(self) -> ParallelLinear:
        for p in self.base.parameters():
            p.requires_grad_(True)
        return self.base
