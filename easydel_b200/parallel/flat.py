"""Flat parameter / gradient / optimizer-state storage.

All trainable parameters of a model are re-pointed to views of ONE contiguous working buffer
(bf16 on the GPU), and get an fp32 ``main_grad`` view into ONE contiguous gradient buffer that
the backward GEMMs accumulate into. Master weights and optimizer moments are fp32 buffers of the
same layout, restricted to the range a rank owns.

Why flat: the optimizer step is a single kernel launch over the owned range, the gradient norm is
one reduction, and under data/FSDP parallelism the owned range of rank r is simply
``[r * n/N, (r+1) * n/N)`` of every buffer, so the fused reduce-scatter + AdamW + all-gather
kernel (``csrc/dist_optim.cu``) needs nothing but base pointers and a range.

This is how the framework carries out what the reference expresses as sharded ``opt_state`` plus
XLA-inserted reduce-scatter / all-gather (easydel/infra/base_state.py:353-419, 575-666).
"""

from __future__ import annotations

import re
import typing as tp

import torch
from torch import nn

ALIGN = 128  # elements; keeps every parameter view 256-byte aligned in bf16


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    def __init__(self, model: nn.Module, *, world_size: int = 1, rank: int = 0, grad_dtype=torch.float32,
                 no_decay_patterns: tp.Sequence[str] = (), alloc: tp.Callable | None = None,
                 param_filter: tp.Callable[[str, nn.Parameter], bool] | None = None):
        """``param_filter(name, param)`` selects the parameters this storage owns (default: all trainable ones);
        the rest belong to another runtime, e.g. the layer-sharded one of ``parallel.fsdp``."""
        self.model = model
        self.world_size, self.rank = world_size, rank
        params = [(n, p) for n, p in model.named_parameters()
                  if p.requires_grad and (param_filter is None or param_filter(n, p))]
        # parameters shared under several names (tied embeddings) appear once
        seen: dict[int, str] = {}
        uniq = []
        for n, p in params:
            if id(p) in seen:
                continue
            seen[id(p)] = n
            uniq.append((n, p))
        if not uniq:
            raise ValueError("model has no trainable parameters")
        dev = uniq[0][1].device
        wdtype = uniq[0][1].dtype
        if any(p.dtype != wdtype for _, p in uniq):
            raise ValueError("all trainable parameters must share one dtype to be flattened")
        self.device, self.work_dtype = dev, wdtype
        nd = [re.compile(x) for x in no_decay_patterns]
        self.entries: list[tuple[str, int, int, tuple[int, ...], bool]] = []
        off = 0
        for n, p in uniq:
            decay = not any(r.search(n) for r in nd)
            self.entries.append((n, off, p.numel(), tuple(p.shape), decay))
            off = _round_up(off + p.numel(), ALIGN)
        self.numel = _round_up(off, ALIGN * max(world_size, 1))
        alloc = alloc or (lambda n, dt: torch.zeros(n, dtype=dt, device=dev))
        self.work = alloc(self.numel, wdtype)
        self.grad = alloc(self.numel, grad_dtype)
        name_to_param = dict(uniq)
        with torch.no_grad():
            for n, o, sz, shape, _ in self.entries:
                p = name_to_param[n]
                view = self.work[o:o + sz].view(shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grad[o:o + sz].view(shape)
                p.grad = None
        self.params = name_to_param
        # owned range of this rank (everything when world_size == 1)
        per = self.numel // max(world_size, 1)
        self.shard_lo, self.shard_hi = rank * per, (rank + 1) * per
        self.master = self.work[self.shard_lo:self.shard_hi].float() if wdtype != torch.float32 \
            else self.work[self.shard_lo:self.shard_hi]
        self.master_is_work = wdtype == torch.float32 and world_size == 1
        self.opt_state: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ views
    @property
    def work_shard(self) -> torch.Tensor:
        return self.work[self.shard_lo:self.shard_hi]

    @property
    def grad_shard(self) -> torch.Tensor:
        return self.grad[self.shard_lo:self.shard_hi]

    def decay_ranges(self) -> list[tuple[int, int, bool]]:
        """Maximal runs of the owned range with a uniform weight-decay flag: ``(lo, hi, decay)`` in shard
        coordinates."""
        runs: list[tuple[int, int, bool]] = []
        for i, (n, o, sz, _, decay) in enumerate(self.entries):
            end = self.entries[i + 1][1] if i + 1 < len(self.entries) else self.numel
            lo, hi = max(o, self.shard_lo), min(end, self.shard_hi)
            if lo >= hi:
                continue
            lo -= self.shard_lo
            hi -= self.shard_lo
            if runs and runs[-1][2] == decay and runs[-1][1] == lo:
                runs[-1] = (runs[-1][0], hi, decay)
            else:
                runs.append((lo, hi, decay))
        return runs

    def replicated_ranges(self) -> list[tuple[int, int]]:
        """Maximal runs of the flat buffer that hold parameters replicated across the expert-parallel group
        (everything except the per-rank expert weights, which are tagged ``_ep_local`` by the MoE block)."""
        runs: list[tuple[int, int]] = []
        for i, (n, o, sz, _, _) in enumerate(self.entries):
            if getattr(self.params[n], "_ep_local", False):
                continue
            end = self.entries[i + 1][1] if i + 1 < len(self.entries) else self.numel
            if runs and runs[-1][1] == o:
                runs[-1] = (runs[-1][0], end)
            else:
                runs.append((o, end))
        return runs

    def model_parallel_ranges(self) -> dict[str, list[tuple[int, int]]]:
        """Flat ranges (element offsets, without padding) of the parameters that differ across the model-parallel
        groups: ``"tp"`` = column / row shards of tensor-parallel linears, ``"ep"`` = per-rank expert weights.
        Everything else is replicated over those groups."""
        if getattr(self, "_mp_ranges", None) is not None:
            return self._mp_ranges
        owner = {}
        for mod_name, mod in self.model.named_modules():
            style = getattr(mod, "parallel_style", None)
            if getattr(mod, "tp_size", 1) > 1 and style in ("column", "row"):
                for leaf, p in mod.named_parameters(recurse=False):
                    if not (style == "row" and leaf == "bias"):
                        owner[id(p)] = "tp"
        out: dict[str, list[tuple[int, int]]] = {"tp": [], "ep": []}
        for n, o, sz, _, _ in self.entries:
            p = self.params[n]
            if getattr(p, "_ep_local", False):
                kind = "tp" if getattr(p, "_ep_over_tp", False) else "ep"    # expert tensor mode: spread over tp
            else:
                kind = owner.get(id(p))
            if kind is None:
                continue
            runs = out[kind]
            if runs and runs[-1][1] == o:
                runs[-1] = (runs[-1][0], o + sz)
            else:
                runs.append((o, o + sz))
        self._mp_ranges = out
        return out

    def global_sumsq(self, sumsq: torch.Tensor, grad: torch.Tensor, grad_lo: int, mesh, dp_group=None) -> torch.Tensor:
        """Sum of squared gradients over the whole model from the sum over this rank's flat buffer.

        ``sumsq`` (1-element tensor) already covers the local flat buffer (summed over the data-parallel group when
        the buffer is sharded over it); ``grad`` is the slice of the gradient buffer this rank reduced, starting at
        flat offset ``grad_lo``. Parameters sharded over the tensor- or expert-parallel group contribute every
        rank's piece, replicated parameters count once, so every rank of those groups ends up with the same norm
        (and the same clip coefficient and skip decision)."""
        import torch.distributed as dist

        ranges = self.model_parallel_ranges()
        if mesh is None or not (ranges["tp"] or ranges["ep"]):
            return sumsq
        parts = torch.zeros(2, dtype=torch.float32, device=sumsq.device)
        hi_lim = grad_lo + grad.numel()
        for i, kind in enumerate(("tp", "ep")):
            for lo, hi in ranges[kind]:
                a, b = max(lo, grad_lo), min(hi, hi_lim)
                if a < b:
                    parts[i] += grad[a - grad_lo:b - grad_lo].float().pow(2).sum()
        if dp_group is not None and self.world_size > 1:
            dist.all_reduce(parts, group=dp_group)
        local = parts.clone()
        if ranges["tp"]:
            dist.all_reduce(parts[0:1], group=mesh.get_group("tp"))
        if ranges["ep"]:
            dist.all_reduce(parts[1:2], group=mesh.get_group("ep"))
        return sumsq + (parts - local).sum()

    def sync_partial_grads_over_tp(self, group) -> None:
        """After a sequence-parallel backward every rank of the tensor-parallel group has seen only its own token
        rows, so the gradient of each parameter that is not a tensor-parallel shard (norm scales, embeddings, the
        LM head, row-parallel biases) is a partial sum: add the group's pieces."""
        import torch.distributed as dist

        tp_runs = self.model_parallel_ranges()["tp"]
        pos, runs = 0, []
        for lo, hi in tp_runs:
            if lo > pos:
                runs.append((pos, lo))
            pos = max(pos, hi)
        if pos < self.numel:
            runs.append((pos, self.numel))
        for lo, hi in runs:
            dist.all_reduce(self.grad[lo:hi], group=group)

    def sync_replicated_grads(self, group) -> None:
        """Sums the gradients of the replicated parameters over the expert-parallel group (each rank saw different
        tokens); expert weights already received every token's contribution through the token exchange."""
        import torch.distributed as dist

        for lo, hi in self.replicated_ranges():
            dist.all_reduce(self.grad[lo:hi], group=group)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def named_views(self, flat: torch.Tensor, full: bool = True):
        """Yields ``(name, view)`` of a flat buffer laid out like the working buffer."""
        for n, o, sz, shape, _ in self.entries:
            yield n, flat[o:o + sz].view(shape)

    def sync_master_from_work(self) -> None:
        """Re-reads the master copy from the working weights (after loading a checkpoint into the model)."""
        if not self.master_is_work:
            self.master.copy_(self.work[self.shard_lo:self.shard_hi])

    # torch .grad -> main_grad (for autograd nodes that returned a regular gradient)
    def fold_param_grads(self) -> None:
        for n, p in self.params.items():
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
