"""Sharded optimizer state over the data-parallel ranks (the ``dp`` x ``fsdp`` axes of the mesh).

Every rank keeps the full bf16 working weights and the full fp32 gradient accumulation buffer;
fp32 master weights and optimizer moments exist only for the slice a rank owns (1/N of the flat
storage). The optimizer step is:

1. barrier: every rank has finished its backward passes;
2. reduce-scatter: each rank sums its slice of all ranks' gradient buffers;
3. global gradient norm (one scalar all-reduce) and the clip / non-finite decision;
4. the optimizer update on the slice, and all-gather of the refreshed working weights.

On B200s steps 2 and 4 are this framework's own kernels reading / writing peer memory over NVLink
(``csrc/dist_optim.cu``; buffers live in ``torch.distributed._symmetric_memory``). On CPU ranks
(gloo, used by the multi-process tests) and for non-AdamW optimizers the same algorithm runs with
``reduce_scatter`` / ``all_gather`` collectives.

Because 180 GB of HBM holds the full bf16 weights of the benchmarked models many times over, the
gathered weights persist across the whole step instead of being re-gathered per layer; this is the
FSDP axis of the reference (sharded parameters + optimizer state, easydel/infra/base_config.py:793)
with the all-gather hoisted to once per optimizer step.
"""

from __future__ import annotations

import ctypes as C
import typing as tp

import torch
import torch.distributed as dist

from ..ops import _lib
from .flat import FlatParams

_lib.register("edl_dist_reduce_sumsq", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i64, _lib.i64, _lib.vp, _lib.vp])
_lib.register("edl_dist_adamw_bcast", _lib.i32, [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                                 _lib.i64, _lib.i64] + [_lib.f32] * 7 + [_lib.vp, _lib.f32, _lib.vp,
                                                                                         _lib.i32, _lib.vp])


class DistributedFlat:
    def __init__(self, model, mesh, no_decay_patterns: tp.Sequence[str] = (), use_peer_kernels: bool | None = None,
                 param_filter=None):
        self.mesh = mesh
        axes = ("dp", "fsdp")
        self.group = mesh.get_group(axes)
        self.world = mesh.axis_size(axes)
        self.rank = mesh.axis_index(axes)
        dev = next(model.parameters()).device
        self.peer = bool(dev.type == "cuda" and _lib.available()) if use_peer_kernels is None else use_peer_kernels
        self._handles = []
        alloc = None
        if self.peer:
            import torch.distributed._symmetric_memory as symm

            def alloc(n, dt):
                t = symm.empty(n, dtype=dt, device=dev)
                t.zero_()
                return t

        self.flat = FlatParams(model, world_size=self.world, rank=self.rank, no_decay_patterns=no_decay_patterns,
                               alloc=alloc, param_filter=param_filter)
        self.last_clip = (None, None, 1.0)   # (clip coefficient, non-finite flag, gradient scale) of the last step
        flat = self.flat
        # identical starting weights everywhere: rank 0 of the group is the source
        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast(flat.work, src=src, group=self.group)
        flat.sync_master_from_work()
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.peer:
            import torch.distributed._symmetric_memory as symm

            self.h_work = symm.rendezvous(flat.work, self.group)
            self.h_grad = symm.rendezvous(flat.grad, self.group)
            # buffer_ptrs are the bases of the symmetric blocks; a tensor sits at `offset` inside its block
            wo, go = int(getattr(self.h_work, "offset", 0)), int(getattr(self.h_grad, "offset", 0))
            self._work_ptrs = (C.c_ulonglong * self.world)(*[int(p) + wo for p in self.h_work.buffer_ptrs])
            self._grad_ptrs = (C.c_ulonglong * self.world)(*[int(p) + go for p in self.h_grad.buffer_ptrs])
            if self._work_ptrs[self.rank] != flat.work.data_ptr() or self._grad_ptrs[self.rank] != flat.grad.data_ptr():
                raise RuntimeError("symmetric-memory handle does not address this rank's own buffers")

    # ------------------------------------------------------------------
    def _barrier(self, channel: int = 0) -> None:
        if self.peer:
            self.h_grad.barrier(channel=channel)
        else:
            dist.barrier(group=self.group)

    @torch.no_grad()
    def step(self, tx, *, step: int, lr: float, grad_scale: float = 1.0, zero_grad: bool = True,
             extra_sumsq: torch.Tensor | None = None) -> torch.Tensor:
        """One sharded optimizer step. Returns the global gradient norm (device tensor). ``extra_sumsq``: sum of
        squared gradients of parameters kept elsewhere (already summed over every group), to be part of the norm;
        the clip factor and the non-finite flag of the step are left in ``last_clip`` for that other runtime."""
        flat = self.flat
        n_shard = flat.shard_hi - flat.shard_lo
        # the mean over ranks is part of the gradient scale
        gscale = grad_scale / self.world
        fused = self.peer and tx.name == "adamw"
        self._sumsq.zero_()
        if self.peer:
            self._barrier(0)
            _lib.call("edl_dist_reduce_sumsq", C.cast(self._grad_ptrs, C.c_void_p), self.world, self.rank,
                      flat.shard_lo, n_shard, self._sumsq.data_ptr(), _lib.stream_ptr())
            self._barrier(1)
            g = flat.grad_shard
        else:
            if dist.get_backend(self.group) == "gloo":
                # gloo has no reduce-scatter: all-reduce and keep the owned slice
                dist.all_reduce(flat.grad, group=self.group)
                g = flat.grad_shard
            else:
                g = torch.empty(n_shard, dtype=flat.grad.dtype, device=flat.grad.device)
                dist.reduce_scatter_tensor(g, flat.grad, op=dist.ReduceOp.SUM, group=self.group)
            self._sumsq += g.float().pow(2).sum()
        dist.all_reduce(self._sumsq, group=self.group)
        # tensor- / expert-parallel shards: add the other ranks' pieces so that every rank clips with one norm
        self._sumsq.copy_(flat.global_sumsq(self._sumsq, g, flat.shard_lo, self.mesh, dp_group=self.group))
        if extra_sumsq is not None:
            self._sumsq += extra_sumsq.reshape(-1)[:1].to(self._sumsq.dtype)
        if g.is_cuda and _lib.available():
            from ..ops import kernels as K

            norm, coef, skip = K.clip_coef(self._sumsq, gscale, tx.clip_grad or 0.0)
        else:
            norm = self._sumsq.sqrt() * gscale
            skip = (~torch.isfinite(norm)).to(torch.int32).reshape(1)
            coef = torch.clamp((tx.clip_grad or float("inf")) / (norm + 1e-6), max=1.0).reshape(1) \
                if tx.clip_grad else None
        self.last_clip = (coef, skip, gscale)
        for lo, hi, decay in flat.decay_ranges():
            state = {k: v[lo:hi] for k, v in flat.opt_state.items()}
            if fused:
                wd = tx.weight_decay if decay else 0.0
                bc1, bc2 = 1.0 - tx.b1 ** step, 1.0 - tx.b2 ** step
                _lib.call("edl_dist_adamw_bcast", flat.master[lo:hi].data_ptr(), state["mu"].data_ptr(),
                          state["nu"].data_ptr(), g[lo:hi].data_ptr(), C.cast(self._work_ptrs, C.c_void_p),
                          self.world, self.rank, flat.shard_lo + lo, hi - lo, float(lr), float(tx.b1), float(tx.b2),
                          float(tx.eps), float(wd), float(bc1), float(bc2), _lib.ptr(coef), float(gscale),
                          _lib.ptr(skip), 0, _lib.stream_ptr())
            else:
                tx.update(flat.master[lo:hi], flat.work_shard[lo:hi], g[lo:hi], state, step=step, lr=lr,
                          gscale=gscale, gscale_tensor=coef, skip_tensor=skip, decay=decay, zero_grad=False)
        if not fused:
            # all-gather of the refreshed working weights
            if dist.get_backend(self.group) == "gloo":
                parts = [flat.work[r * n_shard:(r + 1) * n_shard] for r in range(self.world)]
                dist.all_gather(parts, flat.work_shard.clone(), group=self.group)
            else:
                dist.all_gather_into_tensor(flat.work, flat.work_shard.clone(), group=self.group)
        if zero_grad:
            flat.grad.zero_()
        if self.peer:
            self._barrier(2)
        return norm
