"""Tensor parallelism: the collectives around column- and row-parallel linears.

Column-parallel layers split output features, row-parallel layers split input features; the pair
needs one all-reduce in the forward pass (after the row-parallel GEMM) and one in the backward
pass (of the gradient entering the column-parallel GEMM). The reference gets both from XLA's SPMD
partitioner (easydel/layers/linears/_linear.py:348-378). Here:

* small messages (decode steps) use the one-shot peer-memory all-reduce kernel in
  ``csrc/collectives.cu``: the row-parallel GEMM writes its partial result straight into a
  symmetric buffer and the kernel sums all ranks' partials over NVLink;
* large messages (prefill, training) use NCCL all-reduce.
"""

from __future__ import annotations

import ctypes as C
import typing as tp

import torch
import torch.distributed as dist

from ..ops import _lib

_lib.register("edl_allreduce_oneshot", _lib.i32, [_lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.vp,
                                                  _lib.i64, _lib.i32, _lib.vp, _lib.vp])

_lib.register("edl_allreduce_add_rmsnorm", _lib.i32, [_lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.vp,
                                                      _lib.f32, _lib.f32, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                                      _lib.i32, _lib.vp, _lib.vp])

ONE_SHOT_MAX_BYTES = 1 << 20
_FLAG_BYTES = 256


class _PeerAllReduce:
    """Symmetric buffers + flags of one process group."""

    def __init__(self, group, device, max_bytes: int = ONE_SHOT_MAX_BYTES):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_bytes = max_bytes
        total = 2 * max_bytes + _FLAG_BYTES
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        off = int(getattr(self.handle, "offset", 0))
        base = [int(p) + off for p in self.handle.buffer_ptrs]
        if base[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric-memory handle does not address this rank's own buffer")
        self.slot_ptrs = [(C.c_ulonglong * self.world)(*[b + s * max_bytes for b in base]) for s in range(2)]
        self.flag_ptrs = (C.c_ulonglong * self.world)(*[b + 2 * max_bytes for b in base])
        self.epoch = 0          # host-side call count: selects the slot; the kernel keeps its own count in `sync`
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def slot_tensor(self, shape, dtype) -> torch.Tensor:
        """A tensor view of the slot the *next* call will reduce (GEMMs write their partials here)."""
        s = (self.epoch + 1) & 1
        n = 1
        for d in shape:
            n *= d
        off = s * self.max_bytes
        return self.buf[off:off + n * 2].view(dtype).view(shape)

    def reduce(self, partial_in_slot: torch.Tensor, residual: torch.Tensor | None = None,
               wait_ms: int = 2000) -> torch.Tensor:
        self.epoch += 1
        s = self.epoch & 1
        out = torch.empty_like(partial_in_slot, memory_format=torch.contiguous_format)
        _lib.call("edl_allreduce_oneshot", C.cast(self.slot_ptrs[s], C.c_void_p), C.cast(self.flag_ptrs, C.c_void_p),
                  self.world, self.rank, self.sync.data_ptr(), out.data_ptr(), _lib.ptr(residual), partial_in_slot.numel(),
                  wait_ms, _lib.status_word(out.device).data_ptr(), _lib.stream_ptr())
        return out


class PendingReduce:
    """A row-parallel product whose partial sums still sit in the symmetric slot.

    The consumer either calls :meth:`add_rms_norm` (one kernel: sum over ranks + residual add + RMSNorm) or
    :meth:`resolve` (the plain one-shot all-reduce). Exactly one of them must be called, and before the next
    row-parallel product of the same group is formed.
    """

    def __init__(self, ctx: "_PeerAllReduce", slot: torch.Tensor, shape, bias=None, scale=None):
        self.ctx, self.slot, self.shape, self.bias, self.scale = ctx, slot, tuple(shape), bias, scale
        self.dtype, self.device = slot.dtype, slot.device

    def resolve(self) -> torch.Tensor:
        y = self.ctx.reduce(self.slot).view(self.shape)
        if self.bias is not None:
            y = y + self.bias
        return y if self.scale is None else y * self.scale

    def add_rms_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, w_offset: float = 0.0):
        """Returns ``(rmsnorm(residual + sum) * (weight + w_offset), residual + sum)``."""
        if self.bias is not None or self.scale is not None or residual.dtype != torch.bfloat16 \
                or weight.dtype != torch.bfloat16 or self.shape[-1] > 16384:
            y = self.resolve()
            from ..ops import functional as F

            return F.add_rms_norm(y, residual, weight, eps, w_offset)
        c = self.ctx
        c.epoch += 1
        s = c.epoch & 1
        res = residual.contiguous()
        x_out = torch.empty_like(res)
        h_out = torch.empty_like(res)
        width = self.shape[-1]
        rows = res.numel() // width
        _lib.call("edl_allreduce_add_rmsnorm", C.cast(c.slot_ptrs[s], C.c_void_p), C.cast(c.flag_ptrs, C.c_void_p),
                  c.world, c.rank, c.sync.data_ptr(), res.data_ptr(), weight.data_ptr(), float(eps), float(w_offset),
                  x_out.data_ptr(), h_out.data_ptr(), rows, width, 2000, _lib.status_word(res.device).data_ptr(),
                  _lib.stream_ptr())
        return h_out.view(residual.shape), x_out.view(residual.shape)


def resolve(x):
    """Materialises a :class:`PendingReduce`; passes tensors (and ``None``) through."""
    return x.resolve() if isinstance(x, PendingReduce) else x


_CTX: dict[int, _PeerAllReduce] = {}


def _peer_ctx(group, device) -> _PeerAllReduce | None:
    key = id(group)
    if key not in _CTX:
        if device.type != "cuda" or not _lib.available():
            return None
        _CTX[key] = _PeerAllReduce(group, device)
    return _CTX[key]


def all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    """Sum over the tensor-parallel group (out of place)."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    nbytes = x.numel() * x.element_size()
    if x.is_cuda and x.dtype == torch.bfloat16 and nbytes <= ONE_SHOT_MAX_BYTES and x.numel() % 8 == 0 \
            and not torch.is_grad_enabled():
        ctx = _peer_ctx(group, x.device)
        if ctx is not None:
            slot = ctx.slot_tensor(x.shape, x.dtype)
            slot.copy_(x)
            return ctx.reduce(slot)
    y = x.contiguous().clone()
    dist.all_reduce(y, group=group)
    return y


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        y = dy.contiguous().clone()
        dist.all_reduce(y, group=ctx.group)
        return y, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce(x, group)

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def copy_to_tp(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or not x.requires_grad:
        return x
    return _CopyToTP.apply(x, group)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, bias, group, scale=None, defer: bool = False):
    """``all_reduce(x_local @ w_local.T) + bias``. In inference the GEMM writes into the symmetric slot."""
    from ..ops import functional as F
    from ..ops import kernels as K

    nbytes = x.numel() // x.shape[-1] * w.shape[0] * 2
    if (not torch.is_grad_enabled()) and x.is_cuda and x.dtype == torch.bfloat16 and nbytes <= ONE_SHOT_MAX_BYTES:
        ctx = _peer_ctx(group, x.device)
        if ctx is not None:
            x2 = x.reshape(-1, x.shape[-1])
            if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8):
                x2 = x2.contiguous()
            slot = ctx.slot_tensor((x2.shape[0], w.shape[0]), x.dtype)
            K.gemm(x2, w, out=slot)
            if defer:
                return PendingReduce(ctx, slot, (*x.shape[:-1], w.shape[0]), bias, scale)
            y = ctx.reduce(slot).view(*x.shape[:-1], w.shape[0])
            if bias is not None:
                y = y + bias
            return y if scale is None else y * scale
    y = F.linear(x, w, None)
    y = _ReduceFromTP.apply(y, group) if torch.is_grad_enabled() else all_reduce(y, group)
    if bias is not None:
        y = y + bias
    return y if scale is None else y * scale
