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

ONE_SHOT_MAX_BYTES = 1 << 20     # up to here every rank reads every rank's whole partial (one flag round)
# up to here rank r reduces its own rows and stores them to every rank (two rounds); EDL_TP_TWO_SHOT=0 leaves
# messages above the one-shot limit to NCCL
TWO_SHOT_MAX_BYTES = (8 << 20) if __import__("os").environ.get("EDL_TP_TWO_SHOT", "1") != "0" else ONE_SHOT_MAX_BYTES
_FLAG_BYTES = 256
_lib.register("edl_allreduce_twoshot", _lib.i32, [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp,
                                                  _lib.vp, _lib.vp, _lib.f32, _lib.f32, _lib.i32, _lib.i32, _lib.i32,
                                                  _lib.vp, _lib.vp])


_lib.register("edl_allreduce_add_rmsnorm_mc", _lib.i32, [_lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.vp,
                                                         _lib.f32, _lib.f32, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                                         _lib.i32, _lib.vp, _lib.vp, _lib.u64])
_lib.register("edl_allreduce_twoshot_mc", _lib.i32, [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp,
                                                     _lib.vp, _lib.vp, _lib.f32, _lib.f32, _lib.i32, _lib.i32,
                                                     _lib.i32, _lib.vp, _lib.vp, _lib.u64, _lib.u64, _lib.u64])
# The two-shot kernel can sum and broadcast through the NVLink switch (multimem) where the symmetric buffer has a
# multicast mapping. EDL_TP_MULTIMEM: "auto" (default) uses it from four ranks up (with two ranks the per-peer form
# measured faster: 6.86 vs 7.09 ms for a 16-layer decode step of 256 rows), "1" always, "0" never.
_MULTIMEM_MODE = __import__("os").environ.get("EDL_TP_MULTIMEM", "auto")


class _PeerAllReduce:
    """Symmetric buffers + flags of one process group."""

    def __init__(self, group, device, max_bytes: int = TWO_SHOT_MAX_BYTES):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_bytes = max_bytes
        # [partial slot 0 | partial slot 1 | flags | gathered residual rows | gathered normalised rows]
        total = 4 * max_bytes + _FLAG_BYTES
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        off = int(getattr(self.handle, "offset", 0))
        base = [int(p) + off for p in self.handle.buffer_ptrs]
        if base[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric-memory handle does not address this rank's own buffer")
        self.slot_ptrs = [(C.c_ulonglong * self.world)(*[b + s * max_bytes for b in base]) for s in range(2)]
        self.flag_ptrs = (C.c_ulonglong * self.world)(*[b + 2 * max_bytes for b in base])
        self.out_off = [2 * max_bytes + _FLAG_BYTES, 3 * max_bytes + _FLAG_BYTES]
        self.out_ptrs = [(C.c_ulonglong * self.world)(*[b + o for b in base]) for o in self.out_off]
        use_mc = _MULTIMEM_MODE == "1" or (_MULTIMEM_MODE == "auto" and self.world >= 4)
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0) if use_mc else 0
        self.mc_base = mc + off if mc else 0   # multicast address of this buffer: in-switch sums and broadcasts
        self.epoch = 0          # host-side call count: selects the slot; the kernel keeps its own count in `sync`
        self.sync = torch.zeros(4, dtype=torch.int32, device=device)
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


    def out_tensor(self, which: int, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        off = self.out_off[which]
        return self.buf[off:off + n * 2].view(dtype).view(shape)

    def two_shot_ok(self, rows: int, width: int) -> bool:
        return rows % self.world == 0 and width % 8 == 0 and width <= 16384 and rows * width * 2 <= self.max_bytes

    def reduce_two_shot(self, rows: int, width: int, residual=None, weight=None, eps: float = 0.0,
                        w_offset: float = 0.0, sum_into: int = 0, wait_ms: int = 2000):
        """Two-shot all-reduce of the partial in the next slot. Returns views of this rank's gathered outputs:
        ``(residual + sum, rmsnorm(...) * (weight + w_offset))`` (the second is None without ``weight``). The views
        live in the symmetric buffer and are overwritten by a later call; ``sum_into`` selects which of the two
        output regions receives the summed rows."""
        self.epoch += 1
        s = self.epoch & 1
        x_ptrs = self.out_ptrs[sum_into]
        h_ptrs = self.out_ptrs[1 - sum_into] if weight is not None else None
        mcb = self.mc_base
        _lib.call("edl_allreduce_twoshot_mc", C.cast(self.slot_ptrs[s], C.c_void_p),
                  C.cast(self.flag_ptrs, C.c_void_p), C.cast(x_ptrs, C.c_void_p),
                  C.cast(h_ptrs, C.c_void_p) if h_ptrs is not None else None, self.world, self.rank,
                  self.sync.data_ptr(), _lib.ptr(residual), _lib.ptr(weight), float(eps), float(w_offset), rows, width,
                  wait_ms, _lib.status_word(self.buf.device).data_ptr(), _lib.stream_ptr(),
                  mcb + s * self.max_bytes if mcb else 0, mcb + self.out_off[sum_into] if mcb else 0,
                  mcb + self.out_off[1 - sum_into] if mcb and weight is not None else 0)
        x = self.out_tensor(sum_into, (rows, width), torch.bfloat16)
        h = self.out_tensor(1 - sum_into, (rows, width), torch.bfloat16) if weight is not None else None
        return x, h


class PendingReduce:
    """A row-parallel product whose partial sums still sit in the symmetric slot.

    The consumer either calls :meth:`add_rms_norm` (one kernel: sum over ranks + residual add + RMSNorm) or
    :meth:`resolve` (the plain one-shot all-reduce). Exactly one of them must be called, and before the next
    row-parallel product of the same group is formed.
    """

    def __init__(self, ctx: "_PeerAllReduce", slot: torch.Tensor, shape, bias=None, scale=None):
        self.ctx, self.slot, self.shape, self.bias, self.scale = ctx, slot, tuple(shape), bias, scale
        self.dtype, self.device = slot.dtype, slot.device

    def _big(self) -> bool:
        width = self.shape[-1]
        rows = self.slot.numel() // width
        return self.slot.numel() * 2 > ONE_SHOT_MAX_BYTES and self.ctx.two_shot_ok(rows, width)

    def resolve(self) -> torch.Tensor:
        if self._big():
            width = self.shape[-1]
            # the sum goes to the region of the normalised rows (whose last content has been consumed) and is copied
            # out: the residual rows in the other region may still be needed by the caller
            y, _ = self.ctx.reduce_two_shot(self.slot.numel() // width, width, sum_into=1)
            y = y.clone().view(self.shape)
        else:
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
        if self._big():
            # rank r reduces, normalises and stores its own rows to everybody; the results are views of the
            # symmetric buffer (the next all-reduce of this group overwrites them, after its own flag round)
            width = self.shape[-1]
            res = residual.reshape(-1, width)
            if not res.is_contiguous():
                res = res.contiguous()
            x_new, h_new = c.reduce_two_shot(res.shape[0], width, res, weight, eps, w_offset)
            return h_new.view(residual.shape), x_new.view(residual.shape)
        c.epoch += 1
        s = c.epoch & 1
        res = residual.contiguous()
        x_out = torch.empty_like(res)
        h_out = torch.empty_like(res)
        width = self.shape[-1]
        rows = res.numel() // width
        _lib.call("edl_allreduce_add_rmsnorm_mc", C.cast(c.slot_ptrs[s], C.c_void_p),
                  C.cast(c.flag_ptrs, C.c_void_p), c.world, c.rank, c.sync.data_ptr(), res.data_ptr(),
                  weight.data_ptr(), float(eps), float(w_offset), x_out.data_ptr(), h_out.data_ptr(), rows, width, 2000,
                  _lib.status_word(res.device).data_ptr(), _lib.stream_ptr(),
                  c.mc_base + s * c.max_bytes if c.mc_base else 0)
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


def release_peer_buffers() -> None:
    """Drops the symmetric buffers of the one-shot all-reduce and of the fused GEMM plans. Call with no kernel
    in flight (after a synchronize) and before the process groups are destroyed."""
    _CTX.clear()
    _PLANS.clear()


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
    if (not torch.is_grad_enabled()) and x.is_cuda and x.dtype == torch.bfloat16 and nbytes <= TWO_SHOT_MAX_BYTES:
        ctx = _peer_ctx(group, x.device)
        rows_ = x.numel() // x.shape[-1]
        if ctx is not None and (nbytes <= ONE_SHOT_MAX_BYTES or ctx.two_shot_ok(rows_, w.shape[0])):
            x2 = x.reshape(-1, x.shape[-1])
            if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8):
                x2 = x2.contiguous()
            slot = ctx.slot_tensor((x2.shape[0], w.shape[0]), x.dtype)
            K.gemm(x2, w, out=slot)
            pend = PendingReduce(ctx, slot, (*x.shape[:-1], w.shape[0]), bias, scale)
            return pend if defer else pend.resolve()
    y = F.linear(x, w, None)
    y = _ReduceFromTP.apply(y, group) if torch.is_grad_enabled() else all_reduce(y, group)
    if bias is not None:
        y = y + bias
    return y if scale is None else y * scale


# ------------------------------------------------------------------------------------------------
# Sequence-parallel tensor parallelism: the residual stream between the linears is sharded by rows
# (tokens) over the group; a column-parallel linear all-gathers its input inside the GEMM, a
# row-parallel linear reduce-scatters its output inside the GEMM (csrc/gemm_collective.cu). The
# backward products are the mirrored pair. On CPU ranks (gloo) and for shapes the kernels do not
# take, the same algebra runs through torch.distributed collectives.
# ------------------------------------------------------------------------------------------------
class SequenceParallelState:
    """What the linears need to know while a model runs with sequence-sharded activations.

    Set by the model's forward before its layers run and left in place afterwards, because the
    activation-checkpoint recompute of a layer happens during backward."""

    def __init__(self):
        self.active = False
        self.group = None
        self.world = 1
        self.rank = 0
        self.batch = 1
        self.seq = 0

    @property
    def rows(self) -> int:
        return self.batch * self.seq

    @property
    def rows_local(self) -> int:
        return self.rows // self.world

    def begin(self, group, batch: int, seq: int) -> None:
        self.active, self.group = True, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.batch, self.seq = batch, seq

    def end(self) -> None:
        self.active = False


_PLANS: dict[tuple, tp.Any] = {}


def sequence_parallel_usable(group, batch: int, seq: int, hidden: int, device) -> bool:
    """Rows must split evenly; the fused kernels additionally want 128-row shards and a hidden size that is a
    multiple of 128 (other shapes take the collective + GEMM path, which has no such limits)."""
    if group is None:
        return False
    world = dist.get_world_size(group)
    return world > 1 and (batch * seq) % world == 0


def _fused_ok(sp, x: torch.Tensor, rows_local: int, k: int, n: int) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and _lib.available() and rows_local % 128 == 0
            and k % 128 == 0 and n % 8 == 0 and sp.world <= 8)


def _plan(sp, kind: str, rows_local: int, width: int, device):
    from . import fused

    key = (kind, id(sp.group), rows_local, width, device.index)
    p = _PLANS.get(key)
    if p is None:
        if kind == "ag":
            p = fused.AllGatherGemm(sp.group, rows_local, width, device)
        else:
            p = fused.GemmReduceScatter(sp.group, rows_local, width, device)
        _PLANS[key] = p
    return p


def _all_gather_rows(sp, x: torch.Tensor) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(sp.world)]
    dist.all_gather(parts, x.contiguous(), group=sp.group)
    return torch.cat(parts, 0)


def _reduce_scatter_rows(sp, y: torch.Tensor) -> torch.Tensor:
    """Sum over the group, keep this rank's row block."""
    rows = y.shape[0] // sp.world
    if y.is_cuda and dist.get_backend(sp.group) != "gloo":
        out = torch.empty(rows, y.shape[1], dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y.contiguous(), group=sp.group)
        return out
    y = y.contiguous().clone()
    dist.all_reduce(y, group=sp.group)
    return y[sp.rank * rows:(sp.rank + 1) * rows].clone()


def _ag_gemm(sp, x_shard: torch.Tensor, w: torch.Tensor, b_mn: bool, keep_gathered: bool = False):
    """``(all_gather_rows(x_shard) @ op(w), gathered x)``; ``op(w) = w.T`` for ``[N, K]`` weights, ``w`` itself
    when ``b_mn`` (weights stored ``[K, N]``)."""
    from ..ops import functional as F

    k = x_shard.shape[1]
    n = w.shape[1] if b_mn else w.shape[0]
    if _fused_ok(sp, x_shard, x_shard.shape[0], k, n) and w.stride(-1) == 1:
        c, g = _plan(sp, "ag", x_shard.shape[0], k, x_shard.device)(x_shard, w, b_mn=b_mn)
        # the gathered rows live in a buffer of the plan that its next call overwrites
        return c, (g.clone() if keep_gathered else g)
    g = _all_gather_rows(sp, x_shard)
    with torch.no_grad():
        return (g @ w if b_mn else F.linear(g, w, None)), g


def _gemm_rs(sp, x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """``reduce_scatter_rows(x @ op(w))``: every rank holds a slice of the reduction dimension."""
    from ..ops import functional as F

    n = w.shape[1] if b_mn else w.shape[0]
    rows_local = x.shape[0] // sp.world
    if _fused_ok(sp, x, rows_local, 128, n) and x.shape[1] % 8 == 0 and w.stride(-1) == 1 and x.stride(-1) == 1:
        return _plan(sp, "rs", rows_local, n, x.device)(x, w, b_mn=b_mn)
    with torch.no_grad():
        y = x @ w if b_mn else F.linear(x, w, None)
    return _reduce_scatter_rows(sp, y)


def _weight_grad(w: torch.Tensor, dy: torch.Tensor, x: torch.Tensor):
    """dW[N, K] = dy[T, N]^T x[T, K]: accumulated into ``w.main_grad`` when the flat gradient buffer exists."""
    from ..ops import kernels as K

    mg = getattr(w, "main_grad", None)
    if dy.is_cuda and _lib.available() and dy.dtype == torch.bfloat16:
        if mg is not None:
            K.gemm(dy, x, a_mn=True, b_mn=True, out=mg, accumulate=True)
            w.grad_added_to_main_grad = True
            return None
        return K.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)
    return (dy.float().t() @ x.float()).to(w.dtype)


class _ColumnSP(torch.autograd.Function):
    """y[T, N_local] = all_gather_rows(x[T/n, K]) @ w[N_local, K]^T  (+ bias)."""

    @staticmethod
    def forward(ctx, sp, x_shard, w, bias):
        ctx.sp = sp
        y, g = _ag_gemm(sp, x_shard, w, b_mn=False, keep_gathered=True)   # the gathered input is needed for dW
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(g, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        g, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _gemm_rs(ctx.sp, dy, w, b_mn=True) if ctx.needs_input_grad[1] else None   # dY[T, N_l] @ W[N_l, K]
        dw = _weight_grad(w, dy, g) if ctx.needs_input_grad[2] else None
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[3] else None
        return None, dx, dw, db


class _RowSP(torch.autograd.Function):
    """y[T/n, N] = reduce_scatter_rows(x[T, K_local] @ w[N, K_local]^T)."""

    @staticmethod
    def forward(ctx, sp, x, w):
        ctx.sp = sp
        ctx.save_for_backward(x, w)
        return _gemm_rs(sp, x.contiguous(), w, b_mn=False)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dx, g = _ag_gemm(ctx.sp, dy_shard.contiguous(), w, b_mn=True)   # gather(dY)[T, N] @ W[N, K_l]
        dw = _weight_grad(w, g, x.reshape(-1, x.shape[-1])) if ctx.needs_input_grad[2] else None
        return None, (dx if ctx.needs_input_grad[1] else None), dw


def column_parallel_sp(sp, x_shard: torch.Tensor, w: torch.Tensor, bias) -> torch.Tensor:
    """Column-parallel linear on a row-sharded input; returns ``[batch, seq, N_local]``."""
    x2 = x_shard.reshape(-1, x_shard.shape[-1])
    y = _ColumnSP.apply(sp, x2, w, bias)
    return y.view(sp.batch, sp.seq, y.shape[-1])


def row_parallel_sp(sp, x: torch.Tensor, w: torch.Tensor, bias) -> torch.Tensor:
    """Row-parallel linear whose output comes back row-sharded: ``[1, rows/n, N]``. The bias (replicated) is
    added once per row, after the reduction."""
    x2 = x.reshape(-1, x.shape[-1])
    y = _RowSP.apply(sp, x2, w)
    if bias is not None:
        y = y + bias
    return y.view(1, y.shape[0], y.shape[1])


class _GatherRows(torch.autograd.Function):
    """All-gather of row shards whose consumer is replicated on every rank (backward keeps this rank's rows)."""

    @staticmethod
    def forward(ctx, sp, x):
        ctx.sp = sp
        return _all_gather_rows(sp, x)

    @staticmethod
    def backward(ctx, dy):
        sp = ctx.sp
        n = dy.shape[0] // sp.world
        return None, dy[sp.rank * n:(sp.rank + 1) * n].contiguous()


def gather_rows(sp, x: torch.Tensor) -> torch.Tensor:
    """``[1, rows/n, H]`` shards -> ``[batch, seq, H]`` on every rank."""
    y = _GatherRows.apply(sp, x.reshape(-1, x.shape[-1]))
    return y.view(sp.batch, sp.seq, y.shape[-1])


def shard_rows(sp, x: torch.Tensor) -> torch.Tensor:
    """This rank's block of the flattened ``[batch * seq, ...]`` rows, as ``[1, rows/n, ...]``."""
    flat = x.reshape(sp.rows, *x.shape[2:])
    n = sp.rows_local
    return flat[sp.rank * n:(sp.rank + 1) * n].unsqueeze(0)


class _SumOverGroupValue(torch.autograd.Function):
    """Forward: sum of a scalar over the group (for reporting); backward: identity (each rank differentiates
    its own term of the sum)."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.detach().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def sum_value_over_group(x: torch.Tensor, group) -> torch.Tensor:
    return _SumOverGroupValue.apply(x, group)
