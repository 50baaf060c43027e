"""GEMMs fused with their collective over NVLink peer memory (``csrc/gemm_collective.cu``).

* :class:`GemmReduceScatter`: row-parallel linear whose epilogue pushes each output tile to the
  rank that owns those rows, followed in the same kernel by the reduction of the owner's shard.
  It replaces ``matmul`` + NCCL ``reduce_scatter`` of a sequence-parallel tensor-parallel block
  (the reference leaves this to XLA's partitioner: easydel/layers/linears/_linear.py:348-378).
* :class:`AllGatherGemm`: the mirror image: row shards of the activation (or of an FSDP-sharded
  weight) are pulled from the peers by copier CTAs while the tensor cores already work on the
  local shard.

Both keep their staging buffers in one symmetric allocation per (group, shape) and fall back to
``torch.distributed`` collectives + a plain GEMM where peer memory is not available (CPU, gloo).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib

_lib.register("edl_gemm_reduce_scatter", _lib.i32,
              [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i64, _lib.i64,
               _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.i32])
_lib.register("edl_allgather_gemm", _lib.i32,
              [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i64, _lib.i64,
               _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.i32])

_FLAG_BYTES = 256


def _peer_capable(x: torch.Tensor) -> bool:
    return x.is_cuda and _lib.available()


class _LocalHandle:
    """Stand-in for the symmetric-memory handle of a one-rank group."""

    def barrier(self, channel: int = 0):
        return None


def _world(group) -> tuple[int, int]:
    if group is None:
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _rendezvous(nbytes: int, group, device):
    if _world(group)[0] == 1:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        return buf, _LocalHandle(), [buf.data_ptr()]
    import torch.distributed._symmetric_memory as symm

    buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    handle = symm.rendezvous(buf, group)
    off = int(getattr(handle, "offset", 0))
    base = [int(p) + off for p in handle.buffer_ptrs]
    if base[dist.get_rank(group)] != buf.data_ptr():
        raise RuntimeError("symmetric-memory handle does not address this rank's own buffer")
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    return buf, handle, base


class GemmReduceScatter:
    """``out[M/n, N] = reduce_scatter_rows(a @ w.T) (+ residual) (+ bias)`` with ``a``/``w`` sharded over K."""

    def __init__(self, group, rows_per_rank: int, n_out: int, device):
        self.group = group
        self.world, self.rank = _world(group)
        self.rows, self.n_out = rows_per_rank, n_out
        self.slot_bytes = self.world * rows_per_rank * n_out * 2
        w = self.world
        blocks = rows_per_rank // 128
        # one flag per (source rank, 128-row block) and slot
        flag_bytes = max(_FLAG_BYTES, (4 * w * blocks + 255) // 256 * 256)
        self.buf, self.handle, base = _rendezvous(2 * self.slot_bytes + 2 * flag_bytes, group, device)
        self.stage_ptrs = [(C.c_ulonglong * w)(*[b + s * self.slot_bytes for b in base]) for s in range(2)]
        self.flag_ptrs = [(C.c_ulonglong * w)(*[b + 2 * self.slot_bytes + s * flag_bytes for b in base])
                          for s in range(2)]
        self.counters = torch.zeros(w * blocks + 1, dtype=torch.int32, device=device)
        self.epoch = 0

    def __call__(self, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
                 bias: torch.Tensor | None = None, wait_ms: int = 2000, b_mn: bool = False) -> torch.Tensor:
        """``b_mn``: ``w`` is stored ``[K, N]`` (the product is ``a @ w``, a data-gradient GEMM)."""
        M, K = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if M != self.rows * self.world or N != self.n_out:
            raise ValueError(f"shape ({M},{N}) does not match the plan ({self.rows * self.world},{self.n_out})")
        self.epoch += 1
        s = self.epoch & 1
        out = torch.empty(self.rows, N, dtype=torch.bfloat16, device=a.device)
        _lib.call("edl_gemm_reduce_scatter", a.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(residual),
                  _lib.ptr(bias), M, N, K, a.stride(0), w.stride(0), C.cast(self.stage_ptrs[s], C.c_void_p),
                  C.cast(self.flag_ptrs[s], C.c_void_p), self.counters.data_ptr(), self.world, self.rank,
                  self.epoch, wait_ms, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr(), int(b_mn))
        return out


class AllGatherGemm:
    """``c[n*Ms, N] = all_gather_rows(a_shard) @ w.T (+ bias)``; also returns the gathered operand."""

    def __init__(self, group, rows_per_rank: int, k: int, device, n_copy: int = 0):
        self.group = group
        self.world, self.rank = _world(group)
        self.rows, self.k, self.n_copy = rows_per_rank, k, n_copy
        self.buf, self.handle, base = _rendezvous(rows_per_rank * k * 2, group, device)
        self.shard = self.buf.view(torch.bfloat16).view(rows_per_rank, k)
        self.shard_ptrs = (C.c_ulonglong * self.world)(*base)
        self.gathered = torch.empty(self.world * rows_per_rank, k, dtype=torch.bfloat16, device=device)
        self.counters = torch.zeros(self.world * (rows_per_rank // 128), dtype=torch.int32, device=device)

    def __call__(self, a_shard: torch.Tensor | None, w: torch.Tensor, bias: torch.Tensor | None = None,
                 copy_own: bool = True, wait_ms: int = 2000, b_mn: bool = False):
        """``a_shard=None`` means the caller already wrote its rows into ``self.shard``. ``b_mn``: ``w`` is
        stored ``[K, N]`` (the product is ``gather(a) @ w``)."""
        if a_shard is not None:
            self.shard.copy_(a_shard)
        N = w.shape[1] if b_mn else w.shape[0]
        c = torch.empty(self.world * self.rows, N, dtype=torch.bfloat16, device=w.device)
        self.handle.barrier(channel=0)     # every rank's shard is in place
        _lib.call("edl_allgather_gemm", C.cast(self.shard_ptrs, C.c_void_p), w.data_ptr(), c.data_ptr(),
                  _lib.ptr(bias), self.gathered.data_ptr(), self.rows, N, self.k, w.stride(0), c.stride(0),
                  self.counters.data_ptr(), self.world, self.rank, self.n_copy, int(copy_own), wait_ms,
                  _lib.status_word(w.device).data_ptr(), _lib.stream_ptr(), int(b_mn))
        self.handle.barrier(channel=1)     # nobody rewrites a shard that a peer is still reading
        return c, self.gathered


# ------------------------------------------------------------------------------------------------
# Reference implementations over torch.distributed (CPU / gloo, and the oracle of the GPU tests)
# ------------------------------------------------------------------------------------------------
def gemm_reduce_scatter_reference(a, w, group, residual=None, bias=None):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full = a.float() @ w.float().t()
    dist.all_reduce(full, group=group)
    rows = full.shape[0] // world
    out = full[rank * rows:(rank + 1) * rows]
    if residual is not None:
        out = out + residual.float()
    if bias is not None:
        out = out + bias.float()
    return out


def allgather_gemm_reference(a_shard, w, group, bias=None):
    world = dist.get_world_size(group)
    parts = [torch.empty_like(a_shard) for _ in range(world)]
    dist.all_gather(parts, a_shard.contiguous(), group=group)
    g = torch.cat(parts, 0)
    c = g.float() @ w.float().t()
    if bias is not None:
        c = c + bias.float()
    return c, g
