"""Expert parallelism over NVLink peer memory.

Each rank owns ``E / ep`` experts and a slice of the tokens. The expert FFN of one MoE layer runs as

    all-gather(tokens, routing)  ->  local experts on every token routed to them  ->  reduce-scatter(outputs)

where both collectives are kernels that read the peers' symmetric buffers directly (``csrc/collectives.cu``) and
are autograd functions of each other (the backward of the gather is the reduce-scatter and vice versa). For the
top-8-of-128 routing of Qwen3-MoE on 8 ranks the volume equals that of a token all-to-all (each token visits about
5 of the 8 ranks either way), without the variable-size bookkeeping: the device-side routing tables simply skip
the pairs whose expert lives elsewhere. The reference reaches the same result through ``shard_map`` +
``ragged_all_to_all`` / ``psum_scatter`` (easydel/layers/moe: MoE fused dispatch with expert-parallel axes).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe_kernels as G

_lib.register("edl_peer_gather", _lib.i32, [_lib.vp, _lib.i32, _lib.i64, _lib.vp, _lib.vp])
_lib.register("edl_peer_reduce_bf16", _lib.i32, [_lib.vp, _lib.i32, _lib.i64, _lib.i64, _lib.vp, _lib.vp])


class _PeerExchange:
    """Two alternating symmetric slots per process group, grown on demand (collectively: shapes are symmetric)."""

    def __init__(self, group, device):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.capacity = 0
        self.calls = 0

    def _ensure(self, nbytes: int) -> None:
        if nbytes <= self.capacity:
            return
        import torch.distributed._symmetric_memory as symm

        cap = max(nbytes, 2 * self.capacity, 1 << 20)
        cap = (cap + 255) // 256 * 256
        self.buf = symm.empty(2 * cap, dtype=torch.uint8, device=self.device)
        self.handle = symm.rendezvous(self.buf, self.group)
        off = int(getattr(self.handle, "offset", 0))
        base = [int(p) + off for p in self.handle.buffer_ptrs]
        self.ptrs = [(C.c_ulonglong * self.world)(*[b + s * cap for b in base]) for s in range(2)]
        self.capacity = cap
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _stage(self, t: torch.Tensor) -> int:
        """Copies ``t`` into this rank's current slot; returns the slot index."""
        nbytes = t.numel() * t.element_size()
        self._ensure(nbytes)
        self.calls += 1
        s = self.calls & 1
        flat = self.buf[s * self.capacity: s * self.capacity + nbytes]
        flat.copy_(t.contiguous().view(-1).view(torch.uint8))
        self.handle.barrier(channel=s)
        return s

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        nbytes = t.numel() * t.element_size()
        pad = (-nbytes) % 16
        if pad:
            raise ValueError("peer all-gather needs a multiple of 16 bytes per rank")
        s = self._stage(t)
        out = torch.empty((self.world * t.shape[0], *t.shape[1:]), dtype=t.dtype, device=t.device)
        _lib.call("edl_peer_gather", C.cast(self.ptrs[s], C.c_void_p), self.world, nbytes, out.data_ptr(),
                  _lib.stream_ptr())
        return out

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """``t [world * rows, ...]`` bf16 on every rank -> this rank's ``rows`` summed over ranks."""
        if t.dtype != torch.bfloat16:
            raise ValueError("peer reduce-scatter works on bf16")
        rows = t.shape[0] // self.world
        per = t[0].numel() * rows
        if per % 8:
            raise ValueError("peer reduce-scatter needs a multiple of 8 elements per rank")
        s = self._stage(t)
        out = torch.empty((rows, *t.shape[1:]), dtype=t.dtype, device=t.device)
        _lib.call("edl_peer_reduce_bf16", C.cast(self.ptrs[s], C.c_void_p), self.world, self.rank * per, per,
                  out.data_ptr(), _lib.stream_ptr())
        return out


_EXCHANGES: dict[int, _PeerExchange] = {}


def _exchange(group, device) -> _PeerExchange | None:
    if device.type != "cuda" or not _lib.available():
        return None
    key = id(group)
    if key not in _EXCHANGES:
        _EXCHANGES[key] = _PeerExchange(group, device)
    return _EXCHANGES[key]


def _ag_raw(t: torch.Tensor, group) -> torch.Tensor:
    ex = _exchange(group, t.device)
    if ex is not None:
        return ex.all_gather(t)
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, 0)


def _rs_raw(t: torch.Tensor, group) -> torch.Tensor:
    ex = _exchange(group, t.device)
    if ex is not None and t.dtype == torch.bfloat16:
        return ex.reduce_scatter(t)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full = t.contiguous().clone()
    dist.all_reduce(full, group=group)
    rows = t.shape[0] // world
    return full[rank * rows:(rank + 1) * rows].contiguous()


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _ag_raw(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _rs_raw(dy.contiguous(), ctx.group), None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _rs_raw(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _ag_raw(dy.contiguous(), ctx.group), None


def all_gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _AllGather.apply(x, group)


def reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    return _ReduceScatter.apply(x, group)


def expert_parallel_ffn(block, x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor) -> torch.Tensor:
    """``block`` is a ``MoEBlock`` holding this rank's experts (``gate_up_proj`` / ``down_proj`` of
    ``num_local_experts``); x ``[T, H]`` are this rank's tokens with global expert indices ``topk_idx [T, k]``."""
    group = block.ep_group
    x_all = all_gather_tokens(x, group)
    w_all = all_gather_tokens(topk_w.to(torch.float32).contiguous(), group).to(topk_w.dtype)
    idx_all = _ag_raw(topk_idx.to(torch.int32).contiguous(), group).long()
    offset = block.ep_rank * block.num_local_experts
    from ..ops import grouped

    b_gu, b_d = block.gate_up_proj.bias, block.down_proj.bias
    if _lib.use_kernels(x_all):
        y_part = grouped.moe_ffn(x_all, block.gate_up_proj.weight, block.down_proj.weight, w_all, idx_all, block.act,
                                 expert_offset=offset, b_gate_up=b_gu, b_down=b_d)
    else:   # reference path: pairs owned by other ranks get weight zero
        local = idx_all - offset
        mine = (local >= 0) & (local < block.num_local_experts)
        y_part = grouped.moe_ffn(x_all, block.gate_up_proj.weight, block.down_proj.weight,
                                 w_all * mine.to(w_all.dtype), local.clamp(0, block.num_local_experts - 1), block.act,
                                 b_gate_up=b_gu, b_down=b_d)
    return reduce_scatter_tokens(y_part.contiguous(), group)
