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


# ---------------------------------------------------------------------------------------------- all-to-all form
_lib.register("edl_ep_arena_bytes", _lib.i64, [_lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32])
_lib.register("edl_ep_arena_offsets", _lib.i32, [_lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp])
_lib.register("edl_ep_plan", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.vp,
                                        _lib.vp, _lib.vp])
_lib.register("edl_ep_dispatch", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                            _lib.vp, _lib.i64, _lib.vp, _lib.i32, _lib.vp, _lib.vp, _lib.vp, _lib.vp,
                                            _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp])
_lib.register("edl_ep_return", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                          _lib.vp, _lib.i64, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.vp, _lib.i64,
                                          _lib.vp, _lib.i32, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp])

PEER_WAIT_MS = 20000     # how long an exchange kernel waits for a peer before it gives up with a status code


class ExchangePlan:
    """Where every token of one MoE call goes: ``send_pos [T, W]`` (row in the region on rank d, or -1),
    ``send_tok [W, cap]``, ``send_count [W]``; ``recv_count [W]`` is filled by the dispatch."""

    __slots__ = ("T", "send_pos", "send_tok", "send_count", "recv_count")


class TokenExchange:
    """Dispatch / return of token rows between the ranks of an expert-parallel group.

    A token row travels once to every rank that owns one of its top-k experts and one partial result per such rank
    travels back (csrc/ep_exchange.cu). On the GPU the rows are stored straight into the peers' symmetric arenas by
    the exchange kernels; without the kernel library (CPU, gloo) the same plan runs over ``all_to_all_single`` with
    fixed-capacity regions, which is what the multi-process CPU tests exercise."""

    def __init__(self, group, device, cap: int, hidden: int, k: int):
        self.group, self.device = group, device
        # group None: one rank exchanging with itself (the kernels run unchanged; used by single-GPU tests)
        self.world, self.rank = (dist.get_world_size(group), dist.get_rank(group)) if group is not None else (1, 0)
        self.cap, self.hidden, self.k = int(cap), int(hidden), int(k)
        self.x_bytes = hidden * 2
        self.a_bytes = (8 * k + 15) // 16 * 16          # k fp32 routing weights | k int32 expert ids
        self.ra_bytes = (4 * k + 15) // 16 * 16         # k fp32 routing-weight gradients
        self.native = device.type == "cuda" and _lib.available()
        # with ``track`` on, every dispatch adds the rows it stores into OTHER ranks to a device counter (reporting)
        self.track = False
        self.rows_remote = torch.zeros((), dtype=torch.int64, device=device)
        self.dispatches = 0
        if self.native:
            import torch.distributed._symmetric_memory as symm

            n = _lib.get().edl_ep_arena_bytes(self.world, self.cap, self.x_bytes, self.a_bytes, self.ra_bytes)
            if n <= 0:
                raise RuntimeError("edl_ep_arena_bytes: " + _lib.get().edl_last_error().decode(errors="replace"))
            if group is None:
                self.arena = torch.zeros(int(n), dtype=torch.uint8, device=device)
                self.ptrs = (C.c_ulonglong * 1)(self.arena.data_ptr())
            else:
                self.arena = symm.empty(int(n), dtype=torch.uint8, device=device)
                self.arena.zero_()
                self.handle = symm.rendezvous(self.arena, group)
                off = int(getattr(self.handle, "offset", 0))
                self.ptrs = (C.c_ulonglong * self.world)(*[int(p) + off for p in self.handle.buffer_ptrs])
            offs = (C.c_longlong * 4)()
            _lib.call("edl_ep_arena_offsets", self.world, self.cap, self.x_bytes, self.a_bytes, self.ra_bytes,
                      C.cast(offs, C.c_void_p))
            self.off_recv_x, self.off_recv_a, self.off_ret_x, self.off_ret_a = (int(v) for v in offs)
            self.sync = torch.zeros(8, dtype=torch.int32, device=device)
            self.tick = torch.zeros(16, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
            if group is not None:
                dist.barrier(group=group)

    # -- plan
    def plan(self, topk_idx: torch.Tensor, experts_per_rank: int) -> ExchangePlan:
        T, k = topk_idx.shape
        if T > self.cap:
            raise ValueError(f"{T} tokens exceed the exchange capacity {self.cap}")
        p = ExchangePlan()
        p.T = T
        W = self.world
        dev = topk_idx.device
        if self.native:
            idx32 = topk_idx.to(torch.int32).contiguous()
            p.send_pos = torch.empty(T, W, dtype=torch.int32, device=dev)
            p.send_tok = torch.empty(W, self.cap, dtype=torch.int32, device=dev)
            p.send_count = torch.empty(W, dtype=torch.int32, device=dev)
            p.recv_count = torch.zeros(W, dtype=torch.int32, device=dev)
            _lib.call("edl_ep_plan", idx32.data_ptr(), T, k, experts_per_rank, W, self.cap, p.send_pos.data_ptr(),
                      p.send_tok.data_ptr(), p.send_count.data_ptr(), _lib.stream_ptr())
            return p
        owner = torch.where(topk_idx >= 0, topk_idx // experts_per_rank, torch.full_like(topk_idx, -1))
        hit = (owner[:, :, None] == torch.arange(W, device=dev)[None, None, :]).any(1)          # [T, W]
        pos = hit.long().cumsum(0) - 1
        p.send_pos = torch.where(hit, pos, torch.full_like(pos, -1)).to(torch.int32)
        p.send_count = hit.sum(0).to(torch.int32)
        p.send_tok = torch.zeros(W, self.cap, dtype=torch.int32, device=dev)
        for d in range(W):
            toks = hit[:, d].nonzero()[:, 0]
            p.send_tok[d, :toks.numel()] = toks.to(torch.int32)
        p.recv_count = torch.zeros(W, dtype=torch.int32, device=dev)
        return p

    # -- dispatch
    def dispatch(self, x: torch.Tensor, aux: torch.Tensor | None, p: ExchangePlan, mask_k: int = 0):
        """``x [T, H]`` bf16 (+ ``aux [T, a_bytes / 4]`` as 32-bit words) -> ``(x_recv [W * cap, H], aux_recv)``.
        On the GPU the results are VIEWS of this rank's arena: they are valid until the next dispatch."""
        W, cap = self.world, self.cap
        if self.track:
            self.rows_remote += p.send_count.sum() - p.send_count[self.rank]
            self.dispatches += 1
        if self.native:
            if x.dtype != torch.bfloat16 or x.stride(-1) != 1 or x.shape[1] != self.hidden:
                raise ValueError("exchange rows must be bf16 [T, hidden] with unit inner stride")
            if aux is not None and (not aux.is_contiguous() or aux.shape[1] * aux.element_size() != self.a_bytes):
                raise ValueError("aux rows must be contiguous and a_bytes wide")
            _lib.call("edl_ep_dispatch", C.cast(self.ptrs, C.c_void_p), W, self.rank, cap, self.x_bytes, self.a_bytes,
                      self.ra_bytes, x.data_ptr(), x.stride(0) * 2, _lib.ptr(aux), mask_k, p.send_tok.data_ptr(),
                      p.send_count.data_ptr(), p.recv_count.data_ptr(), self.sync.data_ptr(), self.tick.data_ptr(), 0,
                      PEER_WAIT_MS, _lib.status_word(x.device).data_ptr(), _lib.stream_ptr())
            rows = W * cap
            x_recv = self.arena[self.off_recv_x:self.off_recv_x + rows * self.x_bytes].view(torch.bfloat16) \
                .view(rows, self.hidden)
            a_recv = None
            if aux is not None:
                a_recv = self.arena[self.off_recv_a:self.off_recv_a + rows * self.a_bytes].view(torch.int32) \
                    .view(rows, self.a_bytes // 4)
            return x_recv, a_recv
        # torch.distributed form: fixed-capacity regions, counts first
        H = x.shape[1]
        send = x.new_zeros(W, cap, H)
        tok = p.send_tok.long()
        for d in range(W):
            n = int(p.send_count[d])
            send[d, :n] = x[tok[d, :n]]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv.view(W * cap, H), send.view(W * cap, H), group=self.group)
        counts = p.send_count.clone()
        rc = torch.empty_like(counts)
        dist.all_to_all_single(rc, counts, group=self.group)
        p.recv_count = rc
        a_recv = None
        if aux is not None:
            A = aux.shape[1]
            sa = aux.new_zeros(W, cap, A)
            for d in range(W):
                n = int(p.send_count[d])
                sa[d, :n] = aux[tok[d, :n]]
            ra = torch.empty_like(sa)
            dist.all_to_all_single(ra.view(W * cap, A), sa.view(W * cap, A), group=self.group)
            if mask_k:
                unused = torch.arange(cap, device=ra.device)[None, :] >= rc.long()[:, None]
                ra[:, :, mask_k:2 * mask_k] = torch.where(unused[:, :, None], torch.full_like(ra[:, :, :mask_k], -1),
                                                          ra[:, :, mask_k:2 * mask_k])
            a_recv = ra.view(W * cap, A)
        return recv.view(W * cap, H), a_recv

    # -- return
    def ret(self, y: torch.Tensor, aux: torch.Tensor | None, p: ExchangePlan, aux_floats: int = 0):
        """``y [W * cap, H]`` (+ fp32 ``aux [W * cap, ra_bytes / 4]``) -> ``(out [T, H], out_aux [T, aux_floats])``:
        for every token the sum, in rank order, of the rows the expert ranks computed for it."""
        W, cap, T = self.world, self.cap, p.T
        if self.native:
            if y.dtype != torch.bfloat16 or y.stride(-1) != 1 or y.shape != (W * cap, self.hidden):
                raise ValueError("returned rows must be bf16 [world * cap, hidden]")
            if aux is not None and (aux.dtype != torch.float32 or not aux.is_contiguous() or
                                    aux.shape[1] * 4 != self.ra_bytes):
                raise ValueError("returned aux rows must be contiguous fp32, ra_bytes wide")
            out = torch.empty(T, self.hidden, dtype=torch.bfloat16, device=y.device)
            out_aux = torch.empty(T, aux_floats, dtype=torch.float32, device=y.device) if aux is not None else None
            _lib.call("edl_ep_return", C.cast(self.ptrs, C.c_void_p), W, self.rank, cap, self.x_bytes, self.a_bytes,
                      self.ra_bytes, y.data_ptr(), y.stride(0) * 2, _lib.ptr(aux), p.recv_count.data_ptr(),
                      p.send_pos.data_ptr(), T, out.data_ptr(), out.stride(0) * 2, _lib.ptr(out_aux), aux_floats,
                      self.sync.data_ptr(), self.tick.data_ptr(), 0, PEER_WAIT_MS,
                      _lib.status_word(y.device).data_ptr(), _lib.stream_ptr())
            return out, out_aux
        H = y.shape[1]
        back = torch.empty(W, cap, H, dtype=y.dtype, device=y.device)
        dist.all_to_all_single(back.view(W * cap, H), y.contiguous().view(W * cap, H), group=self.group)
        pos = p.send_pos.long()                                  # [T, W]
        ok = pos >= 0
        rows = back[torch.arange(W, device=y.device)[None, :].expand(T, W), pos.clamp_min(0)]      # [T, W, H]
        out = (rows.float() * ok[:, :, None]).sum(1).to(y.dtype)
        out_aux = None
        if aux is not None:
            A = aux.shape[1]
            ba = torch.empty(W, cap, A, dtype=aux.dtype, device=aux.device)
            dist.all_to_all_single(ba.view(W * cap, A), aux.contiguous().view(W * cap, A), group=self.group)
            ra = ba[torch.arange(W, device=y.device)[None, :].expand(T, W), pos.clamp_min(0)]
            out_aux = (ra * ok[:, :, None]).sum(1)[:, :aux_floats].contiguous()
        return out, out_aux

    def remote_rows(self, p: ExchangePlan) -> int:
        """Rows this rank sends to OTHER ranks under ``p`` (a host read: for reporting, not for the hot path)."""
        c = p.send_count.clone()
        c[self.rank] = 0
        return int(c.sum())


_TOKEN_EXCHANGES: dict[tuple, TokenExchange] = {}


def token_exchange(group, device, cap: int, hidden: int, k: int) -> TokenExchange:
    key = (id(group), device.type, device.index, int(hidden), int(k))
    ex = _TOKEN_EXCHANGES.get(key)
    if ex is None or ex.cap < cap:
        ex = _TOKEN_EXCHANGES[key] = TokenExchange(group, device, cap, hidden, k)
    return ex


def release_token_exchanges() -> None:
    """Drops the symmetric arenas (before the process group is destroyed)."""
    _TOKEN_EXCHANGES.clear()


class _DispatchTokens(torch.autograd.Function):
    """x, routing weights, expert ids -> the rows (and routing data) this rank's experts have to process.
    Backward: the gradients of those rows (and of the received routing weights) travel back and are summed."""

    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, ex: TokenExchange, experts_per_rank: int):
        k = topk_idx.shape[1]
        plan = ex.plan(topk_idx, experts_per_rank)
        aux = torch.zeros(x.shape[0], ex.a_bytes // 4, dtype=torch.int32, device=x.device)
        aux[:, :k] = topk_w.detach().to(torch.float32).contiguous().view(torch.int32)
        aux[:, k:2 * k] = topk_idx.to(torch.int32)
        x_recv, a_recv = ex.dispatch(x.detach(), aux, plan, mask_k=k)
        w_recv = a_recv[:, :k].contiguous().view(torch.float32)       # copies: the arena is overwritten later
        idx_recv = a_recv[:, k:2 * k].contiguous().long()
        ctx.ex, ctx.plan, ctx.k, ctx.w_dtype = ex, plan, k, topk_w.dtype
        ctx.mark_non_differentiable(idx_recv)
        ctx.set_materialize_grads(False)
        return x_recv, w_recv, idx_recv, _PlanHandle(plan)

    @staticmethod
    def backward(ctx, dx_recv, dw_recv, _idx, _plan):
        ex, plan, k = ctx.ex, ctx.plan, ctx.k
        rows = ex.world * ex.cap
        if dx_recv is None:
            dx_recv = torch.zeros(rows, ex.hidden, dtype=torch.bfloat16, device=plan.send_pos.device)
        aux = None
        if dw_recv is not None:
            aux = torch.zeros(rows, ex.ra_bytes // 4, dtype=torch.float32, device=dx_recv.device)
            aux[:, :k] = dw_recv.to(torch.float32)
        dx, dw = ex.ret(dx_recv.contiguous(), aux, plan, aux_floats=k)
        return dx, (dw.to(ctx.w_dtype) if dw is not None else None), None, None, None


class _PlanHandle:
    """Carries the plan of a dispatch to the matching return through autograd (an opaque, non-tensor output)."""

    def __init__(self, plan):
        self.plan = plan


class _ReturnTokens(torch.autograd.Function):
    """Partial results of the received rows -> per-token sums on the owner. Backward: the gradient of every token's
    result is dispatched to the ranks that contributed to it."""

    @staticmethod
    def forward(ctx, y_part, ex: TokenExchange, plan: ExchangePlan):
        ctx.ex, ctx.plan = ex, plan
        out, _ = ex.ret(y_part.detach().contiguous(), None, plan)
        return out

    @staticmethod
    def backward(ctx, dy):
        dy_recv, _ = ctx.ex.dispatch(dy.contiguous(), None, ctx.plan)
        return dy_recv, None, None


def expert_parallel_ffn_alltoall(block, x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor) -> torch.Tensor:
    """The expert FFN of one MoE layer with tokens dispatched only to the ranks that own their experts."""
    from ..ops import grouped

    group = block.ep_group
    T, H = x.shape
    k = topk_idx.shape[1]
    ex = token_exchange(group, x.device, T, H, k)
    x_recv, w_recv, idx_recv, handle = _DispatchTokens.apply(x, topk_w, topk_idx, ex, block.num_local_experts)
    offset = block.ep_rank * block.num_local_experts
    b_gu, b_d = block.gate_up_proj.bias, block.down_proj.bias
    if _lib.use_kernels(x_recv):
        y_part = grouped.moe_ffn(x_recv, block.gate_up_proj.weight, block.down_proj.weight, w_recv, idx_recv, block.act,
                                 expert_offset=offset, b_gate_up=b_gu, b_down=b_d)
    else:
        local = idx_recv - offset
        mine = (local >= 0) & (local < block.num_local_experts) & (idx_recv >= 0)
        y_part = grouped.moe_ffn(x_recv, block.gate_up_proj.weight, block.down_proj.weight,
                                 w_recv * mine.to(w_recv.dtype), local.clamp(0, block.num_local_experts - 1), block.act,
                                 b_gate_up=b_gu, b_down=b_d)
    return _ReturnTokens.apply(y_part, ex, handle.plan)


def ep_dispatch_mode() -> str:
    """``EP_DISPATCH`` = auto | alltoall | allgather (auto: all-to-all)."""
    import os

    mode = os.environ.get("EP_DISPATCH", "auto").lower()
    if mode not in ("auto", "alltoall", "allgather"):
        raise ValueError(f"EP_DISPATCH={mode!r}: expected auto, alltoall or allgather")
    return "alltoall" if mode == "auto" else mode


def expert_parallel_ffn(block, x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor) -> torch.Tensor:
    """``block`` is a ``MoEBlock`` holding this rank's experts (``gate_up_proj`` / ``down_proj`` of
    ``num_local_experts``); x ``[T, H]`` are this rank's tokens with global expert indices ``topk_idx [T, k]``."""
    if ep_dispatch_mode() == "alltoall":
        return expert_parallel_ffn_alltoall(block, x, topk_w, topk_idx)
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
