"""Context-parallel (sequence-sharded) attention over NVLink peer memory.

Each rank holds a contiguous slice of the sequence. Keys and values live in a symmetric allocation, so the flash
attention kernel of rank ``i`` reads the slice of rank ``r`` straight from that GPU's memory with its TMA loads
(no staging copy, no collective): one kernel launch per visited rank produces a partial output and its
log-sum-exp, and the partials are merged exactly by ``attn_combine``. With a causal mask rank ``i`` visits ranks
``0..i`` (the diagonal block is the only one that needs the mask).

The backward pass re-visits the same blocks with the merged ``(o, lse)``; the key / value gradients of a remote
block are written by the kernel into the owner's staging slot for this rank and summed by the owner.

This is what the reference's ring attention (ejkernel ring attention reached from
easydel/operations/kernels/ring_attention.py, rotating KV with ``ppermute``) computes; on NVSwitch every peer is one
hop away at full bandwidth, so blocks are pulled directly instead of being passed around a ring.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import serving as S


class ContextParallelAttention:
    def __init__(self, group, tokens_per_rank: int, num_kv_heads: int, head_dim: int, device,
                 dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.T, self.Hkv, self.D, self.dtype = tokens_per_rank, num_kv_heads, head_dim, dtype
        n_kv = tokens_per_rank * num_kv_heads * head_dim
        # [k | v | dk slots (world) | dv slots (world)]
        self.numel = n_kv * (2 + 2 * self.world)
        self.buf = symm.empty(self.numel, dtype=dtype, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        self.n_kv = n_kv
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _peer(self, rank: int, index: int) -> torch.Tensor:
        """Block ``index`` (0 = k, 1 = v, 2 + s = dk slot s, 2 + world + s = dv slot s) of ``rank``'s buffer."""
        t = self.handle.get_buffer(rank, (self.n_kv,), self.dtype, index * self.n_kv)
        return t.view(self.T, self.Hkv, self.D)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                scale: float | None = None) -> torch.Tensor:
        """q ``[T, Hq, D]``, k / v ``[T, Hkv, D]``: this rank's slice of one sequence. Returns ``[T, Hq, D]``."""
        return _CPAttn.apply(q, k, v, self, causal, scale)

    __call__ = forward


class _CPAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cp: ContextParallelAttention, causal, scale):
        T, Hq, D = q.shape
        me, n = cp.rank, cp.world
        cp._peer(me, 0).copy_(k)
        cp._peer(me, 1).copy_(v)
        cp.handle.barrier(channel=0)
        visit = list(range(me + 1)) if causal else list(range(n))
        o_parts = torch.empty(len(visit), T, Hq, D, dtype=q.dtype, device=q.device)
        lses = []
        q4 = q.contiguous()[None]
        for s, r in enumerate(visit):
            kr, vr = cp._peer(r, 0)[None], cp._peer(r, 1)[None]
            _, lse = A.attn_fwd(q4, kr, vr, causal=bool(causal and r == me), scale=scale, out=o_parts[s][None])
            lses.append(lse)
        o, lse = S.attn_combine(o_parts, torch.stack(lses), want_lse=True)
        cp.handle.barrier(channel=1)      # every rank is done reading before anybody overwrites its keys
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cp, ctx.causal, ctx.scale, ctx.visit = cp, causal, scale, visit
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        cp, causal, scale, visit = ctx.cp, ctx.causal, ctx.scale, ctx.visit
        me, n = cp.rank, cp.world
        cp._peer(me, 0).copy_(k)
        cp._peer(me, 1).copy_(v)
        for s in range(n):                # zero my staging slots: ranks that do not visit me leave them untouched
            cp._peer(me, 2 + s).zero_()
            cp._peer(me, 2 + n + s).zero_()
        cp.handle.barrier(channel=2)
        dq = torch.zeros_like(q, dtype=torch.float32)
        q4, o4, do4 = q.contiguous()[None], o.contiguous()[None], do.contiguous()[None]
        for r in visit:
            kr, vr = cp._peer(r, 0)[None], cp._peer(r, 1)[None]
            dkr, dvr = cp._peer(r, 2 + me)[None], cp._peer(r, 2 + n + me)[None]   # my slot on the owner
            dq_r, _, _ = A.attn_bwd(q4, kr, vr, o4, lse, do4, causal=bool(causal and r == me), scale=scale,
                                    dk=dkr, dv=dvr)
            dq += dq_r[0].float()
        cp.handle.barrier(channel=3)      # all partial key / value gradients have landed
        dk = torch.zeros_like(k, dtype=torch.float32)
        dv = torch.zeros_like(v, dtype=torch.float32)
        for s in range(n):
            dk += cp._peer(me, 2 + s).float()
            dv += cp._peer(me, 2 + n + s).float()
        cp.handle.barrier(channel=4)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None


def context_parallel_attention_reference(q, k, v, group, causal=True, scale=None):
    """All-gather keys / values with NCCL and run dense attention for this rank's queries (test oracle)."""
    from ..ops import reference as R

    n, me = dist.get_world_size(group), dist.get_rank(group)
    ks = [torch.empty_like(k) for _ in range(n)]
    vs = [torch.empty_like(v) for _ in range(n)]
    dist.all_gather(ks, k.contiguous(), group=group)
    dist.all_gather(vs, v.contiguous(), group=group)
    kf, vf = torch.cat(ks, 0), torch.cat(vs, 0)
    T = q.shape[0]
    if causal:
        kf, vf = kf[: (me + 1) * T], vf[: (me + 1) * T]
    return R.attention(q[None], kf[None], vf[None], causal=causal, scale=scale)[0]


# ------------------------------------------------------------------------------------------------------------------
# Sequence sharding of a batch and the attention that goes with it on the model path (``attn_mechanism="ring"`` with
# an ``sp`` mesh axis > 1; the reference shards the batch ``P(("dp", "fsdp"), "sp")``,
# easydel/trainers/training_utils.py:763-765, and runs ring attention, easydel/operations/kernels/ring_attention.py:84-260).
#
# Layouts of the sequence over the ``n`` ranks of the group:
#   contiguous  rank r holds tokens [r * T/n, (r + 1) * T/n)
#   zigzag      the sequence is cut into 2n chunks and rank r holds chunks r and 2n - 1 - r, so that under a causal
#               mask every rank has the same number of (query, key) pairs to compute
# Keys and values are small next to the queries under grouped-query attention, so every rank gathers all of them
# (the gather's backward is the reduce-scatter that sums the key / value gradients on their owners) and runs the flash
# kernel once per local chunk against the keys in front of that chunk's end; the "fewer queries than keys" causal
# form of the kernel puts the diagonal where it belongs.
LAYOUTS = ("contiguous", "zigzag")


def shard_positions(total: int, rank: int, world: int, layout: str = "zigzag") -> torch.Tensor:
    """Global positions of the tokens rank ``rank`` holds, in the order it holds them."""
    if layout not in LAYOUTS:
        raise ValueError(f"sequence layout {layout!r}: expected one of {LAYOUTS}")
    parts = world if layout == "contiguous" else 2 * world
    if total % parts:
        raise ValueError(f"sequence length {total} is not a multiple of {parts} ({layout} over {world} ranks)")
    c = total // parts
    if layout == "contiguous":
        return torch.arange(rank * c, (rank + 1) * c)
    return torch.cat([torch.arange(rank * c, (rank + 1) * c),
                      torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)])


def shard_sequence(t: torch.Tensor, rank: int, world: int, layout: str = "zigzag", dim: int = 1) -> torch.Tensor:
    idx = shard_positions(t.shape[dim], rank, world, layout).to(t.device)
    return t.index_select(dim, idx)


def shard_batch(batch: dict, rank: int, world: int, layout: str = "zigzag") -> dict:
    """This rank's slice of a causal-LM batch. Labels are shifted to the next token on the whole sequence first (the
    token after a shard's last one lives on another rank), so the result carries ``labels_shifted=True``;
    ``position_ids`` hold the global positions."""
    ids = batch["input_ids"]
    B, T = ids.shape
    labels = batch.get("labels", ids)
    shifted = torch.full_like(labels, -100)
    shifted[:, :-1] = labels[:, 1:]
    if batch.get("attention_mask") is not None:
        shifted = torch.where(torch.nn.functional.pad(batch["attention_mask"][:, 1:], (0, 1)).bool(), shifted,
                              torch.full_like(shifted, -100))
    pos = batch.get("position_ids")
    if pos is None:
        pos = torch.arange(T, device=ids.device)[None].expand(B, T)
    out = dict(batch)
    for name, t in (("input_ids", ids), ("labels", shifted), ("position_ids", pos)):
        out[name] = shard_sequence(t, rank, world, layout)
    for name in ("attention_mask", "segment_ids"):
        if batch.get(name) is not None:
            out[name] = shard_sequence(batch[name], rank, world, layout)
    out["labels_shifted"] = True
    return out


def gathered_kv_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, *, layout: str = "zigzag",
                          causal: bool = True, scale: float | None = None, softcap: float = 0.0) -> torch.Tensor:
    """Attention of this rank's query shard ``[B, Tl, Hq, D]`` over the keys / values of the whole sequence, whose
    shards ``[B, Tl, Hkv, D]`` are spread over ``group`` in ``layout``. Differentiable."""
    from ..ops import functional as F
    from .ep import all_gather_tokens

    n, r = dist.get_world_size(group), dist.get_rank(group)
    B, Tl, Hkv, D = k.shape
    kv = torch.stack([k, v], 0).reshape(2 * B * Tl, Hkv * D)              # one exchange for both
    kv_all = all_gather_tokens(kv.contiguous(), group).view(n, 2, B, Tl, Hkv, D)
    if layout == "contiguous":
        k_all = kv_all[:, 0].permute(1, 0, 2, 3, 4).reshape(B, n * Tl, Hkv, D)
        v_all = kv_all[:, 1].permute(1, 0, 2, 3, 4).reshape(B, n * Tl, Hkv, D)
        if not causal:
            return F.attention(q, k_all, v_all, causal=False, scale=scale, softcap=softcap)
        end = (r + 1) * Tl
        return F.attention(q, k_all[:, :end], v_all[:, :end], causal=True, scale=scale, softcap=softcap)
    c = Tl // 2
    # global order: chunk s is the first half of rank s, chunk 2n - 1 - s the second half of rank s
    halves = kv_all.view(n, 2, B, 2, c, Hkv, D)
    early = halves[:, :, :, 0]                                             # [n, 2, B, c, Hkv, D] chunks 0 .. n-1
    late = halves[:, :, :, 1].flip(0)                                      # chunks n .. 2n-1
    full = torch.cat([early, late], 0)                                     # [2n, 2, B, c, Hkv, D] in global order
    k_all = full[:, 0].permute(1, 0, 2, 3, 4).reshape(B, 2 * n * c, Hkv, D)
    v_all = full[:, 1].permute(1, 0, 2, 3, 4).reshape(B, 2 * n * c, Hkv, D)
    if not causal:
        return F.attention(q, k_all, v_all, causal=False, scale=scale, softcap=softcap)
    e0, e1 = (r + 1) * c, (2 * n - r) * c
    o0 = F.attention(q[:, :c], k_all[:, :e0], v_all[:, :e0], causal=True, scale=scale, softcap=softcap)
    o1 = F.attention(q[:, c:], k_all[:, :e1], v_all[:, :e1], causal=True, scale=scale, softcap=softcap)
    return torch.cat([o0, o1], 1)


_PEER_CP: dict[tuple, ContextParallelAttention] = {}


def ring_attention(q, k, v, group, *, layout: str = "zigzag", causal: bool = True, scale: float | None = None,
                   softcap: float = 0.0, impl: str = "auto") -> torch.Tensor:
    """Sequence-parallel attention for the model path. ``impl``: ``gather`` = all keys / values gathered, flash
    kernel per local chunk (any layout, any device); ``peer`` = remote key blocks read in place over NVLink by the
    flash kernel's own loads (contiguous layout, CUDA, no soft-cap, batch 1); ``auto`` picks ``peer`` when it
    applies and the layout is contiguous."""
    from ..ops import _lib

    peer_ok = (layout == "contiguous" and q.is_cuda and _lib.available() and not softcap and q.shape[0] == 1 and
               q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128))
    if impl == "peer" and not peer_ok:
        raise ValueError("the peer-memory form needs the contiguous layout, one bf16 sequence per rank on CUDA, "
                         "head size 64 or 128 and no soft-cap")
    if impl == "peer" or (impl == "auto" and peer_ok):
        T, Hkv, D = k.shape[1], k.shape[2], k.shape[3]
        key = (id(group), T, Hkv, D, q.device.index)
        cp = _PEER_CP.get(key)
        if cp is None:
            cp = _PEER_CP[key] = ContextParallelAttention(group, T, Hkv, D, q.device, q.dtype)
        return cp(q[0], k[0], v[0], causal=causal, scale=scale)[None]
    return gathered_kv_attention(q, k, v, group, layout=layout, causal=causal, scale=scale, softcap=softcap)


def release_peer_buffers() -> None:
    _PEER_CP.clear()
