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
