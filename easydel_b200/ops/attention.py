"""Flash-attention entry points backed by the tcgen05 kernels in ``csrc/attention_*.cu``."""

from __future__ import annotations

import math

import torch

from . import _lib

vp, i32, i64, f32 = _lib.vp, _lib.i32, _lib.i64, _lib.f32
_lib.register("edl_attn_fwd", i32, [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, vp, i32, i32, i32, i64, i64, i32, i32,
                                    i32, f32, i32, i32, f32, vp, vp, vp])
_lib.register("edl_attn_bwd", i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64,
                                    vp, vp, i32, i32, i32, i64, i64, i32, i32, i32, f32, i32, i32, f32, vp, vp])


def _rows(t: torch.Tensor) -> tuple[torch.Tensor, int]:
    """Views ``[..., H, D]`` as token rows; returns (tensor, row stride in elements)."""
    assert t.stride(-1) == 1 and t.stride(-2) == t.shape[-1], "heads must be packed contiguously inside a token row"
    return t, t.stride(-3)


def attn_fwd(q, k, v, *, causal=True, scale=None, window=0, softcap=0.0, sinks=None, cu_q=None, cu_k=None,
             max_q=None, max_k=None, out=None, want_lse=True):
    """q ``[B,Tq,Hq,D]`` (or ``[total,Hq,D]`` with ``cu_q``), k/v likewise. Returns (o, lse[Hq,total_q])."""
    varlen = cu_q is not None
    if varlen:
        total_q, Hq, D = q.shape
        total_k, Hkv = k.shape[0], k.shape[1]
        B = cu_q.numel() - 1
        Tq, Tk = int(max_q), int(max_k)
        if cu_k is None:
            cu_k = cu_q
    else:
        B, Tq, Hq, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        total_q, total_k = B * Tq, B * Tk
        # token rows of a [B,T,H,D] tensor must be equally spaced across the batch boundary
        for t in (q, k, v):
            assert t.shape[0] == 1 or t.stride(0) == t.shape[1] * t.stride(1), "batch dim must be dense over tokens"
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.stride(-2) == D
    ldq, ldk, ldv = q.stride(-3), k.stride(-3), v.stride(-3)
    if out is None:
        out = torch.empty((*q.shape[:-2], Hq, D), dtype=q.dtype, device=q.device)
    ldo = out.stride(-3)
    lse = torch.empty((Hq, total_q), dtype=torch.float32, device=q.device) if want_lse else None
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    _lib.call("edl_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _lib.ptr(lse), ldq, ldk, ldv,
              ldo, _lib.ptr(cu_q), _lib.ptr(cu_k), B, Tq, Tk, total_q, total_k, Hq, Hkv, D, float(scale),
              int(causal), int(window or 0), float(softcap or 0.0), _lib.ptr(sinks),
              _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    return out, lse


def attn_bwd(q, k, v, o, lse, do, *, causal=True, scale=None, window=0, softcap=0.0, cu_q=None, cu_k=None,
             max_q=None, max_k=None, dq=None, dk=None, dv=None, want_delta=False):
    """Gradients of :func:`attn_fwd`. Returns (dq, dk, dv) in the layouts of q, k, v (and ``delta = rowsum(o * do)``,
    ``[Hq, total_q]`` fp32, when ``want_delta``)."""
    varlen = cu_q is not None
    if varlen:
        total_q, Hq, D = q.shape
        total_k, Hkv = k.shape[0], k.shape[1]
        B = cu_q.numel() - 1
        Tq, Tk = int(max_q), int(max_k)
        if cu_k is None:
            cu_k = cu_q
    else:
        B, Tq, Hq, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        total_q, total_k = B * Tq, B * Tk
    if not do.is_contiguous():
        do = do.contiguous()
    if not o.is_contiguous():
        o = o.contiguous()
    dq = torch.empty((*q.shape[:-2], Hq, D), dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty((*k.shape[:-2], Hkv, D), dtype=k.dtype, device=k.device) if dk is None else dk
    dv = torch.empty((*v.shape[:-2], Hkv, D), dtype=v.dtype, device=v.device) if dv is None else dv
    delta = torch.empty((Hq, total_q), dtype=torch.float32, device=q.device)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    _lib.call("edl_attn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
              delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), q.stride(-3), k.stride(-3),
              v.stride(-3), o.stride(-3), do.stride(-3), dq.stride(-3), dk.stride(-3), dv.stride(-3), _lib.ptr(cu_q),
              _lib.ptr(cu_k), B, Tq, Tk, total_q, total_k, Hq, Hkv, D, float(scale), int(causal), int(window or 0),
              float(softcap or 0.0), _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    if want_delta:
        return dq, dk, dv, delta
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, window, softcap, sinks, cu, max_len):
        from . import remat

        hit, kept = remat.saved_output("attn_core", "attn")   # recompute of a unit that kept the kernel's result
        if hit:
            o, lse = kept
        else:
            o, lse = attn_fwd(q, k, v, causal=causal, scale=scale, window=window, softcap=softcap, sinks=sinks,
                              cu_q=cu, cu_k=cu, max_q=max_len, max_k=max_len)
            remat.keep_output("attn_core", "attn", (o, lse))
        ctx.save_for_backward(q, k, v, o, lse, cu, sinks)
        ctx.args = (causal, scale, window, softcap, max_len)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu, sinks = ctx.saved_tensors
        causal, scale, window, softcap, max_len = ctx.args
        # With sinks the forward's log-sum-exp already counts the sink logit, so P = exp(S - lse) recomputed by the
        # backward kernels is the true probability and dq / dk / dv need nothing else. The sink itself has a zero
        # value row, hence dP_sink = 0 and d sink[h] = sum_rows P_sink * (0 - delta) = -sum exp(sink - lse) * delta.
        bufs = {}
        if q.dim() == 4 and k.shape[:2] == q.shape[:2] and k.dtype == q.dtype and v.dtype == q.dtype:
            # the three gradients as slices of one packed buffer: a packed projection's backward takes it as it is
            from .functional import packed_qkv_buffers

            _, bufs["dq"], bufs["dk"], bufs["dv"] = packed_qkv_buffers(q.shape[0], q.shape[1], q.shape[2], k.shape[2],
                                                                       q.shape[3], q.dtype, q.device)
        dq, dk, dv, delta = attn_bwd(q, k, v, o, lse, do, causal=causal, scale=scale, window=window, softcap=softcap,
                                     cu_q=cu, cu_k=cu, max_q=max_len, max_k=max_len, want_delta=True, **bufs)
        dsinks = None
        if sinks is not None and ctx.needs_input_grad[7]:
            dsinks = -(torch.exp(sinks.float()[:, None] - lse) * delta).sum(1).to(sinks.dtype)
        return dq, dk, dv, None, None, None, None, dsinks, None, None


def segment_ids_to_cu_seqlens(segment_ids: torch.Tensor):
    """Turns per-token segment ids ``[B,T]`` (0 = padding, contiguous segments) into varlen metadata.

    Returns (cu_seqlens int32 [n+1] over the flattened ``B*T`` token axis, max_len). Padding runs
    become their own sequences, so their rows are computed but isolated from real tokens.
    """
    B, T = segment_ids.shape
    flat = segment_ids.reshape(-1)
    change = torch.ones(B * T, dtype=torch.bool, device=flat.device)
    change[1:] = flat[1:] != flat[:-1]
    change[::T] = True  # a new row of the batch always starts a sequence
    starts = change.nonzero().reshape(-1).to(torch.int32)
    cu = torch.cat([starts, torch.tensor([B * T], dtype=torch.int32, device=flat.device)])
    max_len = int((cu[1:] - cu[:-1]).max().item())
    return cu, max_len


def flash_attention(q, k, v, *, causal=True, scale=None, segment_ids=None, sliding_window=None, softcap=0.0,
                    sinks=None, cu_seqlens=None, max_seqlen=None):
    """Differentiable attention. ``[B,T,H,D]`` inputs; ``segment_ids`` or ``cu_seqlens`` select packed-document masking."""
    if segment_ids is not None and cu_seqlens is None:
        cu_seqlens, max_seqlen = segment_ids_to_cu_seqlens(segment_ids)
    if cu_seqlens is not None:
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())
        shape = q.shape
        q3 = q.reshape(-1, q.shape[-2], q.shape[-1]) if q.dim() == 4 else q
        k3 = k.reshape(-1, k.shape[-2], k.shape[-1]) if k.dim() == 4 else k
        v3 = v.reshape(-1, v.shape[-2], v.shape[-1]) if v.dim() == 4 else v
        o = _FlashAttnFn.apply(q3, k3, v3, causal, scale, sliding_window or 0, softcap, sinks, cu_seqlens,
                               max_seqlen)
        return o.view(shape)
    return _FlashAttnFn.apply(q, k, v, causal, scale, sliding_window or 0, softcap, sinks, None, None)
