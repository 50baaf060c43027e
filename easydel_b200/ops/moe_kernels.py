"""Expert FFN on the GPU: device-side routing tables, grouped tcgen05 GEMMs, fused combine.

Forward:  route (bucket pairs by expert, 128-row segments) -> gather -> grouped GEMM (gate|up) ->
gated activation -> grouped GEMM (down) -> weighted combine. Backward mirrors it with the grouped
data-gradient and per-expert weight-gradient GEMMs. Nothing synchronises with the host.
"""

from __future__ import annotations

import torch

from . import _lib, kernels as K

vp, i32, i64 = _lib.vp, _lib.i32, _lib.i64
_lib.register("edl_moe_route", i32, [vp, i64, i32, i32, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp])
_lib.register("edl_moe_gather", i32, [vp, vp, vp, vp, i32, i64, i64, vp])
_lib.register("edl_moe_combine", i32, [vp, vp, vp, vp, i64, i32, i32, i32, vp])
_lib.register("edl_moe_combine_bwd", i32, [vp, vp, vp, vp, vp, vp, i64, i32, i32, vp])
_lib.register("edl_moe_gather_bwd", i32, [vp, vp, vp, i64, i32, i32, vp])
_lib.register("edl_gemm_grouped", i32, [i32, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, i32, vp, vp])


class Routing:
    """Device-side routing tables for one MoE call."""

    def __init__(self, topk_idx: torch.Tensor, num_local_experts: int, expert_offset: int = 0):
        T, k = topk_idx.shape
        dev = topk_idx.device
        E = num_local_experts
        self.T, self.k, self.E = T, k, E
        self.max_rows = ((T * k + 127) // 128 + E) * 128
        self.max_tiles = self.max_rows // 128
        ints = torch.empty(3 * E + 1 + self.max_tiles + 2 + T * k + self.max_rows, dtype=torch.int32, device=dev)
        o = 0

        def take(n):
            nonlocal o
            v = ints[o:o + n]
            o += n
            return v

        self.counts, self.offsets, self.cursors = take(E), take(E + 1), take(E)
        self.tile_expert, self.meta = take(self.max_tiles), take(2)
        self.slot_pos, self.row_token = take(T * k), take(self.max_rows)
        idx = topk_idx.reshape(-1).to(torch.int64).contiguous()
        _lib.call("edl_moe_route", idx.data_ptr(), T, k, expert_offset, E, self.counts.data_ptr(),
                  self.offsets.data_ptr(), self.cursors.data_ptr(), self.tile_expert.data_ptr(), self.max_tiles,
                  self.meta.data_ptr(), self.slot_pos.data_ptr(), self.row_token.data_ptr(), _lib.stream_ptr())

    def gather(self, x: torch.Tensor) -> torch.Tensor:
        H = x.shape[1]
        xs = torch.empty(self.max_rows, H, dtype=x.dtype, device=x.device)
        _lib.call("edl_moe_gather", x.data_ptr(), self.row_token.data_ptr(), self.meta.data_ptr(), xs.data_ptr(), H,
                  x.stride(0), self.max_rows, _lib.stream_ptr())
        return xs

    def grouped(self, kind: int, x, w, out, dy=None, N: int = 0, Kd: int = 0, accumulate: bool = False):
        _lib.call("edl_gemm_grouped", kind, _lib.ptr(x), w.data_ptr() if kind != 2 else None, out.data_ptr(),
                  _lib.ptr(dy), self.max_rows, N, Kd, self.E, self.tile_expert.data_ptr(), self.meta.data_ptr(),
                  self.offsets.data_ptr(), 2 if accumulate else 0, _lib.status_word(out.device).data_ptr(),
                  _lib.stream_ptr())
        return out


def _grouped_fwd(r: Routing, xs: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    E, N, Kd = w.shape
    # rows past the last segment are never written: start from zeros so later passes read defined values
    out = torch.zeros(r.max_rows, N, dtype=xs.dtype, device=xs.device)
    return r.grouped(0, xs, w, out, N=N, Kd=Kd)


def _grouped_dgrad(r: Routing, dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    E, N, Kd = w.shape
    out = torch.zeros(r.max_rows, Kd, dtype=dy.dtype, device=dy.device)
    return r.grouped(1, dy, w, out, N=N, Kd=Kd)


def _grouped_wgrad(r: Routing, dy: torch.Tensor, xs: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
    N, Kd = dy.shape[1], xs.shape[1]
    _lib.call("edl_gemm_grouped", 2, xs.data_ptr(), None, out.data_ptr(), dy.data_ptr(), r.max_rows, N, Kd, r.E,
              r.tile_expert.data_ptr(), r.meta.data_ptr(), r.offsets.data_ptr(), 2 if accumulate else 0,
              _lib.status_word(out.device).data_ptr(), _lib.stream_ptr())


class _MoEFFN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gu, w_d, topk_w, topk_idx, act, expert_offset):
        T, H = x.shape
        k = topk_idx.shape[1]
        r = Routing(topk_idx, w_gu.shape[0], expert_offset)
        xs = r.gather(x)
        h = _grouped_fwd(r, xs, w_gu)
        a = K.gated_act_fwd(h, act)
        ys = _grouped_fwd(r, a, w_d)
        wf = topk_w.to(torch.float32).contiguous()
        y = torch.empty(T, H, dtype=x.dtype, device=x.device)
        _lib.call("edl_moe_combine", ys.data_ptr(), wf.data_ptr(), r.slot_pos.data_ptr(), y.data_ptr(), T, k, H, 0,
                  _lib.stream_ptr())
        ctx.save_for_backward(xs, h, ys, wf, w_gu, w_d)
        ctx.r, ctx.act, ctx.shape = r, act, (T, H, k)
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, h, ys, wf, w_gu, w_d = ctx.saved_tensors
        r, act = ctx.r, ctx.act
        T, H, k = ctx.shape
        dy = dy.contiguous()
        dys = torch.zeros_like(ys)
        dwr = torch.empty(T, k, dtype=torch.float32, device=dy.device)
        _lib.call("edl_moe_combine_bwd", dy.data_ptr(), ys.data_ptr(), wf.data_ptr(), r.slot_pos.data_ptr(),
                  dys.data_ptr(), dwr.data_ptr(), T, k, H, _lib.stream_ptr())
        a = K.gated_act_fwd(h, act)
        da = _grouped_dgrad(r, dys, w_d)
        g_wd = g_wgu = None
        for w, dyv, xin, name in ((w_d, dys, a, "d"), (None, None, None, None)):
            if w is None:
                break
            mg = getattr(w, "main_grad", None)
            if ctx.needs_input_grad[2]:
                if mg is not None:
                    _grouped_wgrad(r, dyv, xin, mg, True)
                    w.grad_added_to_main_grad = True
                else:
                    buf = torch.zeros(w.shape, dtype=torch.float32, device=dy.device)
                    _grouped_wgrad(r, dyv, xin, buf, False)
                    g_wd = buf.to(w.dtype)
        dh = K.gated_act_bwd(h, da, act)
        if ctx.needs_input_grad[1]:
            mg = getattr(w_gu, "main_grad", None)
            if mg is not None:
                _grouped_wgrad(r, dh, xs, mg, True)
                w_gu.grad_added_to_main_grad = True
            else:
                buf = torch.zeros(w_gu.shape, dtype=torch.float32, device=dy.device)
                _grouped_wgrad(r, dh, xs, buf, False)
                g_wgu = buf.to(w_gu.dtype)
        dx = None
        if ctx.needs_input_grad[0]:
            dxs = _grouped_dgrad(r, dh, w_gu)
            dx = torch.empty(T, H, dtype=dy.dtype, device=dy.device)
            _lib.call("edl_moe_gather_bwd", dxs.data_ptr(), r.slot_pos.data_ptr(), dx.data_ptr(), T, k, H,
                      _lib.stream_ptr())
        return dx, g_wgu, g_wd, dwr.to(wf.dtype) if ctx.needs_input_grad[3] else None, None, None, None


def moe_ffn(x, w_gate_up, w_down, topk_w, topk_idx, act: str = "silu", expert_offset: int = 0):
    if act not in K.ACT_IDS:
        raise ValueError(f"activation {act!r} has no fused gated kernel")
    if not x.is_contiguous():
        x = x.contiguous()
    return _MoEFFN.apply(x, w_gate_up, w_down, topk_w, topk_idx, act, expert_offset)


class _GatherFn(torch.autograd.Function):
    """Rows of ``x`` copied into the expert-sorted, 128-row-padded layout of a :class:`Routing`."""

    @staticmethod
    def forward(ctx, x, r):
        ctx.r, ctx.shape = r, x.shape
        return r.gather(x.contiguous())

    @staticmethod
    def backward(ctx, dxs):
        r = ctx.r
        T, H = ctx.shape
        dxs = dxs.contiguous()
        dx = torch.empty(T, H, dtype=dxs.dtype, device=dxs.device)
        _lib.call("edl_moe_gather_bwd", dxs.data_ptr(), r.slot_pos.data_ptr(), dx.data_ptr(), T, r.k, H,
                  _lib.stream_ptr())
        return dx, None


class _GroupedLinearFn(torch.autograd.Function):
    """``ys = xs @ w[expert of row].T`` over the padded layout, with data and weight gradients."""

    @staticmethod
    def forward(ctx, xs, w, r):
        ctx.r = r
        ctx.save_for_backward(xs, w)
        return _grouped_fwd(r, xs, w)

    @staticmethod
    def backward(ctx, dy):
        xs, w = ctx.saved_tensors
        r = ctx.r
        dy = dy.contiguous()
        dxs = _grouped_dgrad(r, dy, w) if ctx.needs_input_grad[0] else None
        gw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                _grouped_wgrad(r, dy, xs, mg, True)
                w.grad_added_to_main_grad = True
            else:
                buf = torch.zeros(w.shape, dtype=torch.float32, device=dy.device)
                _grouped_wgrad(r, dy, xs, buf, False)
                gw = buf.to(w.dtype)
        return dxs, gw, None


def moe_ffn_composed(x, w_gate_up, w_down, topk_w, topk_idx, act, b_gate_up=None, b_down=None,
                     expert_offset: int = 0):
    """Expert FFN with per-expert biases and / or a gated activation outside the fused set: the two grouped GEMMs
    run on the tensor cores, the bias adds, the activation and the weighted combine are elementwise torch ops."""
    from . import functional as F

    T, H = x.shape
    k = topk_idx.shape[1]
    E = w_gate_up.shape[0]
    r = Routing(topk_idx, E, expert_offset)
    xs = _GatherFn.apply(x, r)
    # expert of every padded row; tiles past the used range hold arbitrary ids and are never read back
    row_e = r.tile_expert.long().clamp(0, E - 1).repeat_interleave(128)
    h = _GroupedLinearFn.apply(xs, w_gate_up, r)
    if b_gate_up is not None:
        h = h + b_gate_up[row_e]
    a = F.gated_act(h, act)
    ys = _GroupedLinearFn.apply(a.contiguous(), w_down, r)
    if b_down is not None:
        ys = ys + b_down[row_e]
    pos = r.slot_pos.long()
    valid = (pos >= 0).view(T, k)
    picked = ys[pos.clamp_min(0)].view(T, k, H).float()
    return (picked * (topk_w.float() * valid)[..., None]).sum(1).to(x.dtype)


def grouped_linear(x_sorted, w, group_sizes):
    """Grouped linear over rows already sorted by expert with explicit sizes (API parity with
    ``grouped_matmul(x, w, group_sizes)``): re-buckets through the routing tables."""
    E = w.shape[0]
    idx = torch.repeat_interleave(torch.arange(E, device=x_sorted.device), group_sizes.to(x_sorted.device))
    r = Routing(idx[:, None], E)
    xs = r.gather(x_sorted.contiguous())
    ys = _grouped_fwd(r, xs, w)
    return ys[r.slot_pos.long()]
