"""State-space and linear-attention recurrences: Mamba-1 selective scan, Mamba-2 SSD, gated delta rule, KDA and
the ragged causal conv1d in front of them (``csrc/ssm.cu``).

Every op has a PyTorch reference (also its autograd path: training differentiates the reference, chunk by chunk,
while inference and evaluation call the CUDA recurrences). Sequences are packed on the token axis with
``cu_seqlens``; ``state`` tensors are fp32 and updated in place.
"""

from __future__ import annotations

import torch
import torch.nn.functional as tF

from . import _lib

vp, i32, f32 = _lib.vp, _lib.i32, _lib.f32
_lib.register("edl_selective_scan", i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, vp, vp, vp])
_lib.register("edl_ssd_scan", i32, [vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, vp])
_lib.register("edl_delta_rule", i32, [vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, vp, vp, vp])
_lib.register("edl_ragged_conv1d", i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp])
_lib.register("edl_wkv4", i32, [vp, vp, vp, vp, vp, i32, i32, vp, vp, vp])


def _cu(total: int, cu_seqlens, device):
    if cu_seqlens is None:
        return torch.tensor([0, total], dtype=torch.int32, device=device)
    return cu_seqlens.to(device=device, dtype=torch.int32)


def _use_kernel(*ts) -> bool:
    t = ts[0]
    return t.is_cuda and _lib.available() and not (torch.is_grad_enabled() and any(
        x is not None and x.requires_grad for x in ts))


# ----------------------------------------------------------------------------------------- Mamba-1
def selective_scan_reference(u, delta, A, B, C, D=None, z=None, dt_bias=None, softplus=True, cu_seqlens=None,
                             state=None):
    total, Dm = u.shape
    N = A.shape[1]
    cu = _cu(total, cu_seqlens, u.device).tolist()
    dt = delta.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    if softplus:
        dt = tF.softplus(dt)
    ys = []
    new_states = []
    for b in range(len(cu) - 1):
        h = state[b].float().clone() if state is not None else torch.zeros(Dm, N, device=u.device)
        for t in range(cu[b], cu[b + 1]):
            dA = torch.exp(dt[t][:, None] * A.float())
            h = dA * h + dt[t][:, None] * B[t].float()[None] * u[t].float()[:, None]
            y = (h * C[t].float()[None]).sum(-1)
            if D is not None:
                y = y + D.float() * u[t].float()
            if z is not None:
                y = y * tF.silu(z[t].float())
            ys.append(y)
        new_states.append(h)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([s.detach() for s in new_states]))
    return torch.stack(ys).to(u.dtype)


def _scan_chunk(a, b, h0):
    """h_t = a_t * h_{t-1} + b_t over the leading axis (``a``, ``b`` ``[Q, ...]``, ``h0`` ``[...]``) by recursive
    doubling: log2(Q) vectorised steps instead of Q sequential ones; every intermediate stays bounded because the
    decays ``a`` are in (0, 1]."""
    Q = a.shape[0]
    k = 1
    while k < Q:
        a_prev = torch.cat([torch.ones_like(a[:k]), a[:-k]], 0)
        b_prev = torch.cat([torch.zeros_like(b[:k]), b[:-k]], 0)
        b = a * b_prev + b
        a = a * a_prev
        k *= 2
    return a * h0[None] + b


def selective_scan_chunked(u, delta, A, B, C, D=None, z=None, dt_bias=None, softplus=True, cu_seqlens=None,
                           state=None, chunk: int = 256):
    """The recurrence of :func:`selective_scan_reference` evaluated chunk by chunk with a parallel scan inside each
    chunk; differentiable, and every chunk is recomputed in the backward pass (``torch.utils.checkpoint``) so that
    only the states at chunk boundaries are kept. This is what training runs: the sequential reference needs one
    small launch per token."""
    from torch.utils.checkpoint import checkpoint

    total, Dm = u.shape
    cu = _cu(total, cu_seqlens, u.device).tolist()
    Af = A.float()

    def run(u_c, d_c, B_c, C_c, z_c, h0):
        dt = d_c.float() + (dt_bias.float() if dt_bias is not None else 0.0)
        if softplus:
            dt = tF.softplus(dt)
        a = torch.exp(dt[:, :, None] * Af[None])                                     # [Q, D, N]
        b = (dt * u_c.float())[:, :, None] * B_c.float()[:, None, :]
        h = _scan_chunk(a, b, h0)
        y = (h * C_c.float()[:, None, :]).sum(-1)
        if D is not None:
            y = y + D.float()[None] * u_c.float()
        if z_c is not None:
            y = y * tF.silu(z_c.float())
        return y, h[-1]

    need_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad
                                                for t in (u, delta, A, B, C, D, z, dt_bias))
    ys, finals = [], []
    for bi in range(len(cu) - 1):
        h = state[bi].float().clone() if state is not None else torch.zeros(Dm, A.shape[1], device=u.device)
        for lo in range(cu[bi], cu[bi + 1], chunk):
            hi = min(lo + chunk, cu[bi + 1])
            args = (u[lo:hi], delta[lo:hi], B[lo:hi], C[lo:hi], None if z is None else z[lo:hi], h)
            y, h = checkpoint(run, *args, use_reentrant=False) if need_grad else run(*args)
            ys.append(y)
        finals.append(h)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([f.detach() for f in finals]))
    return torch.cat(ys).to(u.dtype) if ys else u.new_zeros(0, Dm)


def selective_scan(u, delta, A, B, C, D=None, z=None, dt_bias=None, softplus=True, cu_seqlens=None, state=None):
    """u, delta, z ``[total, D]``; A ``[D, N]`` (negative); B, C ``[total, N]``; state ``[nseq, D, N]`` fp32."""
    if _use_kernel(u, delta, A, B, C, D, z) and A.shape[1] in (8, 16, 32, 64) and u.dtype == torch.bfloat16:
        total, Dm = u.shape
        cu = _cu(total, cu_seqlens, u.device)
        y = torch.empty_like(u)
        c = lambda t: None if t is None else t.contiguous()  # noqa: E731
        _lib.call("edl_selective_scan", c(u).data_ptr(), c(delta).data_ptr(), A.float().contiguous().data_ptr(),
                  c(B).data_ptr(), c(C).data_ptr(), _lib.ptr(None if D is None else D.float().contiguous()),
                  _lib.ptr(c(z)), _lib.ptr(None if dt_bias is None else dt_bias.float().contiguous()), int(softplus),
                  cu.data_ptr(), cu.numel() - 1, Dm, A.shape[1], _lib.ptr(state), y.data_ptr(), _lib.stream_ptr())
        return y
    if u.shape[0] > 16:
        return selective_scan_chunked(u, delta, A, B, C, D, z, dt_bias, softplus, cu_seqlens, state)
    return selective_scan_reference(u, delta, A, B, C, D, z, dt_bias, softplus, cu_seqlens, state)


# ----------------------------------------------------------------------------------------- Mamba-2
def ssd_scan_reference(x, dt, A, B, C, D=None, dt_bias=None, softplus=True, cu_seqlens=None, state=None):
    total, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    cu = _cu(total, cu_seqlens, x.device).tolist()
    d = dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    if softplus:
        d = tF.softplus(d)
    rep = H // G
    ys, new_states = [], []
    for b in range(len(cu) - 1):
        s = state[b].float().clone() if state is not None else torch.zeros(H, P, N, device=x.device)
        for t in range(cu[b], cu[b + 1]):
            decay = torch.exp(d[t] * A.float())                                   # [H]
            Bt = B[t].float().repeat_interleave(rep, 0)                            # [H, N]
            Ct = C[t].float().repeat_interleave(rep, 0)
            s = decay[:, None, None] * s + (d[t][:, None] * x[t].float())[:, :, None] * Bt[:, None, :]
            y = (s * Ct[:, None, :]).sum(-1)
            if D is not None:
                y = y + D.float()[:, None] * x[t].float()
            ys.append(y)
        new_states.append(s)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([s.detach() for s in new_states]))
    return torch.stack(ys).to(x.dtype)


def ssd_scan_chunked(x, dt, A, B, C, D=None, dt_bias=None, softplus=True, cu_seqlens=None, state=None,
                     chunk: int = 64):
    """The recurrence of :func:`ssd_scan_reference` in its chunked matrix form (state-space duality): inside a chunk
    the output is a masked, decay-weighted ``(C B^T)`` product applied to the inputs, chunks hand a ``[H, P, N]``
    state to one another, and the state's contribution is one more product. Batched matrix products instead of one
    launch per token; differentiable."""
    total, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    cu = _cu(total, cu_seqlens, x.device).tolist()
    d = dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    if softplus:
        d = tF.softplus(d)
    Af = A.float()
    ys, finals = [], []
    for bi in range(len(cu) - 1):
        lo, hi = cu[bi], cu[bi + 1]
        T = hi - lo
        s_in = state[bi].float().clone() if state is not None else torch.zeros(H, P, N, device=x.device)
        if T == 0:
            finals.append(s_in)
            continue
        pad = (-T) % chunk
        nc = (T + pad) // chunk

        def chunks(t, fill=0.0):
            t = t[lo:hi].float()
            if pad:
                t = torch.cat([t, t.new_full((pad, *t.shape[1:]), fill)], 0)
            return t.view(nc, chunk, *t.shape[1:])

        xc, dc = chunks(x), chunks(d)                               # [nc, Q, H, P], [nc, Q, H]  (padded steps: dt = 0)
        Bc = chunks(B).repeat_interleave(rep, 2)                    # [nc, Q, H, N]
        Cc = chunks(C).repeat_interleave(rep, 2)
        la = dc * Af[None, None]                                    # log decay per step, <= 0
        cs = la.cumsum(1)                                           # [nc, Q, H]
        # inside a chunk: y_t = sum_{s <= t} exp(cs_t - cs_s) (C_t . B_s) dt_s x_s
        seg = cs[:, :, None, :] - cs[:, None, :, :]                 # [nc, t, s, H]
        causal = torch.ones(chunk, chunk, dtype=torch.bool, device=x.device).tril()
        L = torch.exp(seg.masked_fill(~causal[None, :, :, None], float("-inf")))
        cb = torch.einsum("cthn,cshn->ctsh", Cc, Bc)
        xd = xc * dc[..., None]
        y = torch.einsum("ctsh,cshp->cthp", cb * L, xd)
        # what every chunk adds to the state, decayed to the chunk's end
        to_end = torch.exp(cs[:, -1:, :] - cs)                      # [nc, Q, H]
        add = torch.einsum("cshn,cshp->chpn", Bc * to_end[..., None], xd)
        total_decay = torch.exp(cs[:, -1, :])                       # [nc, H]
        states = []
        for c in range(nc):                                         # the only sequential part: one step per chunk
            states.append(s_in)
            s_in = total_decay[c][:, None, None] * s_in + add[c]
        st = torch.stack(states)                                    # state entering each chunk [nc, H, P, N]
        y = y + torch.einsum("cthn,chpn->cthp", Cc * torch.exp(cs)[..., None], st)
        y = y.reshape(nc * chunk, H, P)[:T]
        if D is not None:
            y = y + D.float()[None, :, None] * x[lo:hi].float()
        ys.append(y)
        finals.append(s_in)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([f.detach() for f in finals]))
    return torch.cat(ys).to(x.dtype) if ys else x.new_zeros(0, H, P)


def ssd_scan(x, dt, A, B, C, D=None, dt_bias=None, softplus=True, cu_seqlens=None, state=None):
    """x ``[total, H, P]``; dt ``[total, H]``; A ``[H]``; B, C ``[total, G, N]``; state ``[nseq, H, P, N]`` fp32."""
    if _use_kernel(x, dt, A, B, C, D) and B.shape[2] in (16, 32, 64, 128) and x.dtype == torch.bfloat16 \
            and x.shape[2] <= 256:
        total, H, P = x.shape
        cu = _cu(total, cu_seqlens, x.device)
        y = torch.empty_like(x)
        _lib.call("edl_ssd_scan", x.contiguous().data_ptr(), dt.contiguous().data_ptr(),
                  A.float().contiguous().data_ptr(), B.contiguous().data_ptr(), C.contiguous().data_ptr(),
                  _lib.ptr(None if D is None else D.float().contiguous()),
                  _lib.ptr(None if dt_bias is None else dt_bias.float().contiguous()), int(softplus), cu.data_ptr(),
                  cu.numel() - 1, H, P, B.shape[1], B.shape[2], _lib.ptr(state), y.data_ptr(), _lib.stream_ptr())
        return y
    if x.shape[0] > 16:
        return ssd_scan_chunked(x, dt, A, B, C, D, dt_bias, softplus, cu_seqlens, state)
    return ssd_scan_reference(x, dt, A, B, C, D, dt_bias, softplus, cu_seqlens, state)


# ----------------------------------------------------------------------------------------- delta rules
def delta_rule_reference(q, k, v, g=None, beta=None, scale=None, cu_seqlens=None, state=None):
    total, H, DK = q.shape
    DV = v.shape[-1]
    scale = scale if scale is not None else DK ** -0.5
    cu = _cu(total, cu_seqlens, q.device).tolist()
    outs, new_states = [], []
    for b in range(len(cu) - 1):
        S = state[b].float().clone() if state is not None else torch.zeros(H, DK, DV, device=q.device)
        for t in range(cu[b], cu[b + 1]):
            if g is not None:
                gt = torch.exp(g[t].float())
                S = S * (gt[:, :, None] if gt.dim() == 2 else gt[:, None, None])
            kt, qt, vt = k[t].float(), q[t].float(), v[t].float()
            r = vt - torch.einsum("hk,hkv->hv", kt, S)
            if beta is not None:
                r = r * beta[t].float()[:, None]
            S = S + kt[:, :, None] * r[:, None, :]
            outs.append(torch.einsum("hk,hkv->hv", qt, S) * scale)
        new_states.append(S)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([s.detach() for s in new_states]))
    return torch.stack(outs).to(q.dtype)


def delta_rule_chunked(q, k, v, g=None, beta=None, scale=None, cu_seqlens=None, state=None, chunk: int = 64):
    """The gated delta rule in chunk-parallel form: differentiable, matmul-bound (the training path).

    Inside a chunk with cumulative log-decay ``c_t`` the per-token updates ``u_t = beta_t (v_t - k_t^T e^{g_t} S_{t-1})``
    satisfy ``(I + A) U = beta * (V - e^{c} K S_0)`` with the strictly lower-triangular
    ``A[t,s] = beta_t e^{c_t - c_s} (k_t . k_s)``; one triangular solve per chunk replaces the token loop, then
    ``o_t = scale (e^{c_t} q_t^T S_0 + sum_{s<=t} e^{c_t - c_s} (q_t . k_s) u_s)`` and
    ``S_C = e^{c_C} S_0 + sum_s e^{c_C - c_s} k_s u_s^T``. Every exponent is <= 0. Scalar-per-head gates only.
    """
    total, H, DK = q.shape
    DV = v.shape[-1]
    scale = scale if scale is not None else DK ** -0.5
    cu = _cu(total, cu_seqlens, q.device).tolist()
    outs, new_states = [], []
    for b in range(len(cu) - 1):
        s0, s1 = cu[b], cu[b + 1]
        S = state[b].float() if state is not None else torch.zeros(H, DK, DV, device=q.device)
        for c0 in range(s0, s1, chunk):
            c1 = min(c0 + chunk, s1)
            n = c1 - c0
            qc, kc, vc = (t[c0:c1].float().transpose(0, 1) for t in (q, k, v))          # [H, n, D]
            bc = beta[c0:c1].float().t() if beta is not None else torch.ones(H, n, device=q.device)
            cum = torch.cumsum(g[c0:c1].float().t(), -1) if g is not None else torch.zeros(H, n, device=q.device)
            diff = cum[:, :, None] - cum[:, None, :]                                     # c_t - c_s
            tri = torch.ones(n, n, device=q.device, dtype=torch.bool).tril()
            decay = torch.where(tri, diff, torch.full_like(diff, -float("inf"))).exp()   # 0 above the diagonal
            kk = kc @ kc.transpose(1, 2)
            A = (bc[:, :, None] * decay * kk).tril(-1)
            rhs = bc[:, :, None] * (vc - cum.exp()[:, :, None] * (kc @ S))
            eye = torch.eye(n, device=q.device)
            U = torch.linalg.solve_triangular(eye + A, rhs, upper=False)
            o = cum.exp()[:, :, None] * (qc @ S) + (decay * (qc @ kc.transpose(1, 2))) @ U
            outs.append((o * scale).transpose(0, 1))
            tail = (cum[:, -1:] - cum).exp()                                             # e^{c_C - c_s}
            S = cum[:, -1].exp()[:, None, None] * S + (kc * tail[:, :, None]).transpose(1, 2) @ U
        new_states.append(S)
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([x.detach() for x in new_states]))
    if not outs:
        return q.new_zeros(0, H, DV)
    return torch.cat(outs).to(q.dtype)


def gated_delta_rule(q, k, v, g=None, beta=None, scale=None, cu_seqlens=None, state=None):
    """q, k ``[total, H, DK]``; v ``[total, H, DV]``; g ``[total, H]`` log-decay (or ``[total, H, DK]`` for KDA);
    beta ``[total, H]``; state ``[nseq, H, DK, DV]`` fp32. Returns ``[total, H, DV]``.

    Inference on the GPU runs the recurrent kernel; anything that needs gradients (or long CPU inputs) with a
    per-head gate goes through :func:`delta_rule_chunked`."""
    DK, DV = q.shape[-1], v.shape[-1]
    if _use_kernel(q, k, v, g, beta) and DK in (32, 64, 128) and DV <= 256 and q.dtype == torch.bfloat16:
        total, H, _ = q.shape
        cu = _cu(total, cu_seqlens, q.device)
        o = torch.empty(total, H, DV, dtype=q.dtype, device=q.device)
        per_channel = int(g is not None and g.dim() == 3)
        _lib.call("edl_delta_rule", q.contiguous().data_ptr(), k.contiguous().data_ptr(), v.contiguous().data_ptr(),
                  _lib.ptr(None if g is None else g.float().contiguous()),
                  _lib.ptr(None if beta is None else beta.to(torch.bfloat16).contiguous()), per_channel,
                  cu.data_ptr(), cu.numel() - 1, H, DK, DV, float(scale if scale is not None else DK ** -0.5),
                  _lib.ptr(state), o.data_ptr(), _lib.stream_ptr())
        return o
    if (g is None or g.dim() == 2) and q.shape[0] > 16:
        return delta_rule_chunked(q, k, v, g, beta, scale, cu_seqlens, state)
    return delta_rule_reference(q, k, v, g, beta, scale, cu_seqlens, state)


kda = gated_delta_rule   # kernel delta attention: the same recurrence with a per-channel gate ``g [total, H, DK]``


# ----------------------------------------------------------------------------------------- conv1d
def ragged_conv1d_reference(x, w, bias=None, cu_seqlens=None, activation: str | None = "silu", conv_state=None):
    total, Cn = x.shape
    W = w.shape[1]
    cu = _cu(total, cu_seqlens, x.device).tolist()
    outs = []
    for b in range(len(cu) - 1):
        seg = x[cu[b]:cu[b + 1]].float()
        left = conv_state[b].float() if conv_state is not None else torch.zeros(W - 1, Cn, device=x.device)
        padded = torch.cat([left, seg], 0)
        y = sum(padded[j:j + seg.shape[0]] * w[:, j].float()[None] for j in range(W))
        if bias is not None:
            y = y + bias.float()
        outs.append(tF.silu(y) if activation in ("silu", "swish") else y)
        if conv_state is not None and seg.shape[0]:
            with torch.no_grad():
                conv_state[b].copy_(padded[-(W - 1):].to(conv_state.dtype))
    return torch.cat(outs).to(x.dtype)


def ragged_conv1d(x, w, bias=None, cu_seqlens=None, activation: str | None = "silu", conv_state=None):
    """Depth-wise causal conv over packed sequences. x ``[total, C]``; w ``[C, W]``; conv_state ``[nseq, W-1, C]``
    holds the rows before each sequence and receives its last ``W-1`` rows."""
    if _use_kernel(x, w, bias) and x.dtype == torch.bfloat16:
        total, Cn = x.shape
        cu = _cu(total, cu_seqlens, x.device)
        lens = (cu[1:] - cu[:-1]).long()
        seq_of = torch.repeat_interleave(torch.arange(cu.numel() - 1, device=x.device, dtype=torch.int32), lens)
        y = torch.empty_like(x)
        xs = x.contiguous()
        _lib.call("edl_ragged_conv1d", xs.data_ptr(), w.to(torch.bfloat16).contiguous().data_ptr(),
                  _lib.ptr(None if bias is None else bias.to(torch.bfloat16).contiguous()), cu.data_ptr(),
                  seq_of.contiguous().data_ptr(), total, Cn, w.shape[1],
                  int(activation in ("silu", "swish")), _lib.ptr(conv_state), y.data_ptr(), _lib.stream_ptr())
        if conv_state is not None:
            W = w.shape[1]
            with torch.no_grad():     # roll the window: last W-1 rows of (old state ++ sequence)
                cul = cu.tolist()
                for b in range(len(cul) - 1):
                    seg = xs[cul[b]:cul[b + 1]]
                    if seg.shape[0]:
                        conv_state[b].copy_(torch.cat([conv_state[b], seg], 0)[-(W - 1):])
        return y
    return ragged_conv1d_reference(x, w, bias, cu_seqlens, activation, conv_state)


# ----------------------------------------------------------------------------------------- RWKV-4 WKV
def wkv4_reference(time_decay, time_first, k, v, cu_seqlens=None, state=None):
    total, Cn = k.shape
    cu = _cu(total, cu_seqlens, k.device).tolist()
    w = -torch.exp(time_decay.float())
    u = time_first.float()
    outs, new_states = [], []
    for b in range(len(cu) - 1):
        if state is not None:
            num, den, mx = state[b].float().clone().unbind(0)     # not views: the state is overwritten below
        else:
            num = torch.zeros(Cn, device=k.device)
            den = torch.zeros(Cn, device=k.device)
            mx = torch.full((Cn,), -1e38, device=k.device)
        for t in range(cu[b], cu[b + 1]):
            kt, vt = k[t].float(), v[t].float()
            m = torch.maximum(mx, kt + u)
            e1, e2 = torch.exp(mx - m), torch.exp(kt + u - m)
            outs.append((e1 * num + e2 * vt) / (e1 * den + e2))
            m = torch.maximum(mx + w, kt)
            e1, e2 = torch.exp(mx + w - m), torch.exp(kt - m)
            num, den, mx = e1 * num + e2 * vt, e1 * den + e2, m
        new_states.append(torch.stack([num, den, mx]))
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([s.detach() for s in new_states]))
    return torch.stack(outs).to(k.dtype) if outs else k.new_zeros(0, Cn)


def wkv4_chunked(time_decay, time_first, k, v, cu_seqlens=None, state=None, chunk: int = 32):
    """The recurrence of :func:`wkv4_reference` in a chunked matrix form: inside a chunk of ``Q`` tokens every output
    is a ratio of two sums over the earlier tokens with log-weights ``(t-1-s) w + k_s`` (a ``[Q, Q, C]`` tensor), the
    chunk's incoming state with ``mx + t w`` and the token itself with ``u + k_t``, all taken relative to their
    row maximum. The carried ``(num, den, mx)`` is the same triple the sequential form keeps (``mx`` is a maximum over
    the same set of exponents), so states interchange with the kernel's. Differentiable; chunks are recomputed in the
    backward pass."""
    from torch.utils.checkpoint import checkpoint

    total, Cn = k.shape
    cu = _cu(total, cu_seqlens, k.device).tolist()

    def run(td, tf_, k_c, v_c, num0, den0, mx0):
        w, u = -torch.exp(td.float()), tf_.float()
        kf, vf = k_c.float(), v_c.float()
        Q = kf.shape[0]
        t = torch.arange(Q + 1, device=kf.device, dtype=torch.float32)
        # rows 0..Q-1 give the outputs, row Q the state handed to the next chunk
        gap = (t[:, None] - 1 - t[None, :Q])                                       # [Q+1, Q]
        a_in = gap[:, :, None] * w[None, None] + kf[None]                          # [Q+1, Q, C]
        a_in = a_in.masked_fill((gap < 0)[:, :, None], -float("inf"))
        a_car = mx0[None] + t[:, None] * w[None]                                   # [Q+1, C]
        a_cur = u[None] + kf                                                       # [Q, C]
        m_past = torch.maximum(a_in.amax(1), a_car)                                # [Q+1, C]
        m_out = torch.maximum(m_past[:Q], a_cur)
        e_in, e_car, e_cur = torch.exp(a_in[:Q] - m_out[:, None]), torch.exp(a_car[:Q] - m_out), torch.exp(a_cur - m_out)
        top = e_car * num0[None] + (e_in * vf[None]).sum(1) + e_cur * vf
        bot = e_car * den0[None] + e_in.sum(1) + e_cur
        mx1 = m_past[Q]
        s_in, s_car = torch.exp(a_in[Q] - mx1[None]), torch.exp(a_car[Q] - mx1)
        return top / bot, s_car * num0 + (s_in * vf).sum(0), s_car * den0 + s_in.sum(0), mx1

    need_grad = torch.is_grad_enabled() and any(x.requires_grad for x in (time_decay, time_first, k, v))
    outs, finals = [], []
    for b in range(len(cu) - 1):
        if state is not None:
            num, den, mx = state[b].float().clone().unbind(0)     # not views: the state is overwritten below
        else:
            num, den = torch.zeros(Cn, device=k.device), torch.zeros(Cn, device=k.device)
            mx = torch.full((Cn,), -1e38, device=k.device)
        for lo in range(cu[b], cu[b + 1], chunk):
            hi = min(lo + chunk, cu[b + 1])
            args = (time_decay, time_first, k[lo:hi], v[lo:hi], num, den, mx)
            y, num, den, mx = checkpoint(run, *args, use_reentrant=False) if need_grad else run(*args)
            outs.append(y)
        finals.append(torch.stack([num, den, mx]))
    if state is not None:
        with torch.no_grad():
            state.copy_(torch.stack([f.detach() for f in finals]))
    return torch.cat(outs).to(k.dtype) if outs else k.new_zeros(0, Cn)


def wkv4(time_decay, time_first, k, v, cu_seqlens=None, state=None):
    """RWKV-4 time mixing. k, v ``[total, C]``; time_decay / time_first ``[C]``; state ``[nseq, 3, C]`` fp32
    (numerator, denominator, running max exponent), updated in place. Returns ``[total, C]``."""
    if _use_kernel(k, v, time_decay, time_first) and k.dtype == torch.bfloat16:
        total, Cn = k.shape
        cu = _cu(total, cu_seqlens, k.device)
        out = torch.empty_like(k)
        _lib.call("edl_wkv4", time_decay.float().contiguous().data_ptr(), time_first.float().contiguous().data_ptr(),
                  k.contiguous().data_ptr(), v.contiguous().data_ptr(), cu.data_ptr(), cu.numel() - 1, Cn,
                  _lib.ptr(state), out.data_ptr(), _lib.stream_ptr())
        return out
    if k.is_cuda and k.shape[0] > 16:      # launch-bound on a GPU; on the host the per-token loop does less arithmetic
        return wkv4_chunked(time_decay, time_first, k, v, cu_seqlens, state)
    return wkv4_reference(time_decay, time_first, k, v, cu_seqlens, state)
