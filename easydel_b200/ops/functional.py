"""Differentiable ops. CUDA tensors run the sm_100a kernels, CPU tensors the reference math.

Each op is a ``torch.autograd.Function`` over the raw launchers in
:mod:`easydel_b200.ops.kernels`. Weight gradients of linear layers are
accumulated straight into ``weight.main_grad`` (an fp32 view of the flat
gradient buffer owned by the optimizer state) when that attribute exists, so a
micro-batch loop never materialises per-parameter bf16 gradients.
"""

from __future__ import annotations

import math

import torch

from . import _lib, kernels as K, reference as R, remat


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8) or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    return x2


# ---------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, name=None):
        x2 = _as_2d(x)
        hit, y = remat.saved_output(name, "dot")   # recompute of a unit that kept this product: no GEMM
        if not hit:
            y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=x.dtype, device=x.device)
            K.gemm(x2, w, bias=bias, out=y.view(-1, w.shape[0]))
            remat.keep_output(name, "dot", y)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.x_shape, dtype=dy.dtype, device=dy.device)
            K.gemm(dy2, w, b_mn=True, out=dx.view(-1, w.shape[1]))
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
                w.grad_added_to_main_grad = True
            else:
                dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           name: str | None = None) -> torch.Tensor:
    """y = x @ w.T + bias with ``w`` in torch Linear layout ``[out, in]``. ``name``: the activation-checkpoint
    name of this product (see :mod:`.remat`)."""
    if _lib.use_kernels(x):
        if x.dtype != torch.bfloat16:
            raise TypeError(f"GPU linear expects bf16 activations, got {x.dtype}")
        if (w.shape[0] % 8) or (w.shape[1] % 8):
            # rows of the operands / the output would not start on 16-byte boundaries (a 4-way router, a 3-class
            # head ...): a plain library product; such matrices are a few kilobytes
            return torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
        return _LinearFn.apply(x, w, bias, name)
    return R.linear(x, w, bias)


# ---------------------------------------------------------------------------- norms
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, eps, w_offset):
        y, h, rstd = K.rmsnorm_fwd(x, w, eps, residual=residual, w_offset=w_offset)
        ctx.save_for_backward(h, w, rstd)
        ctx.w_offset = w_offset
        ctx.has_res = residual is not None
        ctx.set_materialize_grads(False)
        if residual is not None:
            return y, h
        placeholder = x.new_empty(0)
        ctx.mark_non_differentiable(placeholder)
        return y, placeholder

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        mg = getattr(w, "main_grad", None)
        dres = dh if ctx.has_res else None
        if dy is None:
            dy = torch.zeros_like(h)
        dx, dw = K.rmsnorm_bwd(h, w, dy, rstd, dres=dres, w_offset=ctx.w_offset, dw_out=mg,
                               accumulate=mg is not None)
        dwr = None
        if mg is None:
            dwr = dw.to(w.dtype)
        return dx, dwr, (dx if ctx.has_res else None), None, None


def rms_norm(x, w, eps: float = 1e-6, w_offset: float = 0.0):
    if _lib.use_kernels(x):
        y, _ = _RMSNormFn.apply(x, w, None, eps, w_offset)
        return y
    return R.rms_norm(x, w, eps, w_offset)


def add_rms_norm(x, residual, w, eps: float = 1e-6, w_offset: float = 0.0):
    """Returns (rmsnorm(x + residual), x + residual) with the add fused into the norm kernel."""
    if _lib.use_kernels(x):
        return _RMSNormFn.apply(x, w, residual, eps, w_offset)
    h = x + residual
    return R.rms_norm(h, w, eps, w_offset), h


def layer_norm(x, w, b, eps: float = 1e-5):
    # LayerNorm models (GPT-2/NeoX/OPT/...) are not on a named hot path; torch's kernel serves both devices.
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), w, b, eps)


# ---------------------------------------------------------------------------- activations
class _GatedActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act):
        ctx.save_for_backward(gu)
        ctx.act = act
        return K.gated_act_fwd(gu, act)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        return K.gated_act_bwd(gu, dh, ctx.act), None


def gated_act(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(gu[..., :F]) * gu[..., F:]."""
    if _lib.use_kernels(gu) and act in K.ACT_IDS:
        return _GatedActFn.apply(gu if gu.stride(-1) == 1 else gu.contiguous(), act)
    return R.gated_act(gu, act)


# ---------------------------------------------------------------------------- rotary
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, cos, sin, nheads, head_dim, col0, rot_dim, interleaved):
        ctx.save_for_backward(pos, cos, sin)
        ctx.args = (nheads, head_dim, col0, rot_dim, interleaved)
        x2 = x.reshape(-1, x.shape[-1]) if x.is_contiguous() else None
        if x2 is not None and K.rope_copy_supported(x2, cos, sin, nheads, head_dim, col0, rot_dim):
            y = torch.empty_like(x, memory_format=torch.contiguous_format)   # one pass: rotate and copy the rest
            K.rope_copy(x2, y.view(-1, y.shape[-1]), pos, cos, sin, nheads, head_dim, col0=col0,
                        interleaved=interleaved)
            return y
        y = x.clone(memory_format=torch.contiguous_format)
        K.rope_(y.view(-1, y.shape[-1]), pos, cos, sin, nheads, head_dim, col0=col0, rot_dim=rot_dim,
                interleaved=interleaved)
        return y

    @staticmethod
    def backward(ctx, dx):
        pos, cos, sin = ctx.saved_tensors
        nheads, head_dim, col0, rot_dim, interleaved = ctx.args
        d2 = dx.reshape(-1, dx.shape[-1]) if dx.is_contiguous() else None
        if d2 is not None and K.rope_copy_supported(d2, cos, sin, nheads, head_dim, col0, rot_dim):
            out = torch.empty_like(dx, memory_format=torch.contiguous_format)
            K.rope_copy(d2, out.view(-1, out.shape[-1]), pos, cos, sin, nheads, head_dim, col0=col0,
                        interleaved=interleaved, backward=True)
            return out, None, None, None, None, None, None, None, None
        dx = dx.contiguous() if not dx.is_contiguous() else dx.clone()
        K.rope_(dx.view(-1, dx.shape[-1]), pos, cos, sin, nheads, head_dim, col0=col0, rot_dim=rot_dim,
                interleaved=interleaved, backward=True)
        return dx, None, None, None, None, None, None, None, None


class _SplitQKVFn(torch.autograd.Function):
    """``[B, T, (Hq + 2 Hkv) D]`` -> views ``q [B, T, Hq, D]``, ``k``, ``v [B, T, Hkv, D]``.

    Autograd's own backward of three slices fills three zero tensors of the packed size, copies a slice into each
    and adds them up (eight passes over the packed gradient). Here the three incoming gradients are either already
    the slices of one packed buffer (the attention backward allocates them that way: nothing is copied) or are
    concatenated in one pass."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, D):
        ctx.dims = (Hq, Hkv, D, qkv.shape, qkv.dtype, qkv.device)
        ctx.set_materialize_grads(False)
        B, T, _ = qkv.shape
        q = qkv[..., : Hq * D].view(B, T, Hq, D)
        k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
        v = qkv[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        Hq, Hkv, D, shape, dtype, device = ctx.dims
        B, T, W = shape
        if dq is not None and dk is not None and dv is not None:
            packed = packed_qkv_base(dq, dk, dv, B, T, Hq, Hkv, D)
            if packed is not None:
                return packed, None, None, None
        parts = []
        for g, H in ((dq, Hq), (dk, Hkv), (dv, Hkv)):
            parts.append(torch.zeros(B, T, H * D, dtype=dtype, device=device) if g is None
                         else g.reshape(B, T, H * D).to(dtype))
        return torch.cat(parts, dim=-1), None, None, None


def packed_qkv_buffers(B: int, T: int, Hq: int, Hkv: int, D: int, dtype, device):
    """One ``[B, T, (Hq + 2 Hkv) D]`` buffer and its three head-shaped views (see :class:`_SplitQKVFn`)."""
    base = torch.empty(B, T, (Hq + 2 * Hkv) * D, dtype=dtype, device=device)
    q = base[..., : Hq * D].view(B, T, Hq, D)
    k = base[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v = base[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
    return base, q, k, v


def packed_qkv_base(q, k, v, B, T, Hq, Hkv, D):
    """The packed tensor whose slices ``q``, ``k``, ``v`` are, or None when they do not lie that way in memory."""
    W = (Hq + 2 * Hkv) * D
    want = (T * W, W, D, 1)
    try:
        same = (q.untyped_storage().data_ptr() == k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr())
    except Exception:
        return None
    if not same or q.dtype != k.dtype or q.dtype != v.dtype:
        return None
    o = q.storage_offset()
    if k.storage_offset() != o + Hq * D or v.storage_offset() != o + (Hq + Hkv) * D:
        return None
    for t, H in ((q, Hq), (k, Hkv), (v, Hkv)):
        if tuple(t.shape) != (B, T, H, D):
            return None
        if any(st != w for st, w, n in zip(t.stride(), want, t.shape) if n > 1):
            return None
    return q.as_strided((B, T, W), (T * W, W, 1), o)


def split_qkv(qkv: torch.Tensor, Hq: int, Hkv: int, D: int):
    """Head-shaped views of a packed projection output; differentiable without the zero-fill / add passes."""
    if qkv.dim() == 3 and qkv.is_contiguous() and torch.is_grad_enabled() and qkv.requires_grad:
        return _SplitQKVFn.apply(qkv, Hq, Hkv, D)
    B, T, _ = qkv.shape
    return (qkv[..., : Hq * D].view(B, T, Hq, D), qkv[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D),
            qkv[..., (Hq + Hkv) * D:].view(B, T, Hkv, D))


def rope_packed(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nheads: int,
                head_dim: int, col0: int = 0, rot_dim: int | None = None, interleaved: bool = False,
                inplace: bool = False):
    """Rotates the first ``nheads`` heads (starting at column ``col0``) of a packed ``[T, width]`` projection.

    Returns a new tensor and leaves the input untouched, except with ``inplace=True`` (inference: the projection's
    output has no other reader), where the rotation is done in the input's memory and no copy is made.
    """
    if _lib.use_kernels(qkv):
        if inplace and not (torch.is_grad_enabled() and qkv.requires_grad) and qkv.is_contiguous():
            q2 = qkv.view(-1, qkv.shape[-1])
            if K.rope_copy_supported(q2, cos, sin, nheads, head_dim, col0, rot_dim):
                K.rope_copy(q2, q2, pos.reshape(-1), cos, sin, nheads, head_dim, col0=col0, interleaved=interleaved)
            else:
                K.rope_(q2, pos.reshape(-1), cos, sin, nheads, head_dim, col0=col0, rot_dim=rot_dim,
                        interleaved=interleaved)
            return qkv
        return _RopeFn.apply(qkv, pos.reshape(-1), cos, sin, nheads, head_dim, col0, rot_dim, interleaved)
    T = qkv.reshape(-1, qkv.shape[-1]).shape[0]
    flat = qkv.reshape(T, -1)
    seg = flat[:, col0:col0 + nheads * head_dim].reshape(T, nheads, head_dim)
    rot = R.apply_rope(seg, pos.reshape(-1), cos, sin, rot_dim, interleaved).reshape(T, nheads * head_dim)
    out = torch.cat([flat[:, :col0], rot, flat[:, col0 + nheads * head_dim:]], dim=-1)
    return out.view(qkv.shape)


# ---------------------------------------------------------------------------- embedding
class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids):
        ctx.save_for_backward(ids)
        ctx.table = table
        return K.embed_fwd(table, ids)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            K.embed_bwd_(mg, dout, ids)
            table.grad_added_to_main_grad = True
            return None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        K.embed_bwd_(g, dout, ids)
        return g.to(table.dtype), None


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    if _lib.use_kernels(table) and table.dtype == torch.bfloat16:
        return _EmbedFn.apply(table, ids)
    return torch.nn.functional.embedding(ids, table)


# ---------------------------------------------------------------------------- LM head + cross entropy
class _LinearCEFn(torch.autograd.Function):
    """Chunked LM-head GEMM + cross-entropy that never holds more than one chunk of logits.

    The gradient of each chunk is produced in the same pass (the CE kernel overwrites the
    logits with d loss / d logits), then pushed through the two backward GEMMs, so the
    backward of this node only rescales by the incoming scalar gradient.
    """

    @staticmethod
    def forward(ctx, h, w, labels, bias, ignore_index, label_smoothing, z_loss, softcap, chunk, reduction_scale,
                want_acc, grad_enabled, loss_scale, count_group=None):
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        valid = (labels != ignore_index)
        n_valid = valid.sum().to(torch.float32)
        if count_group is not None:   # rows are sharded over this group: normalise by the group's token count
            import torch.distributed as dist

            dist.all_reduce(n_valid, group=count_group)
        # gscale tensor = 1/max(n_valid,1) * reduction_scale, consumed on-device by the CE kernel
        if reduction_scale is None:
            gs = (float(loss_scale) / n_valid.clamp_min(1.0)).reshape(1)
        else:
            gs = torch.full((1,), float(reduction_scale), dtype=torch.float32, device=dev)
        need_grad = grad_enabled and (h.requires_grad or w.requires_grad)
        losses = torch.empty(T, dtype=torch.float32, device=dev)
        correct = torch.empty(T, dtype=torch.int32, device=dev) if want_acc else None
        dh = torch.empty_like(h) if need_grad and h.requires_grad else None
        mg = getattr(w, "main_grad", None)
        dw = None
        if need_grad and w.requires_grad and mg is None:
            dw = torch.zeros(V, H, dtype=torch.float32, device=dev)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc = h[s:e]
            logits = K.gemm(hc, w, bias=bias)
            l, _, c = K.cross_entropy_(logits, labels[s:e], ignore_index=ignore_index,
                                       label_smoothing=label_smoothing, z_loss=z_loss, softcap=softcap,
                                       grad_scale_tensor=gs, write_grad=need_grad, want_correct=want_acc)
            losses[s:e] = l
            if want_acc:
                correct[s:e] = c
            if need_grad:
                if dh is not None:
                    K.gemm(logits, w, b_mn=True, out=dh[s:e])
                if w.requires_grad:
                    K.gemm(logits, hc, a_mn=True, b_mn=True, out=mg if mg is not None else dw, accumulate=True)
        if mg is not None and need_grad and w.requires_grad:
            w.grad_added_to_main_grad = True
        loss = losses.sum() * gs[0]
        ctx.save_for_backward(dh, dw)
        ctx.w_dtype = w.dtype
        ctx.mark_non_differentiable(n_valid)
        acc = None
        if want_acc:
            acc = correct.sum().to(torch.float32) / n_valid.clamp_min(1.0)
            ctx.mark_non_differentiable(acc)
            return loss, n_valid, acc
        return loss, n_valid, torch.zeros((), device=dev)

    @staticmethod
    def backward(ctx, dloss, _dn, _dacc):
        dh, dw = ctx.saved_tensors
        gh = gw = None
        if dh is not None:
            gh = dh * dloss.to(dh.dtype)
        if dw is not None:
            gw = (dw * dloss).to(ctx.w_dtype)
        return gh, gw, None, None, None, None, None, None, None, None, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, *, bias=None,
                         ignore_index: int = -100, label_smoothing: float = 0.0, z_loss: float = 0.0,
                         softcap: float = 0.0, chunk_size: int = 2048, reduction_scale: float | None = None,
                         loss_scale: float = 1.0,
                         want_accuracy: bool = False, count_group=None):
    """Mean (over non-ignored labels) cross-entropy of ``h @ w.T`` without materialising the logits.

    ``h`` is ``[T, H]``, ``labels`` ``[T]`` (already shifted by the caller). Returns
    ``(loss, n_valid, accuracy)``. ``loss_scale`` multiplies the mean (gradient accumulation passes
    ``1 / steps`` here so that it is part of the gradients produced inside the op). With ``reduction_scale`` the sum of token losses is
    multiplied by that constant instead of ``1 / n_valid``.

    On the GPU with ``w.main_grad`` present the LM-head weight gradient is accumulated
    during this call, which is exact when the scalar gradient reaching ``loss`` is 1
    (the trainer folds 1/accumulation into ``reduction_scale``).
    """
    h2 = h.reshape(-1, h.shape[-1])
    lab = labels.reshape(-1)
    if _lib.use_kernels(h2):
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        return _LinearCEFn.apply(h2, w, lab, bias, ignore_index, label_smoothing, z_loss, softcap, chunk_size,
                                 reduction_scale, want_accuracy, torch.is_grad_enabled(), loss_scale, count_group)
    total = h2.new_zeros((), dtype=torch.float32)
    correct = h2.new_zeros((), dtype=torch.float32)
    for s in range(0, h2.shape[0], chunk_size):
        logits = R.linear(h2[s:s + chunk_size], w, bias)
        l, _ = R.cross_entropy(logits, lab[s:s + chunk_size], ignore_index=ignore_index,
                               label_smoothing=label_smoothing, z_loss=z_loss, softcap=softcap)
        total = total + l.sum()
        if want_accuracy:
            zc = logits.float()
            correct = correct + ((zc.argmax(-1) == lab[s:s + chunk_size]) & (lab[s:s + chunk_size] != ignore_index)
                                 ).sum()
    n_valid = (lab != ignore_index).sum().to(torch.float32)
    if count_group is not None:
        import torch.distributed as dist

        dist.all_reduce(n_valid, group=count_group)
    scale = (loss_scale / n_valid.clamp_min(1.0)) if reduction_scale is None else reduction_scale
    return total * scale, n_valid, correct / n_valid.clamp_min(1.0)


# ---------------------------------------------------------------------------- token log-probs (DPO / GRPO)
class _LinearLogprobFn(torch.autograd.Function):
    """log p(label) per token from hidden states and the LM head, chunked; backward recomputes each chunk."""

    @staticmethod
    def forward(ctx, h, w, labels, bias, ignore_index, temperature, chunk, want_entropy):
        T = h.shape[0]
        logp = torch.empty(T, dtype=torch.float32, device=h.device)
        lse = torch.empty(T, dtype=torch.float32, device=h.device)
        ent = torch.empty(T, dtype=torch.float32, device=h.device) if want_entropy else None
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            logits = K.gemm(h[s:e], w, bias=bias)
            lp, ls, en = K.token_logprob(logits, labels[s:e], ignore_index=ignore_index, temperature=temperature,
                                         want_entropy=want_entropy)
            logp[s:e] = lp
            lse[s:e] = ls
            if want_entropy:
                ent[s:e] = en
        ctx.save_for_backward(h, w, labels, lse, bias)
        ctx.args = (ignore_index, temperature, chunk)
        if want_entropy:
            ctx.mark_non_differentiable(ent)
            return logp, ent
        return logp, torch.zeros((), device=h.device)

    @staticmethod
    def backward(ctx, dlogp, _dent):
        h, w, labels, lse, bias = ctx.saved_tensors
        ignore_index, temperature, chunk = ctx.args
        T, H = h.shape
        dh = torch.empty_like(h) if ctx.needs_input_grad[0] else None
        mg = getattr(w, "main_grad", None)
        dw = None
        if ctx.needs_input_grad[1] and mg is None:
            dw = torch.zeros(w.shape, dtype=torch.float32, device=h.device)
        dlogp = dlogp.contiguous()
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            logits = K.gemm(h[s:e], w, bias=bias)
            K.token_logprob_bwd_(logits, labels[s:e], lse[s:e], dlogp[s:e], ignore_index=ignore_index,
                                 temperature=temperature)
            if dh is not None:
                K.gemm(logits, w, b_mn=True, out=dh[s:e])
            if ctx.needs_input_grad[1]:
                K.gemm(logits, h[s:e], a_mn=True, b_mn=True, out=mg if mg is not None else dw, accumulate=True)
        gw = None
        if dw is not None:
            gw = dw.to(w.dtype)
        elif mg is not None and ctx.needs_input_grad[1]:
            w.grad_added_to_main_grad = True
        return dh, gw, None, None, None, None, None, None


def linear_token_logprob(h, w, labels, *, bias=None, ignore_index: int = -100, temperature: float = 1.0,
                         chunk_size: int = 2048, want_entropy: bool = False):
    """Per-token ``log softmax(h @ w.T / temperature)[label]`` (0 where ignored); optional entropy."""
    shape = labels.shape
    h2 = h.reshape(-1, h.shape[-1])
    lab = labels.reshape(-1)
    if _lib.use_kernels(h2):
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        lp, ent = _LinearLogprobFn.apply(h2, w, lab, bias, ignore_index, temperature, chunk_size, want_entropy)
        return lp.view(shape), (ent.view(shape) if want_entropy else None)
    outs, ents = [], []
    for s in range(0, h2.shape[0], chunk_size):
        logits = R.linear(h2[s:s + chunk_size], w, bias)
        outs.append(R.token_logprob(logits, lab[s:s + chunk_size], ignore_index=ignore_index,
                                    temperature=temperature))
        if want_entropy:
            lpa = torch.log_softmax(logits.float() / temperature, -1)
            ents.append(-(lpa.exp() * lpa).sum(-1))
    return torch.cat(outs).view(shape), (torch.cat(ents).view(shape) if want_entropy else None)


# ---------------------------------------------------------------------------- attention
def _library_attention(q, k, v, causal, scale, segment_ids, sliding_window, softcap, sinks):
    """Shapes outside the flash kernels (head_dim above 128, value width different from the key width, fp32 / fp16
    inputs): the fused attention of the tensor library with an explicit mask; logit caps and sinks, which it has no
    slot for, use the dense fp32 form."""
    if (softcap and softcap > 0) or sinks is not None:
        return R.attention(q, k, v, causal=causal, scale=scale, segment_ids=segment_ids,
                           sliding_window=sliding_window, softcap=softcap, sinks=sinks)
    B, Tq, Hq, _ = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    mask, dead = None, None
    windowed = sliding_window is not None and sliding_window > 0
    if segment_ids is not None or windowed or (causal and Tq != Tk):
        qpos = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
        kpos = torch.arange(Tk, device=q.device)[None, :]
        m = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
        if causal:
            m &= kpos <= qpos
        if windowed:
            m &= kpos > qpos - sliding_window
        mask = m[None, None]
        if segment_ids is not None:
            seg = segment_ids
            mask = mask & (seg[:, None, :, None] == seg[:, None, None, :]) & (seg[:, None, None, :] != 0)
            dead = ~mask.any(-1, keepdim=True)              # padding queries: give them one key, zero the row after
            mask = mask | (dead & (kpos == 0)[None, None])
    if Hq != Hkv:
        k, v = k.repeat_interleave(Hq // Hkv, dim=2), v.repeat_interleave(Hq // Hkv, dim=2)
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
        is_causal=causal and mask is None, scale=scale).transpose(1, 2)
    if dead is not None:
        o = o.masked_fill(dead.transpose(1, 2), 0.0)
    return o


def attention(q, k, v, *, causal: bool = True, scale: float | None = None, segment_ids=None,
              sliding_window: int | None = None, softcap: float = 0.0, sinks=None, cu_seqlens=None):
    """Softmax attention. q ``[B,T,Hq,D]``, k/v ``[B,T,Hkv,D]`` -> ``[B,T,Hq,D]``.

    CUDA tensors run the tcgen05 flash kernels (imported lazily from :mod:`.attention`).
    """
    if _lib.use_kernels(q):
        from .attention import flash_attention

        D = q.shape[-1]
        if q.dtype == k.dtype == v.dtype == torch.bfloat16 and v.shape[-1] == D and D <= 128:
            if D not in (64, 128):
                # zero columns change neither the scores nor the kept output columns
                pad = (64 if D < 64 else 128) - D
                scale = scale if scale is not None else 1.0 / math.sqrt(D)
                q, k, v = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
                return flash_attention(q, k, v, causal=causal, scale=scale, segment_ids=segment_ids,
                                       sliding_window=sliding_window, softcap=softcap, sinks=sinks,
                                       cu_seqlens=cu_seqlens)[..., :D]
            return flash_attention(q, k, v, causal=causal, scale=scale, segment_ids=segment_ids,
                                   sliding_window=sliding_window, softcap=softcap, sinks=sinks,
                                   cu_seqlens=cu_seqlens)
        return _library_attention(q, k, v, causal, scale, segment_ids, sliding_window, softcap, sinks)
    return R.attention(q, k, v, causal=causal, scale=scale, segment_ids=segment_ids, sliding_window=sliding_window,
                       softcap=softcap, sinks=sinks)


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
