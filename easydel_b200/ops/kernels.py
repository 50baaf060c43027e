"""Raw (non-autograd) Python entry points of the sm_100a kernels.

Each function validates shapes, strides and alignment on the host before the
launch, allocates outputs with torch and calls the C launcher on the current
stream. Autograd wiring lives in :mod:`easydel_b200.ops.functional`.
"""

from __future__ import annotations

import torch

from . import _lib

ACT_IDS = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_new": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3}

GEMM_OUT_F32 = 1
GEMM_ACCUMULATE = 2
GEMM_BIAS = 4


def _check_bf16_2d(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D bf16 tensor with unit inner stride, got {t.dtype} {tuple(t.shape)} "
                         f"strides {t.stride()}")
    if t.data_ptr() % 16 or (t.stride(0) % 8 and t.shape[0] > 1):
        raise ValueError(f"{name}: base pointer / leading dimension must be 16-byte aligned")


_SPLITK_OFFSETS: dict[tuple, torch.Tensor] = {}
_SM_COUNT: dict[int, int] = {}


def _splitk_plan(M: int, N: int, K: int, device) -> int:
    """Number of K slices for a skinny GEMM (1 = use the plain kernel).

    Decode-time linears have a handful of rows and are bound by streaming the weight matrix; with one CTA per
    128-column tile a 4096-wide projection would occupy 32 of 148 SMs. Slicing K gives every SM a share.
    """
    if M > 256 or N % 8 or K % 64 or K < 512:
        return 1
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    sms = _SM_COUNT[idx]
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    if tiles * 4 >= sms * 3:
        return 1
    kb = K // 64
    want = min(16, max(2, (2 * sms + tiles - 1) // tiles))
    best = 1
    for s in range(2, want + 1):
        if kb % s == 0 and kb // s >= 2:
            best = s
    return best


def _pair_splitk_plan(M: int, N: int, K: int, device) -> int:
    """K slices for the CTA-pair split-K kernel (0 = use the other kernels).

    Measured on the decode shapes of a 70B model under 8-way tensor parallelism (256 rows; hidden 8192, FFN 3584 per
    GPU), the pair kernel does not beat the 128-wide kernel: with one slice too few CTAs stream (the weight bytes in
    flight per CTA are bounded by its six 32 KB stages), and every extra slice pays ~8 us for the fp32 partial sums
    that meet in L2. So nothing is planned by default; ``gemm(..., pair_splits=n)`` runs it explicitly and
    ``EDL_GEMM_PAIR_SPLITK=1`` enables the two-slice plan for products with fewer than half as many 256 x 256 tiles
    as CTA pairs.
    """
    if not _PAIR_SPLITK_ENV[0] or M <= 128 or M > 512 or N % 8 or K % 64 or N < 512:
        return 0
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    return 2 if 4 * tiles <= _SM_COUNT[idx] and K >= 2048 else 0


def _pair128_plan(M: int, N: int, K: int, device) -> bool:
    """Skinny products (a decode step's few hundred rows): the CTA-pair kernel with 256 x 128 tiles when it gives
    more streaming CTAs than the 128-wide single-CTA kernel has row-tile pairs to spare. Each CTA of a pair loads 16 KB
    of activations and 8 KB of weights per reduction block (24 KB against the single-CTA kernel's 32 KB), and what
    bounds these products is what one SM pulls through its L2 port."""
    if not _PAIR128_ENV[0] or M <= 128 or M > 512 or N % 8 or K % 64 or K < 1024:
        return False
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = _SM_COUNT[idx] // 2
    tiles = ((M + 255) // 256) * ((N + 127) // 128)
    return 0.6 * pairs <= tiles <= 4 * pairs


_PAIR128_ENV = [__import__("os").environ.get("EDL_GEMM_PAIR128", "0") not in ("", "0")]
_PAIR_SPLITK_ENV = [__import__("os").environ.get("EDL_GEMM_PAIR_SPLITK", "0") not in ("", "0")]


_PAIR_WS: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _pair_workspace(strips: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Zeroed fp32 strip accumulators and strip counters (the kernel leaves both zero), one set per (device,
    stream), grown on demand."""
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    cur = _PAIR_WS.get(key)
    if cur is None or cur[1].numel() < strips:
        n = max(strips, 512)
        cur = _PAIR_WS[key] = (torch.zeros(n * 8192, dtype=torch.float32, device=device),
                               torch.zeros(n, dtype=torch.int32, device=device))
    return cur


def _splitk_offsets(K: int, splits: int, device) -> torch.Tensor:
    key = (K, splits, device.index or 0)
    t = _SPLITK_OFFSETS.get(key)
    if t is None:
        step = K // splits
        t = torch.tensor([i * step for i in range(splits + 1)], dtype=torch.int32, device=device)
        _SPLITK_OFFSETS[key] = t
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, accumulate: bool = False, bias: torch.Tensor | None = None,
         max_ctas: int = 0, force_bn: int = 0, pair_splits: int = 0) -> torch.Tensor:
    """C[M,N] (+)= op(A) op(B) on tcgen05 tensor cores.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    Both are bf16 with unit inner stride; the outer stride may exceed the width.
    """
    _check_bf16_2d(a, "a")
    _check_bf16_2d(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: reduction sizes differ ({K} vs {Kb})")
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"gemm: bad output {tuple(out.shape)} {out.dtype} strides {out.stride()}")
    flags = 0
    if out.dtype == torch.float32:
        flags |= GEMM_OUT_F32
    if accumulate:
        flags |= GEMM_ACCUMULATE
    if bias is not None:
        if bias.dtype != torch.bfloat16 or bias.numel() != N or not bias.is_contiguous():
            raise ValueError("gemm: bias must be a contiguous bf16 vector of length N")
        flags |= GEMM_BIAS
    lda = a.stride(0) if a.shape[0] > 1 else a.shape[1]
    ldb = b.stride(0) if b.shape[0] > 1 else b.shape[1]
    ldc = out.stride(0) if out.shape[0] > 1 else out.shape[1]
    if not (a_mn or b_mn or accumulate or max_ctas) and out.dtype == torch.bfloat16 and force_bn in (0, 512):
        ps = pair_splits or (_pair_splitk_plan(M, N, K, a.device) if not force_bn else 0)
        if ps > 1 or (ps == 1 and pair_splits):
            # one 32-row strip per epilogue warp
            ws, counters = _pair_workspace(8 * ((M + 255) // 256) * ((N + 255) // 256), a.device)
            _lib.call("edl_gemm_pair_splitk", a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, lda,
                      ldb, ldc, ps, ws.data_ptr(), counters.data_ptr(), _lib.status_word(a.device).data_ptr(),
                      _lib.stream_ptr())
            return out
    if not (a_mn or b_mn or accumulate or max_ctas or force_bn) and out.dtype == torch.bfloat16 \
            and _pair128_plan(M, N, K, a.device):
        force_bn = 384
    if not (a_mn or b_mn or accumulate or max_ctas or force_bn) and out.dtype == torch.bfloat16:
        splits = _splitk_plan(M, N, K, a.device)
        if splits > 1:
            ws = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
            _lib.call("edl_gemm_splitk", a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, lda, ldb,
                      ldc, splits, ws.data_ptr(), _splitk_offsets(K, splits, a.device).data_ptr(),
                      _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
            return out
    _lib.call("edl_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, lda, ldb, ldc,
              int(a_mn), int(b_mn), flags, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr(), max_ctas,
              force_bn)
    return out


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                w_offset: float = 0.0, want_rstd: bool = True):
    """Returns (y, h, rstd): h = x + residual (or x itself), y = rmsnorm(h) * (w + w_offset)."""
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_rstd else None
    res2 = h = None
    if residual is not None:
        res2 = residual.reshape(-1, D)
        if not res2.is_contiguous():
            res2 = res2.contiguous()
        h = torch.empty_like(x2)
    _lib.call("edl_rmsnorm_fwd", x2.data_ptr(), _lib.ptr(res2), w.data_ptr(), y.data_ptr(), _lib.ptr(h),
              _lib.ptr(rstd), rows, D, float(eps), float(w_offset), _lib.stream_ptr())
    return y.view(x.shape), (h.view(x.shape) if h is not None else x), rstd


def rmsnorm_bwd(h: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None = None, w_offset: float = 0.0, dw_out: torch.Tensor | None = None,
                accumulate: bool = False):
    """Returns (dx, dw). dw is fp32; if ``dw_out`` is given it is written (or added to)."""
    D = h.shape[-1]
    h2 = h.reshape(-1, D)
    dy2 = dy.reshape(-1, D)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    rows = h2.shape[0]
    dx = torch.empty_like(h2)
    lib = _lib.get()
    nws = lib.edl_rmsnorm_bwd_workspace(rows, D)
    ws = torch.empty(nws, dtype=torch.float32, device=h.device)
    if dw_out is None:
        dw_out = torch.empty(D, dtype=torch.float32, device=h.device)
        accumulate = False
    dres2 = None
    if dres is not None:
        dres2 = dres.reshape(-1, D)
        if not dres2.is_contiguous():
            dres2 = dres2.contiguous()
    _lib.call("edl_rmsnorm_bwd", h2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), _lib.ptr(dres2),
              dx.data_ptr(), dw_out.data_ptr(), ws.data_ptr(), rows, D, float(w_offset), int(accumulate),
              _lib.stream_ptr())
    return dx.view(h.shape), dw_out


def gated_act_fwd(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """h = act(gu[..., :F]) * gu[..., F:] for a ``[..., 2F]`` bf16 tensor."""
    F2 = gu.shape[-1]
    F = F2 // 2
    gu2 = gu.reshape(-1, F2)
    assert gu2.stride(1) == 1
    T = gu2.shape[0]
    h = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    _lib.call("edl_gated_act_fwd", gu2.data_ptr(), h.data_ptr(), T, F, gu2.stride(0) if T > 1 else F2,
              ACT_IDS[act], _lib.stream_ptr())
    return h.view(*gu.shape[:-1], F)


def gated_act_bwd(gu: torch.Tensor, dh: torch.Tensor, act: str = "silu") -> torch.Tensor:
    F2 = gu.shape[-1]
    F = F2 // 2
    gu2 = gu.reshape(-1, F2)
    dh2 = dh.reshape(-1, F)
    if not dh2.is_contiguous():
        dh2 = dh2.contiguous()
    if not gu2.is_contiguous():
        gu2 = gu2.contiguous()
    T = gu2.shape[0]
    dgu = torch.empty_like(gu2)
    _lib.call("edl_gated_act_bwd", gu2.data_ptr(), dh2.data_ptr(), dgu.data_ptr(), T, F, F2, ACT_IDS[act],
              _lib.stream_ptr())
    return dgu.view(gu.shape)


def rope_(x: torch.Tensor, pos: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor, nheads: int, head_dim: int,
          col0: int = 0, rot_dim: int | None = None, interleaved: bool = False, backward: bool = False) -> torch.Tensor:
    """In-place rotary embedding on ``nheads`` heads starting at column ``col0`` of a ``[T, ld]`` bf16 matrix."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16
    assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    rot = rot_dim or head_dim
    assert cos.shape[-1] == rot // 2, (cos.shape, rot)
    if pos is not None:
        pos = pos.reshape(-1).to(torch.int32)
        assert pos.numel() == x.shape[0]
    _lib.call("edl_rope", x.data_ptr(), _lib.ptr(pos), cos.data_ptr(), sin.data_ptr(), x.shape[0], nheads, head_dim,
              rot, x.stride(0), col0, int(interleaved), int(backward), cos.shape[0], _lib.stream_ptr())
    return x


def rope_copy_supported(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nheads: int, head_dim: int, col0: int,
                        rot_dim: int | None) -> bool:
    """Whether :func:`rope_copy` takes this layout (full-width rotation, 16-byte aligned rows and tables)."""
    return (x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16 and (rot_dim or head_dim) == head_dim
            and head_dim % 16 == 0 and col0 % 8 == 0 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and cos.data_ptr() % 16 == 0 and sin.data_ptr() % 16 == 0
            and col0 + nheads * head_dim <= x.shape[1])


def rope_copy(x: torch.Tensor, out: torch.Tensor, pos: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor,
              nheads: int, head_dim: int, col0: int = 0, interleaved: bool = False,
              backward: bool = False) -> torch.Tensor:
    """Rotary embedding of ``nheads`` full heads from ``x`` into ``out`` (same shape; may be ``x`` itself) in one
    vectorised pass; columns outside the rotated heads are copied. Layout rules: :func:`rope_copy_supported`."""
    assert out.shape == x.shape and out.dtype == x.dtype and out.stride(1) == 1 and out.stride(0) % 8 == 0
    assert out.data_ptr() % 16 == 0
    assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    assert cos.shape[-1] == head_dim // 2, (cos.shape, head_dim)
    if pos is not None:
        pos = pos.reshape(-1).to(torch.int32)
        assert pos.numel() == x.shape[0]
    _lib.call("edl_rope_copy", x.data_ptr(), out.data_ptr(), _lib.ptr(pos), cos.data_ptr(), sin.data_ptr(),
              x.shape[0], nheads, head_dim, x.stride(0), out.stride(0), x.shape[1], col0, int(interleaved),
              int(backward), cos.shape[0], _lib.stream_ptr())
    return out


def embed_fwd(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    ids1 = ids.reshape(-1).to(torch.int64).contiguous()
    V, D = table.shape
    out = torch.empty((ids1.numel(), D), dtype=table.dtype, device=table.device)
    _lib.call("edl_embed_fwd", table.data_ptr(), ids1.data_ptr(), out.data_ptr(), ids1.numel(), D, V,
              _lib.stream_ptr())
    return out.view(*ids.shape, D)


def embed_bwd_(grad_table: torch.Tensor, dout: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """grad_table (fp32 [V,D]) += scatter(dout)."""
    assert grad_table.dtype == torch.float32 and grad_table.is_contiguous()
    ids1 = ids.reshape(-1).to(torch.int64).contiguous()
    V, D = grad_table.shape
    d2 = dout.reshape(-1, D)
    if not d2.is_contiguous():
        d2 = d2.contiguous()
    _lib.call("edl_embed_bwd", d2.data_ptr(), ids1.data_ptr(), grad_table.data_ptr(), ids1.numel(), D, V,
              _lib.stream_ptr())
    return grad_table


def cross_entropy_(logits: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100,
                   label_smoothing: float = 0.0, z_loss: float = 0.0, softcap: float = 0.0,
                   grad_scale: float = 1.0, grad_scale_tensor: torch.Tensor | None = None, write_grad: bool = True,
                   want_correct: bool = False):
    """Per-row CE over ``[rows, V]`` bf16 logits; overwrites them with the gradient when ``write_grad``.

    Returns (loss[rows] fp32, lse[rows] fp32, correct[rows] int32 or None).
    """
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    rows, V = logits.shape
    labels = labels.reshape(-1).to(torch.int64).contiguous()
    assert labels.numel() == rows
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    correct = torch.empty(rows, dtype=torch.int32, device=logits.device) if want_correct else None
    _lib.call("edl_cross_entropy", logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), lse.data_ptr(),
              _lib.ptr(correct), rows, V, logits.stride(0) if rows > 1 else V, ignore_index, float(label_smoothing),
              float(z_loss), float(softcap), _lib.ptr(grad_scale_tensor), float(grad_scale), int(write_grad),
              _lib.stream_ptr())
    return loss, lse, correct


def token_logprob(logits: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100, temperature: float = 1.0,
                  want_entropy: bool = False):
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    rows, V = logits.shape
    labels = labels.reshape(-1).to(torch.int64).contiguous()
    logp = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    ent = torch.empty(rows, dtype=torch.float32, device=logits.device) if want_entropy else None
    _lib.call("edl_token_logprob", logits.data_ptr(), labels.data_ptr(), logp.data_ptr(), lse.data_ptr(),
              _lib.ptr(ent), rows, V, logits.stride(0) if rows > 1 else V, ignore_index, 1.0 / temperature,
              _lib.stream_ptr())
    return logp, lse, ent


def token_logprob_bwd_(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, dlogp: torch.Tensor, *,
                       ignore_index: int = -100, temperature: float = 1.0) -> torch.Tensor:
    rows, V = logits.shape
    labels = labels.reshape(-1).to(torch.int64).contiguous()
    dlogp = dlogp.reshape(-1).to(torch.float32).contiguous()
    _lib.call("edl_token_logprob_bwd", logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), dlogp.data_ptr(), rows, V,
              logits.stride(0) if rows > 1 else V, ignore_index, 1.0 / temperature, _lib.stream_ptr())
    return logits


def adamw_(p32: torch.Tensor, p16: torch.Tensor | None, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, *,
           lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
           gscale: float = 1.0, gscale_tensor: torch.Tensor | None = None, skip_tensor: torch.Tensor | None = None,
           zero_grad: bool = False) -> None:
    """Fused AdamW over flat buffers (fp32 master/m/v, fp32 or bf16 grads, optional bf16 working copy)."""
    n = p32.numel()
    assert m.numel() == n and v.numel() == n and g.numel() == n
    assert p32.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
    assert g.dtype in (torch.float32, torch.bfloat16)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _lib.call("edl_adamw", p32.data_ptr(), _lib.ptr(p16), m.data_ptr(), v.data_ptr(), g.data_ptr(),
              int(g.dtype == torch.bfloat16), n, float(lr), float(beta1), float(beta2), float(eps),
              float(weight_decay), float(bc1), float(bc2), _lib.ptr(gscale_tensor), float(gscale),
              _lib.ptr(skip_tensor), int(zero_grad), _lib.stream_ptr())


def sumsq_(out: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """out[0] += sum(g*g) (fp32 accumulate)."""
    assert out.dtype == torch.float32
    _lib.call("edl_sumsq", g.data_ptr(), int(g.dtype == torch.bfloat16), g.numel(), out.data_ptr(), _lib.stream_ptr())
    return out


def clip_coef(sumsq: torch.Tensor, gscale: float, max_norm: float):
    """Returns (norm[1], coef[1], skip[1]) device tensors from an accumulated sum of squares."""
    dev = sumsq.device
    norm = torch.empty(1, dtype=torch.float32, device=dev)
    coef = torch.empty(1, dtype=torch.float32, device=dev)
    skip = torch.empty(1, dtype=torch.int32, device=dev)
    _lib.call("edl_clip_coef", sumsq.data_ptr(), float(gscale), float(max_norm or 0.0), norm.data_ptr(),
              coef.data_ptr(), skip.data_ptr(), _lib.stream_ptr())
    return norm, coef, skip
