"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

``edl_rmsnorm_bwd_noalloc`` serves callers that cannot allocate device memory when they call
into the library (all HBM already committed elsewhere, or a loop where cudaMalloc's possible
device synchronisation is not acceptable). Its scratch is a fixed array inside the library, so
this test checks (a) agreement with the regular entry point that takes a caller-provided
workspace, on two calls in a row with different data and shapes (the second call sees the first
call's leftovers in the shared scratch), (b) that no allocation through torch happens during the
call, and (c) that sizes beyond the built-in scratch are rejected with a clear message.

The file name sorts last so a run that stops at the first failure has already run everything else.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from easydel_b200.ops import _lib

    lib = C.CDLL(str(_lib.lib_path()))
    fn = lib.edl_rmsnorm_bwd_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                   C.c_int, C.c_float, C.c_int, C.c_void_p]
    err = lib.edl_last_error
    err.restype = C.c_char_p
    return fn, err


def _case(rows, D, seed, with_dres):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)  # noqa: E731
    x, dy = mk(rows, D), mk(rows, D)
    w = (mk(D) * 0.1 + 1).contiguous()
    dres = mk(rows, D) if with_dres else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, w, dy, rstd, dres


def test_noalloc_matches_regular_entry_point_twice():
    from easydel_b200.ops import kernels as K

    fn, err = _sym()
    stream = torch.cuda.current_stream().cuda_stream
    for rows, D, seed, with_dres in [(700, 4096, 1, True), (333, 2048 + 8, 2, False)]:
        x, w, dy, rstd, dres = _case(rows, D, seed, with_dres)
        dx_ref, dw_ref = K.rmsnorm_bwd(x, w, dy, rstd, dres=dres)
        dx = torch.empty_like(x)
        dw = torch.full((D,), 7.0, device="cuda", dtype=torch.float32)  # overwritten, not accumulated
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dres.data_ptr() if with_dres else None,
                dx.data_ptr(), dw.data_ptr(), rows, D, 0.0, 0, stream)
        after = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        assert rc == 0, err().decode()
        assert after == before, "the call allocated through the caching allocator"
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), dx_ref.float(), atol=3e-2, rtol=2e-2)
        assert torch.allclose(dw, dw_ref, atol=0.15, rtol=2e-2)
        # accumulate mode adds on top of what dw holds
        rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dres.data_ptr() if with_dres else None,
                dx.data_ptr(), dw.data_ptr(), rows, D, 0.0, 1, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert torch.allclose(dw, 2 * dw_ref, atol=0.3, rtol=2e-2)


def _torch_reference(x, w, dy, rstd, dres):
    """RMSNorm backward in plain fp32 PyTorch."""
    xf, wf, dyf = x.float(), w.float(), dy.float()
    xhat = xf * rstd[:, None]
    g = dyf * wf
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, (dyf * xhat).sum(0)


def test_noalloc_matches_fp32_reference_and_allows_aliasing():
    """Against fp32 PyTorch math, twice in a row; the second call writes dx over dy (the aliasing the header allows)."""
    fn, err = _sym()
    stream = torch.cuda.current_stream().cuda_stream
    for rows, D, seed, with_dres, alias in [(513, 4096, 11, False, False), (129, 1024, 12, True, True)]:
        x, w, dy, rstd, dres = _case(rows, D, seed, with_dres)
        dx_ref, dw_ref = _torch_reference(x, w, dy, rstd, dres)
        dx = dy.clone() if alias else torch.empty_like(x)
        dy_arg = dx if alias else dy
        dw = torch.empty(D, device="cuda", dtype=torch.float32)
        rc = fn(x.data_ptr(), w.data_ptr(), dy_arg.data_ptr(), rstd.data_ptr(),
                dres.data_ptr() if with_dres else None, dx.data_ptr(), dw.data_ptr(), rows, D, 0.0, 0, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), dx_ref, atol=3e-2, rtol=2e-2)
        assert torch.allclose(dw, dw_ref, atol=0.15, rtol=2e-2)


def test_noalloc_rejects_misaligned_pointers():
    fn, err = _sym()
    x, w, dy, rstd, _ = _case(4, 1024, 13, False)
    buf = torch.empty(4 * 1024 + 8, device="cuda", dtype=torch.bfloat16)
    dx_misaligned = buf[1:1 + 4 * 1024]          # 2 bytes past a 16-byte boundary
    rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), None, dx_misaligned.data_ptr(), None, 4, 1024,
            0.0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "16-byte aligned" in err().decode()


def test_noalloc_rejects_oversize_rows():
    fn, err = _sym()
    D = 8192 + 8
    x, w, dy, rstd, _ = _case(4, D, 3, False)
    dx = torch.empty_like(x)
    rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), None, 4, D, 0.0, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = err().decode()
    assert "8192" in msg and "edl_rmsnorm_bwd" in msg
