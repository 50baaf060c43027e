"""Bounded waits: a kernel that waits on a flag nothing sets gives up after its limit, reports a status code and
returns, and the context stays usable (the next launch succeeds).

Each case runs ONE kernel that believes it is rank 0 of two; the "peer" buffers are a second local allocation
that no kernel writes, so the peer's flag never arrives. Waits are a few milliseconds. No fault, trap or endless
loop is involved: the waiting loops themselves count clock cycles and leave.
"""

import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

EDL_TIMEOUT_PEER_FLAG = 4


def _take_status(dev):
    from easydel_b200.ops import _lib

    torch.cuda.synchronize(dev)
    w = _lib.status_word(dev)
    code = int(w.item())
    w.zero_()
    return code


def _context_still_works(dev):
    from easydel_b200.ops import kernels as K

    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    b = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    out = K.gemm(a, b)
    torch.cuda.synchronize(dev)
    assert torch.allclose(out.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    assert _take_status(dev) == 0


def test_oneshot_allreduce_gives_up_on_missing_peer():
    from easydel_b200.ops import _lib
    from easydel_b200.parallel import tp  # registers the entry points

    dev = torch.device("cuda", 0)
    n = 4096
    mine = torch.ones(n, device=dev, dtype=torch.bfloat16)
    peer = torch.ones(n, device=dev, dtype=torch.bfloat16)
    flags_mine = torch.zeros(64, device=dev, dtype=torch.int32)
    flags_peer = torch.zeros(64, device=dev, dtype=torch.int32)   # never written: "rank 1" does not exist
    sync = torch.zeros(2, device=dev, dtype=torch.int32)
    out = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    data_ptrs = (C.c_ulonglong * 2)(mine.data_ptr(), peer.data_ptr())
    flag_ptrs = (C.c_ulonglong * 2)(flags_mine.data_ptr(), flags_peer.data_ptr())
    assert _take_status(dev) == 0
    t0 = time.time()
    _lib.call("edl_allreduce_oneshot", C.cast(data_ptrs, C.c_void_p), C.cast(flag_ptrs, C.c_void_p), 2, 0,
              sync.data_ptr(), out.data_ptr(), None, n, 5, _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    code = _take_status(dev)          # synchronises: the kernel has returned
    assert time.time() - t0 < 5.0, "the wait was supposed to last milliseconds"
    assert code == EDL_TIMEOUT_PEER_FLAG
    _context_still_works(dev)
    del tp


def test_allreduce_add_rmsnorm_gives_up_on_missing_peer():
    from easydel_b200.ops import _lib
    from easydel_b200.parallel import tp  # noqa: F401  (registers the entry points)

    dev = torch.device("cuda", 0)
    rows, width = 8, 1024
    mine = torch.ones(rows * width, device=dev, dtype=torch.bfloat16)
    peer = torch.ones(rows * width, device=dev, dtype=torch.bfloat16)
    flags_mine = torch.zeros(64, device=dev, dtype=torch.int32)
    flags_peer = torch.zeros(64, device=dev, dtype=torch.int32)
    sync = torch.zeros(2, device=dev, dtype=torch.int32)
    res = torch.zeros(rows, width, device=dev, dtype=torch.bfloat16)
    w = torch.ones(width, device=dev, dtype=torch.bfloat16)
    x_out, h_out = torch.empty_like(res), torch.empty_like(res)
    data_ptrs = (C.c_ulonglong * 2)(mine.data_ptr(), peer.data_ptr())
    flag_ptrs = (C.c_ulonglong * 2)(flags_mine.data_ptr(), flags_peer.data_ptr())
    assert _take_status(dev) == 0
    _lib.call("edl_allreduce_add_rmsnorm", C.cast(data_ptrs, C.c_void_p), C.cast(flag_ptrs, C.c_void_p), 2, 0,
              sync.data_ptr(), res.data_ptr(), w.data_ptr(), 1e-5, 0.0, x_out.data_ptr(), h_out.data_ptr(), rows,
              width, 5, _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    assert _take_status(dev) == EDL_TIMEOUT_PEER_FLAG
    _context_still_works(dev)


def test_gemm_reduce_scatter_gives_up_on_missing_peer():
    """The fused GEMM -> reduce-scatter kernel as rank 0 of two: it finishes its own tiles, stores the peer's share
    into the (local) stand-in for the peer's staging area, then waits for the peer's release flag, which never
    comes."""
    from easydel_b200.ops import _lib
    from easydel_b200.parallel import fused  # noqa: F401  (registers the entry points)

    dev = torch.device("cuda", 0)
    rows, N, K = 128, 256, 128
    a = torch.randn(2 * rows, K, device=dev).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev).to(torch.bfloat16)
    stage = [torch.zeros(2 * rows * N, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(64, device=dev, dtype=torch.int32) for _ in range(2)]
    counters = torch.zeros(2 * (rows // 128) + 1, device=dev, dtype=torch.int32)   # arrivals per block + queue head
    out = torch.zeros(rows, N, device=dev, dtype=torch.bfloat16)
    stage_ptrs = (C.c_ulonglong * 2)(*[t.data_ptr() for t in stage])
    flag_ptrs = (C.c_ulonglong * 2)(*[t.data_ptr() for t in flags])
    assert _take_status(dev) == 0
    t0 = time.time()
    _lib.call("edl_gemm_reduce_scatter", a.data_ptr(), w.data_ptr(), out.data_ptr(), None, None, 2 * rows, N, K,
              a.stride(0), w.stride(0), C.cast(stage_ptrs, C.c_void_p), C.cast(flag_ptrs, C.c_void_p),
              counters.data_ptr(), 2, 0, 1, 5, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(), 0)
    code = _take_status(dev)
    assert time.time() - t0 < 5.0
    assert code == EDL_TIMEOUT_PEER_FLAG
    _context_still_works(dev)
