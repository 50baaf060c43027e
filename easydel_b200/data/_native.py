"""ctypes bindings of the host-side native helpers in ``csrc/host_native.cu`` (no GPU needed to call them)."""

from __future__ import annotations

import ctypes as C

import numpy as np

from ..ops import _lib as L

L.register("edl_host_pack_bfd", C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p])
L.register("edl_host_hash_pages", C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_uint64, C.c_uint64, C.c_void_p])
L.register("edl_host_fill_decode", None, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p])


def _lib():
    try:
        lib = L._load()
    except OSError:
        return None
    return lib if lib is not None and hasattr(lib, "edl_host_pack_bfd") else None


def available() -> bool:
    return _lib() is not None


def pack_bfd(lengths, capacity: int) -> list[list[int]]:
    """Best-fit-decreasing packing: list of bins, each a list of item indices (longest first)."""
    arr = np.ascontiguousarray(lengths, dtype=np.int32)
    out = np.empty(arr.shape[0], dtype=np.int32)
    n_bins = _lib().edl_host_pack_bfd(arr.ctypes.data, arr.shape[0], int(capacity), out.ctypes.data)
    bins: list[list[int]] = [[] for _ in range(n_bins)]
    for i in np.argsort(-arr, kind="stable"):
        bins[out[i]].append(int(i))
    return bins


def hash_pages(tokens, page_size: int, seed: int = 0, extra: int = 0) -> list[bytes]:
    arr = np.ascontiguousarray(tokens, dtype=np.int32)
    pages = arr.shape[0] // page_size
    out = np.empty(2 * pages, dtype=np.uint64)
    _lib().edl_host_hash_pages(arr.ctypes.data, arr.shape[0], int(page_size), C.c_uint64(seed & (2 ** 64 - 1)),
                               C.c_uint64(extra & (2 ** 64 - 1)), out.ctypes.data)
    raw = out.tobytes()
    return [raw[16 * i:16 * i + 16] for i in range(pages)]
