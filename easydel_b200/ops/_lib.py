"""ctypes binding of the sm_100a kernel library (``lib/libedl_b200.so``).

The library exposes plain C launchers; tensors are passed as raw device
pointers, the stream as the current torch CUDA stream handle. A missing library
on a machine that has a GPU is an error (there is no silent PyTorch fallback for
CUDA tensors); on a CPU-only machine ``available()`` is simply False and the
callers use the fp32 reference math in :mod:`easydel_b200.ops.reference`.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

# EDL_LIB_PATH points at another build of the library (e.g. one compiled with bounds checks)
_LIB_PATH = Path(os.environ.get("EDL_LIB_PATH") or
                 Path(__file__).resolve().parent.parent / "lib" / "libedl_b200.so")
_lib = None
_lock = threading.Lock()
_status: dict[int, torch.Tensor] = {}

#: number of kernel-library launches issued by this process (for benchmarks)
launch_count = 0

vp, i32, i64, f32, u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong

_SIGS = {
    "edl_last_error": (C.c_char_p, []),
    "edl_sm_count": (i32, []),
    "edl_abi_version": (i32, []),
    "edl_gemm_bf16": (i32, [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, i32, vp, vp, i32, i32]),
    "edl_gemm_splitk": (i32, [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp, vp]),
    "edl_gemm_pair_splitk": (i32, [vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp, vp]),
    "edl_gemm_pair_splitk_workspace": (i64, [i32, i32]),
    "edl_rmsnorm_fwd": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32, f32, vp]),
    "edl_rmsnorm_bwd_workspace": (i64, [i32, i32]),
    "edl_rmsnorm_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, i32, vp]),
    "edl_gated_act_fwd": (i32, [vp, vp, i64, i32, i64, i32, vp]),
    "edl_gated_act_bwd": (i32, [vp, vp, vp, i64, i32, i64, i32, vp]),
    "edl_rope": (i32, [vp, vp, vp, vp, i64, i32, i32, i32, i64, i32, i32, i32, i32, vp]),
    "edl_rope_copy": (i32, [vp, vp, vp, vp, vp, i64, i32, i32, i64, i64, i32, i32, i32, i32, i32, vp]),
    "edl_embed_fwd": (i32, [vp, vp, vp, i64, i32, i32, vp]),
    "edl_embed_bwd": (i32, [vp, vp, vp, i64, i32, i32, vp]),
    "edl_cross_entropy": (i32, [vp, vp, vp, vp, vp, i32, i32, i64, i32, f32, f32, f32, vp, f32, i32, vp]),
    "edl_token_logprob": (i32, [vp, vp, vp, vp, vp, i32, i32, i64, i32, f32, vp]),
    "edl_token_logprob_bwd": (i32, [vp, vp, vp, vp, i32, i32, i64, i32, f32, vp]),
    "edl_adamw": (i32, [vp, vp, vp, vp, vp, i32, i64, f32, f32, f32, f32, f32, f32, f32, vp, f32, vp, i32, vp]),
    "edl_sumsq": (i32, [vp, i32, i64, vp, vp]),
    "edl_clip_coef": (i32, [vp, f32, f32, vp, vp, vp, vp]),
}


def lib_path() -> Path:
    return _LIB_PATH


def _load():
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            return None
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGS.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return _lib


def register(name: str, restype, argtypes) -> None:
    """Registers the signature of an exported launcher defined in another module."""
    _SIGS[name] = (restype, argtypes)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes


def available() -> bool:
    """True when CUDA tensors can be served by the kernel library."""
    return torch.cuda.is_available() and _load() is not None


def get():
    """Returns the loaded library or raises with build instructions."""
    lib = _load()
    if lib is None:
        raise RuntimeError(
            f"easydel_b200 kernel library not found at {_LIB_PATH}. Build it with "
            "`python -m easydel_b200.csrc.build` (needs nvcc, no GPU required). CUDA tensors are only "
            "served by these sm_100a kernels; there is no PyTorch fallback on the GPU."
        )
    return lib


def use_kernels(*tensors: torch.Tensor) -> bool:
    """Decides the code path for an op: kernels for CUDA tensors, reference math on CPU."""
    t = next((x for x in tensors if isinstance(x, torch.Tensor)), None)
    if t is None or not t.is_cuda:
        return False
    get()
    return True


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
    return t


_STATUS_TEXT = {
    1: "TMA producer wait ran out",
    2: "MMA issuer wait ran out",
    3: "epilogue wait ran out",
    4: "peer flag wait ran out",
    5: "softmax wait ran out",
    6: "index out of range",
}


def check_status(device=None) -> None:
    """Synchronising check of the kernel status word; raises if a kernel gave up."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"easydel_b200 kernel reported status {code}: {_STATUS_TEXT.get(code, 'unknown')}")


def call(name: str, *args) -> None:
    """Calls a launcher and raises with the library's message on failure."""
    global launch_count
    lib = get()
    rc = getattr(lib, name)(*args)
    launch_count += 1
    if rc != 0:
        msg = lib.edl_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed: {msg}")


def build_if_possible() -> bool:
    """Builds the library in-tree when nvcc is present. Returns availability of the file."""
    if _LIB_PATH.exists() and not os.environ.get("EDL_FORCE_BUILD"):
        return True
    try:
        from ..csrc.build import build

        build()
    except Exception:
        return _LIB_PATH.exists()
    return _LIB_PATH.exists()
