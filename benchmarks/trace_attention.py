"""Cycle trace of the flash-attention forward kernel: where one step of the key loop spends its clocks.

Needs a build of the library with the trace compiled in, loaded instead of the regular one:

    EDL_NVCC_EXTRA=-DEDL_ATTN_TRACE python -m easydel_b200.csrc.build --out /tmp/libedl_trace.so
    EDL_LIB_PATH=/tmp/libedl_trace.so python -m benchmarks.trace_attention

CTA 0 (the last 256-query block of the first head: 64 key tiles) stamps ``clock64`` at the phase boundaries of the
MMA-issuing lane and of one softmax thread per query tile. Printed: mean / min / max clocks per phase over the
steady-state steps, and one step's stamps relative to the top of the MMA loop. The stamps of the issuing lane mark
when an instruction group was *issued*; when a product finished is seen from the softmax thread that waits for it.
"""

from __future__ import annotations

import argparse
import ctypes

import numpy as np
import torch

from easydel_b200.ops import _lib
from easydel_b200.ops import attention as A


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--step", type=int, default=30, help="the step whose stamps are listed")
    a = ap.parse_args()
    T, Hq, Hkv, D = a.tokens, 32, 8, 128
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(1, T, Hq, D, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(1, T, Hkv, D, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(1, T, Hkv, D, device=dev, dtype=torch.bfloat16, generator=g)
    for _ in range(3):
        A.flash_attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    lib = _lib.get()
    if not hasattr(lib, "edl_attn_trace_read"):
        raise SystemExit("this library was built without -DEDL_ATTN_TRACE")
    buf = (ctypes.c_longlong * (4 * 64 * 8))()
    fn = lib.edl_attn_trace_read
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p]
    if fn(ctypes.cast(buf, ctypes.c_void_p)):
        raise SystemExit("reading the trace failed")
    t = np.array(list(buf), dtype=np.int64).reshape(4, 64, 8)
    steps = min(60, T // 128 - 4)

    def stats(name, arr):
        arr = arr[8:steps]
        print(f"  {name:44s} mean {arr.mean():7.0f}  min {arr.min():6d}  max {arr.max():6d}")

    for role, nm in ((0, "softmax, query tile A"), (1, "softmax, query tile B")):
        r = t[role]
        print(nm)
        stats("wait for S", r[:, 1] - r[:, 0])
        stats("load scores, mask, own maximum", r[:, 2] - r[:, 1])
        stats("exchange of maxima + rescale decision", r[:, 3] - r[:, 2])
        stats("exponentials, pack, store issued", r[:, 4] - r[:, 3])
        stats("wait for the stores", r[:, 5] - r[:, 4])
        stats("fence + arrive", r[:, 6] - r[:, 5])
        stats("busy (S seen -> P published)", r[:, 6] - r[:, 1])
        stats("whole step", r[1:, 0] - r[:-1, 0])
    r = t[2]
    print("MMA-issuing lane (issue times)")
    stats("wait for V and the next K", r[:, 1] - r[:, 0])
    stats("wait for P_A + issue PV_A", r[:, 2] - r[:, 1])
    stats("issue QK_A of the next tile", r[:, 3] - r[:, 2])
    stats("wait for P_B + issue PV_B", r[:, 4] - r[:, 3])
    stats("issue QK_B of the next tile + commits", r[:, 5] - r[:, 4])
    stats("whole step", r[1:, 0] - r[:-1, 0])
    n = a.step
    print(f"stamps of step {n} (and the next) relative to the top of the MMA loop")
    for role, nm in ((2, "mma"), (0, "softmax A"), (1, "softmax B")):
        cols = 6 if role == 2 else 7
        print(f"  {nm:10s}", [int(x - t[2, n, 0]) for x in t[role, n, :cols]],
              [int(x - t[2, n, 0]) for x in t[role, n + 1, :cols]])
    m = t[3]
    print("prologue (softmax warps idle): issue of the first QK_A", int(m[0, 1] - m[0, 0]), "clocks, of QK_B",
          int(m[0, 2] - m[0, 1]), "; S_A seen", int(t[0, 0, 1] - m[0, 0]), "after the first issue, S_B",
          int(t[1, 0, 1] - t[0, 0, 1]), "after S_A")


if __name__ == "__main__":
    main()
