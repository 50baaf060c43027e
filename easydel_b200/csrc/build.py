"""Builds the sm_100a kernel library in-tree with nvcc.

Every ``*.cu`` file next to this script is compiled to an object file under
``csrc/build/`` and the objects are linked into ``easydel_b200/lib/libedl_b200.so``.
The library has a plain C ABI (``extern "C"`` launchers taking raw device pointers
and a stream handle) and is loaded with ``ctypes``; no Python headers are needed,
so a file compiles in seconds and cross-compiles on a machine without a GPU.

Run ``python -m easydel_b200.csrc.build`` (add ``--force`` to rebuild everything,
``--verbose`` for ptxas register/shared-memory reports). ``EDL_NVCC_EXTRA`` adds compiler flags, and
``--out PATH`` links the result somewhere else, so that a checking build
(``EDL_NVCC_EXTRA=-DEDL_BOUNDS_CHECK python -m easydel_b200.csrc.build --out /tmp/libedl_check.so``, loaded
with ``EDL_LIB_PATH``) can sit beside the production library.
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
BUILD = CSRC / "build"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libedl_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, flags: list[str], force: bool, verbose: bool) -> tuple[Path, bool, str]:
    obj = BUILD / (src.stem + ".o")
    stamp = BUILD / (src.stem + ".sha")
    dig = _digest(src, flags)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, False, ""
    cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(dig)
    return obj, True, (proc.stderr if verbose else "")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False, jobs: int | None = None, out: str | None = None) -> Path:
    """Compiles what changed and links the shared library; returns its path. ``out``: link there instead of the
    in-tree location, with the objects in a directory of their own (a build with other flags beside the main one)."""
    global BUILD, LIB_PATH
    nvcc = _nvcc()
    if out is not None:
        LIB_PATH = Path(out).resolve()
        BUILD = CSRC / "build" / ("alt-" + hashlib.sha256(str(LIB_PATH).encode()).hexdigest()[:8])
        BUILD.mkdir(parents=True, exist_ok=True)
        LIB_PATH.parent.mkdir(parents=True, exist_ok=True)
    BUILD.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS)
    extra = os.environ.get("EDL_NVCC_EXTRA", "").split()   # e.g. -DEDL_BOUNDS_CHECK for a checking build
    flags += extra
    if verbose:
        flags += ["-Xptxas", "-v"]
    srcs = sources()
    objs: list[Path] = []
    changed = False
    with cf.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
        futs = [ex.submit(_compile_one, nvcc, s, flags, force, verbose) for s in srcs]
        for f in futs:
            obj, did, log = f.result()
            objs.append(obj)
            changed |= did
            if log:
                print(log, file=sys.stderr)
    if changed or not LIB_PATH.exists():
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-lcudart_static", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("-j", "--jobs", type=int, default=None)
    ap.add_argument("--out", default=None, help="link the library here instead of easydel_b200/lib/")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, jobs=a.jobs, out=a.out))


if __name__ == "__main__":
    main()
