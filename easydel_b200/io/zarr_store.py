"""Minimal zarr-v2 array store compatible with TensorStore's ``zarr`` driver.

One directory per array: a ``.zarray`` JSON document plus C-order chunk files named by their
``.``-separated chunk index (``0.0``, ``0.1`` ...). Chunks are zstd-compressed (codec id ``zstd``,
through pyarrow's native codec) or stored raw. bfloat16 uses TensorStore's ``"bfloat16"`` dtype
string; everything else uses numpy typestrings (``"<f4"``).

This is the storage half of the reference's checkpoint layout, which it reaches through
``jax.experimental.array_serialization`` + TensorStore (easydel/infra/mixins/bridge.py:2641-2685).
Reads and writes are chunk-parallel on a thread pool (the codec releases the GIL).
"""

from __future__ import annotations

import concurrent.futures as cf
import itertools
import json
import math
import os
import typing as tp

import numpy as np
import torch

try:  # pyarrow ships a C++ zstd codec
    import pyarrow as _pa

    _ZSTD = _pa.Codec("zstd", compression_level=1)
except Exception:  # pragma: no cover - pyarrow is part of the image
    _ZSTD = None

_POOL = cf.ThreadPoolExecutor(max_workers=min(16, (os.cpu_count() or 4)))

_TORCH_TO_ZARR = {
    torch.float32: "<f4", torch.float64: "<f8", torch.float16: "<f2", torch.bfloat16: "bfloat16",
    torch.int8: "|i1", torch.uint8: "|u1", torch.int16: "<i2", torch.int32: "<i4", torch.int64: "<i8",
    torch.bool: "|b1", torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
}
_ZARR_TO_TORCH = {v: k for k, v in _TORCH_TO_ZARR.items()}
_DTYPE_NAMES = {torch.float32: "float32", torch.float64: "float64", torch.float16: "float16",
                torch.bfloat16: "bfloat16", torch.int8: "int8", torch.uint8: "uint8", torch.int16: "int16",
                torch.int32: "int32", torch.int64: "int64", torch.bool: "bool",
                torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2"}


def dtype_name(dt: torch.dtype) -> str:
    return _DTYPE_NAMES[dt]


def dtype_from_name(name: str) -> torch.dtype:
    for k, v in _DTYPE_NAMES.items():
        if v == name:
            return k
    raise KeyError(name)


def default_chunks(shape: tp.Sequence[int], itemsize: int, chunk_bytes: int = 256 << 20,
                   per_expert: bool = False) -> list[int]:
    """Splits the leading dimensions until a chunk fits ``chunk_bytes``; stacked experts get one chunk each."""
    shape = [int(s) for s in shape]
    if not shape:
        return []
    chunks = list(shape)
    if per_expert and len(shape) == 3:
        chunks[0] = 1
    i = 0
    while math.prod(chunks) * itemsize > chunk_bytes and i < len(chunks):
        if chunks[i] > 1:
            chunks[i] = max(1, chunks[i] // 2)
        else:
            i += 1
    return [max(1, c) for c in chunks]


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
        view = t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.uint8)
        return view.numpy().tobytes()
    return t.numpy().tobytes()


def _from_raw(buf: bytes | memoryview, dtype: torch.dtype, shape: tp.Sequence[int]) -> torch.Tensor:
    if dtype == torch.bfloat16:
        arr = np.frombuffer(buf, dtype=np.int16).reshape(shape)
        return torch.from_numpy(arr.copy()).view(torch.bfloat16)
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        arr = np.frombuffer(buf, dtype=np.uint8).reshape(shape)
        return torch.from_numpy(arr.copy()).view(dtype)
    np_dt = np.dtype(_TORCH_TO_ZARR[dtype])
    return torch.from_numpy(np.frombuffer(buf, dtype=np_dt).reshape(shape).copy())


def write_array(path: str, tensor: torch.Tensor, chunks: tp.Sequence[int] | None = None, compress: bool = True,
                per_expert: bool = False) -> dict:
    """Writes ``tensor`` (moved to CPU) as a zarr-v2 array directory. Returns its index entry fields."""
    t = tensor.detach().to("cpu")
    os.makedirs(path, exist_ok=True)
    shape = list(t.shape)
    chunks = list(chunks) if chunks is not None else default_chunks(shape, t.element_size(), per_expert=per_expert)
    use_zstd = compress and _ZSTD is not None
    meta = {
        "chunks": chunks if shape else [],
        "compressor": {"id": "zstd", "level": 1} if use_zstd else None,
        "dimension_separator": ".",
        "dtype": _TORCH_TO_ZARR[t.dtype],
        "fill_value": None,
        "filters": None,
        "order": "C",
        "shape": shape,
        "zarr_format": 2,
    }
    grid = [range(math.ceil(s / c)) for s, c in zip(shape, chunks)] if shape else []

    def write_chunk(idx: tuple[int, ...]) -> None:
        if shape:
            sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
            piece = t[sl]
            # zarr stores full-size edge chunks: pad with zeros
            if list(piece.shape) != chunks:
                full = torch.zeros(chunks, dtype=t.dtype)
                full[tuple(slice(0, d) for d in piece.shape)] = piece
                piece = full
            name = ".".join(str(i) for i in idx)
        else:
            piece, name = t.reshape(1), "0"
        raw = _raw_bytes(piece)
        data = _ZSTD.compress(raw, asbytes=True) if use_zstd else raw
        tmp = os.path.join(path, name + ".tmp")
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, os.path.join(path, name))

    idxs = list(itertools.product(*grid)) if shape else [()]
    if len(idxs) == 1:
        write_chunk(idxs[0])
    else:
        list(_POOL.map(write_chunk, idxs))
    with open(os.path.join(path, ".zarray"), "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=1)
    return {"shape": shape, "dtype": dtype_name(t.dtype)}


def read_meta(path: str) -> dict:
    with open(os.path.join(path, ".zarray"), encoding="utf-8") as f:
        return json.load(f)


def read_array(path: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """Reads a zarr-v2 array directory written by :func:`write_array` or by TensorStore."""
    meta = read_meta(path)
    shape, chunks = list(meta["shape"]), list(meta["chunks"])
    zd = meta["dtype"]
    if zd not in _ZARR_TO_TORCH:
        raise ValueError(f"unsupported zarr dtype {zd!r} in {path}")
    dtype = _ZARR_TO_TORCH[zd]
    if meta.get("order", "C") != "C":
        raise ValueError("only C-order zarr arrays are supported")
    comp = meta.get("compressor")
    sep = meta.get("dimension_separator", ".")
    itemsize = torch.empty(0, dtype=dtype).element_size()
    result = torch.empty(shape, dtype=dtype) if out is None else out

    def decode(raw: bytes, n_bytes: int) -> bytes:
        if comp is None:
            return raw
        cid = comp.get("id")
        if cid == "zstd":
            if _ZSTD is None:
                raise RuntimeError("zstd chunks need pyarrow's codec")
            return _ZSTD.decompress(raw, decompressed_size=n_bytes, asbytes=True)
        if cid in ("gzip", "zlib"):
            import zlib

            return zlib.decompress(raw, 31 if cid == "gzip" else 15)
        raise ValueError(f"unsupported zarr compressor {cid!r}")

    if not shape:
        with open(os.path.join(path, "0"), "rb") as f:
            raw = decode(f.read(), itemsize)
        result.copy_(_from_raw(raw, dtype, [1]).reshape(()))
        return result

    grid = [range(math.ceil(s / c)) for s, c in zip(shape, chunks)]
    n_bytes = math.prod(chunks) * itemsize

    def read_chunk(idx: tuple[int, ...]) -> None:
        name = sep.join(str(i) for i in idx)
        fp = os.path.join(path, name)
        sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
        if not os.path.exists(fp):
            result[sl] = 0  # absent chunk = fill value
            return
        with open(fp, "rb") as f:
            raw = decode(f.read(), n_bytes)
        piece = _from_raw(raw, dtype, chunks)
        want = tuple(slice(0, s.stop - s.start) for s in sl)
        result[sl] = piece[want]

    idxs = list(itertools.product(*grid))
    if len(idxs) == 1:
        read_chunk(idxs[0])
    else:
        list(_POOL.map(read_chunk, idxs))
    return result
