"""Sharded data sources (easydel/data/core/protocols.py:70-298, data/sources/base.py:192-908).

A ``ShardedDataSource`` is a list of shards (files, or slices of an in-memory table) that can each be opened as
an iterator of row dicts starting at any row, which is what makes deterministic resume and per-rank sharding
cheap: a reader's position is ``(shard index, row index)``.
"""

from __future__ import annotations

import csv
import glob
import json
import os
import typing as tp
from dataclasses import dataclass


@dataclass
class SourceState:
    """Resume position of an iteration over a source (easydel/data/core/protocols.py:616)."""

    shard: int = 0
    row: int = 0
    epoch: int = 0

    def to_dict(self) -> dict:
        return {"shard": self.shard, "row": self.row, "epoch": self.epoch}

    @classmethod
    def from_dict(cls, d: dict) -> "SourceState":
        return cls(int(d.get("shard", 0)), int(d.get("row", 0)), int(d.get("epoch", 0)))


class ShardedDataSource:
    @property
    def shard_names(self) -> list[str]:
        raise NotImplementedError

    def num_shards(self) -> int:
        return len(self.shard_names)

    def open_shard(self, shard_name: str) -> tp.Iterator[dict]:
        return self.open_shard_at_row(shard_name, 0)

    def open_shard_at_row(self, shard_name: str, row: int) -> tp.Iterator[dict]:
        raise NotImplementedError

    def shard_rows(self, shard_name: str) -> int | None:
        return None

    # ---- conveniences shared by every source -------------------------------------------------------------
    def iterate(self, state: SourceState | None = None, rank: int = 0, world_size: int = 1) -> tp.Iterator[dict]:
        """Rows of the shards owned by ``rank`` (shard i belongs to rank i % world_size), resumable via ``state``."""
        state = state if state is not None else SourceState()
        names = self.shard_names
        mine = [i for i in range(len(names)) if i % world_size == rank] if len(names) >= world_size else None
        if mine is None:     # fewer shards than ranks: every rank reads every shard and keeps every world-th row
            for i in range(state.shard, len(names)):
                start = state.row if i == state.shard else 0
                for j, row in enumerate(self.open_shard_at_row(names[i], start), start=start):
                    state.shard, state.row = i, j + 1
                    if j % world_size == rank:
                        yield row
            return
        for i in mine:
            if i < state.shard:
                continue
            start = state.row if i == state.shard else 0
            for j, row in enumerate(self.open_shard_at_row(names[i], start), start=start):
                state.shard, state.row = i, j + 1
                yield row

    def __iter__(self):
        return self.iterate()

    def map(self, fn: tp.Callable[[dict], dict]) -> "ShardedDataSource":
        from .transforms import MappedSource

        return MappedSource(self, fn)

    def filter(self, pred: tp.Callable[[dict], bool]) -> "ShardedDataSource":
        from .transforms import FilteredSource

        return FilteredSource(self, pred)

    def select_fields(self, fields: tp.Sequence[str]) -> "ShardedDataSource":
        return self.map(lambda r: {k: r[k] for k in fields if k in r})

    def rename_fields(self, mapping: dict[str, str]) -> "ShardedDataSource":
        return self.map(lambda r: {mapping.get(k, k): v for k, v in r.items()})


def _expand(paths: str | tp.Sequence[str]) -> list[str]:
    out: list[str] = []
    for p in ([paths] if isinstance(paths, str) else list(paths)):
        if os.path.isdir(p):
            out += sorted(os.path.join(p, f) for f in os.listdir(p) if not f.startswith("."))
        elif any(c in p for c in "*?["):
            out += sorted(glob.glob(p, recursive=True))
        else:
            out.append(p)
    if not out:
        raise FileNotFoundError(f"no files match {paths!r}")
    return out


class _FileSource(ShardedDataSource):
    def __init__(self, paths: str | tp.Sequence[str]):
        self.files = _expand(paths)

    @property
    def shard_names(self) -> list[str]:
        return self.files


class JsonDataSource(_FileSource):
    """``.jsonl`` (one object per line) or ``.json`` (a list of objects, optionally under ``field``)."""

    def __init__(self, paths, field: str | None = None):
        super().__init__(paths)
        self.field = field

    def open_shard_at_row(self, shard_name, row):
        if shard_name.endswith(".json"):
            with open(shard_name) as f:
                data = json.load(f)
            data = data[self.field] if self.field else data
            yield from data[row:]
            return
        with open(shard_name) as f:
            for i, line in enumerate(f):
                if i >= row and line.strip():
                    yield json.loads(line)


class TextDataSource(_FileSource):
    def __init__(self, paths, text_field: str = "text"):
        super().__init__(paths)
        self.text_field = text_field

    def open_shard_at_row(self, shard_name, row):
        with open(shard_name) as f:
            for i, line in enumerate(f):
                if i >= row:
                    yield {self.text_field: line.rstrip("\n")}


class CsvDataSource(_FileSource):
    def open_shard_at_row(self, shard_name, row):
        with open(shard_name, newline="") as f:
            for i, rec in enumerate(csv.DictReader(f)):
                if i >= row:
                    yield dict(rec)


class ParquetDataSource(_FileSource):
    """Row-group streaming through pyarrow; ``columns`` restricts what is read from disk."""

    def __init__(self, paths, columns: list[str] | None = None, batch_rows: int = 1024):
        super().__init__(paths)
        self.columns, self.batch_rows = columns, batch_rows

    def shard_rows(self, shard_name):
        import pyarrow.parquet as pq

        return pq.ParquetFile(shard_name).metadata.num_rows

    def open_shard_at_row(self, shard_name, row):
        import pyarrow.parquet as pq

        pf = pq.ParquetFile(shard_name)
        seen = 0
        for batch in pf.iter_batches(batch_size=self.batch_rows, columns=self.columns):
            n = batch.num_rows
            if seen + n <= row:
                seen += n
                continue
            rows = batch.to_pylist()
            yield from rows[max(0, row - seen):]
            seen += n


class ArrowDataSource(_FileSource):
    """Arrow IPC files / streams (what ``datasets`` writes to its cache)."""

    def open_shard_at_row(self, shard_name, row):
        import pyarrow as pa

        with pa.memory_map(shard_name) as src:
            try:
                reader = pa.ipc.open_file(src)
                batches = (reader.get_batch(i) for i in range(reader.num_record_batches))
            except pa.ArrowInvalid:
                reader = pa.ipc.open_stream(src)
                batches = iter(reader)
            seen = 0
            for b in batches:
                if seen + b.num_rows <= row:
                    seen += b.num_rows
                    continue
                yield from b.to_pylist()[max(0, row - seen):]
                seen += b.num_rows


class InMemorySource(ShardedDataSource):
    """A python sequence (or anything with ``__len__`` / ``__getitem__``) cut into ``num_shards`` slices."""

    def __init__(self, rows: tp.Sequence[dict], num_shards: int = 1):
        self.rows = rows
        n = len(rows)
        k = max(1, min(num_shards, n or 1))
        self.bounds = [(i * n // k, (i + 1) * n // k) for i in range(k)]

    @property
    def shard_names(self):
        return [f"mem-{i}" for i in range(len(self.bounds))]

    def shard_rows(self, shard_name):
        lo, hi = self.bounds[int(shard_name.split("-")[1])]
        return hi - lo

    def open_shard_at_row(self, shard_name, row):
        lo, hi = self.bounds[int(shard_name.split("-")[1])]
        for i in range(lo + row, hi):
            yield dict(self.rows[i])


class HuggingFaceDataSource(ShardedDataSource):
    """Wraps a ``datasets`` dataset object (map-style or iterable) that the caller has already loaded; the package
    is optional and there is no hub access here (easydel/data/sources/hf_wrapper.py)."""

    def __init__(self, dataset, num_shards: int = 1):
        self.ds = dataset
        self.n = num_shards if hasattr(dataset, "__len__") else 1

    @property
    def shard_names(self):
        return [f"hf-{i}" for i in range(self.n)]

    def open_shard_at_row(self, shard_name, row):
        i = int(shard_name.split("-")[1])
        if hasattr(self.ds, "__len__"):
            n = len(self.ds)
            lo, hi = i * n // self.n, (i + 1) * n // self.n
            for j in range(lo + row, hi):
                yield dict(self.ds[j])
        else:
            for j, r in enumerate(self.ds):
                if j >= row:
                    yield dict(r)


class CompositeDataSource(ShardedDataSource):
    """Concatenation of sources: shards keep their order, names are prefixed with the source index."""

    def __init__(self, sources: tp.Sequence[ShardedDataSource]):
        self.sources = list(sources)

    @property
    def shard_names(self):
        return [f"{i}::{n}" for i, s in enumerate(self.sources) for n in s.shard_names]

    def open_shard_at_row(self, shard_name, row):
        i, name = shard_name.split("::", 1)
        return self.sources[int(i)].open_shard_at_row(name, row)


_BY_EXT = {".jsonl": JsonDataSource, ".json": JsonDataSource, ".parquet": ParquetDataSource, ".arrow": ArrowDataSource,
           ".csv": CsvDataSource, ".txt": TextDataSource}


def create_source(paths: str | tp.Sequence[str], type: str | None = None, **kw) -> ShardedDataSource:
    """Picks the source class from ``type`` or from the first file's extension."""
    if type is None:
        first = _expand(paths)[0]
        type = os.path.splitext(first)[1]
    key = type if type.startswith(".") else "." + {"jsonl": "jsonl", "json": "json", "parquet": "parquet",
                                                   "arrow": "arrow", "csv": "csv", "text": "txt", "txt": "txt"}[type]
    return _BY_EXT[key](paths, **kw)
