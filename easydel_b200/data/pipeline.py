"""``Pipeline``: a declarative chain source -> transforms -> pack -> batch loader, plus dataset writers and a
small on-disk cache (easydel/data/execution/pipeline.py:60, save.py, cache.py, data/core/config.py)."""

from __future__ import annotations

import hashlib
import json
import os
import pickle
import typing as tp
from dataclasses import dataclass, field

from .loader import IterableBatchLoader, PrefetchIterator
from .sources import ShardedDataSource, SourceState, create_source
from .transforms import (ChatTemplateTransform, MixtureSource, PackedShardedSource, TokenizeTransform)


@dataclass
class DatasetConfig:
    """One input of a mixture (``data/core/config.py``)."""

    data_files: str | list[str]
    type: str | None = None
    name: str | None = None
    content_field: str = "text"
    messages_field: str | None = None
    weight: float = 1.0
    columns: list[str] | None = None


@dataclass
class PipelineConfig:
    datasets: list[DatasetConfig] = field(default_factory=list)
    seq_length: int | None = None
    pack: bool = False
    pack_strategy: str = "first_fit"
    batch_size: int = 8
    seed: int = 0
    mixture_block_size: int = 64
    stop_strategy: str = "restart"
    prefetch: int = 2
    cache_dir: str | None = None


class _SourceLoader:
    """Batches the rows of a source for one rank; exposes ``state_dict`` / ``load_state_dict`` for resume."""

    def __init__(self, source: ShardedDataSource, batch_size: int, collate_fn, rank: int, world_size: int,
                 prefetch: int = 2):
        self.source, self.batch_size, self.collate_fn = source, batch_size, collate_fn
        self.rank, self.world_size, self.prefetch = rank, world_size, prefetch
        self.state = SourceState()

    def state_dict(self) -> dict:
        return self.state.to_dict()

    def load_state_dict(self, d: dict) -> None:
        self.state = SourceState.from_dict(d)

    def set_epoch(self, epoch: int) -> None:
        if epoch != self.state.epoch:
            self.state = SourceState(epoch=epoch)

    def _gen(self):
        buf = []
        for row in self.source.iterate(self.state, self.rank, self.world_size):
            buf.append(row)
            if len(buf) == self.batch_size:
                yield self.collate_fn(buf)
                buf = []

    def __iter__(self):
        return iter(PrefetchIterator(self._gen(), self.prefetch)) if self.prefetch > 0 else self._gen()


def _as_batches(self, batch_size: int, rank: int = 0, world_size: int = 1, collate_fn=None, prefetch: int = 2):
    if collate_fn is None:
        from ..trainers.utils import default_collate as collate_fn
    return _SourceLoader(self, batch_size, collate_fn, rank, world_size, prefetch)


ShardedDataSource.as_batches = _as_batches   # every source can feed a trainer directly


class Pipeline:
    """``Pipeline.from_config(cfg, tokenizer).build()`` -> a source; ``.loader(...)`` -> batches."""

    def __init__(self, source: ShardedDataSource):
        self.source = source

    @classmethod
    def from_config(cls, cfg: PipelineConfig, tokenizer=None) -> "Pipeline":
        parts, weights = {}, []
        for i, d in enumerate(cfg.datasets):
            kw = {"columns": d.columns} if d.columns and (d.type == "parquet" or str(d.data_files).endswith(".parquet")) \
                else {}
            src = create_source(d.data_files, d.type, **kw)
            if tokenizer is not None:
                if d.messages_field:
                    src = src.map(ChatTemplateTransform(tokenizer, d.messages_field, max_length=cfg.seq_length))
                else:
                    src = src.map(TokenizeTransform(tokenizer, d.content_field, max_length=cfg.seq_length))
            parts[d.name or f"dataset_{i}"] = src
            weights.append(d.weight)
        src = next(iter(parts.values())) if len(parts) == 1 else \
            MixtureSource(parts, weights, cfg.seed, cfg.mixture_block_size, cfg.stop_strategy)
        p = cls(src)
        if cfg.pack:
            if cfg.seq_length is None:
                raise ValueError("packing needs seq_length")
            p = p.pack(cfg.seq_length, cfg.pack_strategy, getattr(tokenizer, "pad_token_id", None) or 0,
                       getattr(tokenizer, "eos_token_id", None))
        return p

    def map(self, fn) -> "Pipeline":
        return Pipeline(self.source.map(fn))

    def filter(self, pred) -> "Pipeline":
        return Pipeline(self.source.filter(pred))

    def tokenize(self, tokenizer, **kw) -> "Pipeline":
        return self.map(TokenizeTransform(tokenizer, **kw))

    def chat_template(self, tokenizer, **kw) -> "Pipeline":
        return self.map(ChatTemplateTransform(tokenizer, **kw))

    def pack(self, seq_length: int, strategy: str = "first_fit", pad_token_id: int = 0, eos_token_id=None,
             **kw) -> "Pipeline":
        return Pipeline(PackedShardedSource(self.source, seq_length, strategy, pad_token_id, eos_token_id, **kw))

    def build(self) -> ShardedDataSource:
        return self.source

    def loader(self, batch_size: int, rank: int = 0, world_size: int = 1, collate_fn=None, prefetch: int = 2):
        return self.source.as_batches(batch_size, rank, world_size, collate_fn, prefetch)

    def save(self, path: str, format: str = "jsonl", rows_per_shard: int = 100_000) -> list[str]:
        return save_source(self.source, path, format, rows_per_shard)


# ---------------------------------------------------------------------------------------------- writers
def save_source(source: tp.Iterable[dict], path: str, format: str = "jsonl", rows_per_shard: int = 100_000) -> list[str]:
    """Writes rows to ``path/part-00000.<ext>`` shards (jsonl, parquet or arrow); temp file + rename per shard."""
    os.makedirs(path, exist_ok=True)
    files, buf = [], []

    def flush():
        if not buf:
            return
        name = os.path.join(path, f"part-{len(files):05d}.{format}")
        tmp = name + ".tmp"
        if format == "jsonl":
            with open(tmp, "w") as f:
                for r in buf:
                    f.write(json.dumps(r) + "\n")
        else:
            import pyarrow as pa

            table = pa.Table.from_pylist(buf)
            if format == "parquet":
                import pyarrow.parquet as pq

                pq.write_table(table, tmp, compression="zstd")
            elif format == "arrow":
                with pa.OSFile(tmp, "wb") as sink, pa.ipc.new_file(sink, table.schema) as w:
                    w.write_table(table)
            else:
                raise ValueError(f"unknown format {format!r}")
        os.replace(tmp, name)
        files.append(name)
        buf.clear()

    for r in source:
        buf.append(r)
        if len(buf) >= rows_per_shard:
            flush()
    flush()
    return files


class TreeCache:
    """Memory + disk cache keyed by a fingerprint of (inputs, transform description) (``data/cache.py``)."""

    def __init__(self, directory: str | None = None, max_memory_items: int = 64):
        self.dir, self.max_items = directory, max_memory_items
        self.mem: dict[str, tp.Any] = {}
        if directory:
            os.makedirs(directory, exist_ok=True)

    @staticmethod
    def fingerprint(*parts) -> str:
        h = hashlib.sha256()
        for p in parts:
            h.update(json.dumps(p, sort_keys=True, default=str).encode())
        return h.hexdigest()[:32]

    def get(self, key: str):
        if key in self.mem:
            return self.mem[key]
        if self.dir and os.path.exists(os.path.join(self.dir, key + ".pkl")):
            with open(os.path.join(self.dir, key + ".pkl"), "rb") as f:
                v = pickle.load(f)
            self._remember(key, v)
            return v
        return None

    def _remember(self, key, value):
        if len(self.mem) >= self.max_items:
            self.mem.pop(next(iter(self.mem)))
        self.mem[key] = value

    def put(self, key: str, value) -> None:
        self._remember(key, value)
        if self.dir:
            tmp = os.path.join(self.dir, key + ".tmp")
            with open(tmp, "wb") as f:
                pickle.dump(value, f)
            os.replace(tmp, os.path.join(self.dir, key + ".pkl"))

    def get_or_compute(self, key: str, fn: tp.Callable[[], tp.Any]):
        v = self.get(key)
        if v is None:
            v = fn()
            self.put(key, v)
        return v
