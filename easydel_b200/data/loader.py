"""Batch loaders: rank-sharded, shuffled per epoch, optionally prefetched on a background thread.

Stands in for the grain / tf.data loaders and ``AsyncDataLoader`` of the reference
(easydel/data/execution/loader.py:99-525, easydel/trainers/base_trainer.py:4204-4557).
"""

from __future__ import annotations

import queue
import threading
import typing as tp

import torch


class ShardedBatchLoader:
    """Map-style dataset -> batches for one data-parallel rank.

    Every epoch draws a permutation from ``seed + epoch``; rank ``r`` of ``w`` takes the batch slots
    ``r, r+w, ...`` so that the union over ranks is the global batch sequence.
    """

    def __init__(self, dataset, batch_size: int, shuffle: bool, seed: int, collate_fn, rank: int = 0,
                 world_size: int = 1, drop_last: bool = True, pin_memory: bool = False, prefetch: int = 2):
        self.dataset, self.batch_size, self.shuffle, self.seed = dataset, batch_size, shuffle, seed
        self.collate_fn, self.rank, self.world_size = collate_fn, rank, world_size
        self.drop_last, self.pin_memory, self.prefetch = drop_last, pin_memory, prefetch
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self) -> int:
        n = len(self.dataset) // (self.batch_size * self.world_size)
        if not self.drop_last and len(self.dataset) % (self.batch_size * self.world_size):
            n += 1
        return n

    def _indices(self):
        n = len(self.dataset)
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(n, generator=g).tolist()
        else:
            order = list(range(n))
        gb = self.batch_size * self.world_size
        for i in range(len(self)):
            chunk = order[i * gb:(i + 1) * gb]
            mine = chunk[self.rank * self.batch_size:(self.rank + 1) * self.batch_size]
            if mine:
                yield mine

    def _produce(self):
        for idx in self._indices():
            batch = self.collate_fn([self.dataset[i] for i in idx])
            if self.pin_memory:
                batch = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
            yield batch

    def __iter__(self):
        if self.prefetch <= 0:
            yield from self._produce()
            return
        yield from PrefetchIterator(self._produce(), self.prefetch)


class IterableBatchLoader:
    """Wraps an iterable of examples (or of ready batches) for one rank."""

    def __init__(self, iterable, batch_size: int, collate_fn, rank: int = 0, world_size: int = 1,
                 pin_memory: bool = False, already_batched: bool = False):
        self.iterable, self.batch_size, self.collate_fn = iterable, batch_size, collate_fn
        self.rank, self.world_size, self.pin_memory, self.already_batched = rank, world_size, pin_memory, already_batched

    def __len__(self):
        if self.already_batched and hasattr(self.iterable, "__len__"):
            return len(self.iterable)
        raise TypeError("iterable loader has no length")

    def __iter__(self):
        if self.already_batched:
            for b in self.iterable:
                yield b
            return
        buf = []
        for i, ex in enumerate(self.iterable):
            if (i // self.batch_size) % self.world_size != self.rank:
                continue
            buf.append(ex)
            if len(buf) == self.batch_size:
                yield self.collate_fn(buf)
                buf = []


class PrefetchIterator:
    """Runs a generator on a daemon thread, ``depth`` items ahead."""

    _END = object()

    def __init__(self, gen, depth: int = 2):
        self.q: queue.Queue = queue.Queue(maxsize=depth)
        self.err: BaseException | None = None

        def run():
            try:
                for x in gen:
                    self.q.put(x)
            except BaseException as e:  # surfaced on the consumer side
                self.err = e
            finally:
                self.q.put(self._END)

        self.t = threading.Thread(target=run, daemon=True)
        self.t.start()

    def __iter__(self):
        return self

    def __next__(self):
        x = self.q.get()
        if x is self._END:
            if self.err is not None:
                raise self.err
            raise StopIteration
        return x


def build_loader(dataset, batch_size: int, shuffle: bool, seed: int, collate_fn, rank: int = 0, world_size: int = 1,
                 num_workers: int = 0, pin_memory: bool = False, drop_last: bool = True):
    """Chooses a loader for whatever the user handed the trainer."""
    if dataset is None:
        return None
    if isinstance(dataset, (ShardedBatchLoader, IterableBatchLoader)):
        return dataset
    if hasattr(dataset, "as_batches"):  # easydel_b200.data sources
        return dataset.as_batches(batch_size=batch_size, rank=rank, world_size=world_size, collate_fn=collate_fn)
    if getattr(dataset, "already_batched", False):
        return IterableBatchLoader(dataset, batch_size, collate_fn, rank, world_size, pin_memory, already_batched=True)
    if hasattr(dataset, "__len__") and hasattr(dataset, "__getitem__"):
        return ShardedBatchLoader(dataset, batch_size, shuffle, seed, collate_fn, rank, world_size, drop_last,
                                  pin_memory, prefetch=2 if num_workers != -1 else 0)
    return IterableBatchLoader(dataset, batch_size, collate_fn, rank, world_size, pin_memory)
