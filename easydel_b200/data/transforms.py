"""Row transforms: map / filter, tokenisation, chat templates, packing, mixing
(easydel/data/transforms/*, mixture.py:42-481)."""

from __future__ import annotations

import typing as tp

import numpy as np

from .sources import ShardedDataSource, SourceState


class MappedSource(ShardedDataSource):
    def __init__(self, base: ShardedDataSource, fn):
        self.base, self.fn = base, fn

    @property
    def shard_names(self):
        return self.base.shard_names

    def shard_rows(self, n):
        return self.base.shard_rows(n)

    def open_shard_at_row(self, shard_name, row):
        for r in self.base.open_shard_at_row(shard_name, row):
            yield self.fn(r)


class FilteredSource(ShardedDataSource):
    """Row indices refer to the unfiltered shard so that resume positions stay valid."""

    def __init__(self, base, pred):
        self.base, self.pred = base, pred

    @property
    def shard_names(self):
        return self.base.shard_names

    def open_shard_at_row(self, shard_name, row):
        for r in self.base.open_shard_at_row(shard_name, row):
            if self.pred(r):
                yield r


class TokenizeTransform:
    """``text`` (or ``prompt`` + ``completion``) -> ``input_ids`` / ``attention_mask`` (+ ``labels`` masking the
    prompt when ``mask_prompt``)."""

    def __init__(self, tokenizer, text_field: str = "text", max_length: int | None = None, add_eos: bool = True,
                 add_special_tokens: bool = True, mask_prompt: bool = True, keep_fields: tp.Sequence[str] = ()):
        self.tok, self.field, self.max_length = tokenizer, text_field, max_length
        self.add_eos, self.special, self.mask_prompt, self.keep = add_eos, add_special_tokens, mask_prompt, keep_fields

    def __call__(self, row: dict) -> dict:
        eos = getattr(self.tok, "eos_token_id", None)
        if "prompt" in row and "completion" in row:
            p = self.tok(row["prompt"], add_special_tokens=self.special)["input_ids"]
            c = self.tok(row["completion"], add_special_tokens=False)["input_ids"]
            if self.add_eos and eos is not None and (not c or c[-1] != eos):
                c = c + [eos]
            ids = p + c
            labels = ([-100] * len(p) if self.mask_prompt else list(p)) + c
        else:
            ids = list(self.tok(row[self.field], add_special_tokens=self.special)["input_ids"])
            if self.add_eos and eos is not None and (not ids or ids[-1] != eos):
                ids.append(eos)
            labels = list(ids)
        if self.max_length:
            ids, labels = ids[: self.max_length], labels[: self.max_length]
        out = {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}
        for k in self.keep:
            if k in row:
                out[k] = row[k]
        return out


class ChatTemplateTransform:
    """``messages`` -> text (or tokens) through the tokenizer's chat template; with ``assistant_only`` the labels
    cover assistant turns only."""

    def __init__(self, tokenizer, messages_field: str = "messages", tokenize: bool = True, max_length: int | None = None,
                 assistant_only: bool = False, tools_field: str | None = "tools"):
        self.tok, self.field, self.tokenize, self.max_length = tokenizer, messages_field, tokenize, max_length
        self.assistant_only, self.tools_field = assistant_only, tools_field

    @staticmethod
    def _ids(x):
        return list(x["input_ids"] if isinstance(x, dict) else x)

    def __call__(self, row: dict) -> dict:
        msgs = row[self.field]
        kw = {}
        if self.tools_field and row.get(self.tools_field):
            kw["tools"] = row[self.tools_field]
        if not self.tokenize:
            return {"text": self.tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=False, **kw)}
        ids = self._ids(self.tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=False, **kw))
        labels = list(ids)
        if self.assistant_only:
            keep = [False] * len(ids)
            for i, m in enumerate(msgs):
                if m.get("role") != "assistant":
                    continue
                pre = self._ids(self.tok.apply_chat_template(msgs[:i], tokenize=True, add_generation_prompt=True,
                                                             **kw)) if i else []
                upto = self._ids(self.tok.apply_chat_template(msgs[:i + 1], tokenize=True,
                                                              add_generation_prompt=False, **kw))
                for j in range(len(pre), min(len(upto), len(ids))):
                    keep[j] = True
            labels = [t if k else -100 for t, k in zip(ids, keep)]
        if self.max_length:
            ids, labels = ids[: self.max_length], labels[: self.max_length]
        return {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}


# ------------------------------------------------------------------------------------------------ packing
def _emit(members: list[dict], seq_length: int, pad_id: int) -> dict:
    ids, labels, seg = [], [], []
    for sid, r in enumerate(members, start=1):
        t = list(r["input_ids"])
        lab = list(r.get("labels", t))
        if lab:
            lab[0] = -100
        ids += t
        labels += lab
        seg += [sid] * len(t)
    pad = seq_length - len(ids)
    return {"input_ids": ids + [pad_id] * pad, "labels": labels + [-100] * pad, "segment_ids": seg + [0] * pad,
            "attention_mask": [1] * len(ids) + [0] * pad}


class GreedyPacker:
    """Appends examples to the current row until the next one does not fit (``pack.py:77``)."""

    def __init__(self, seq_length: int, pad_token_id: int = 0, eos_token_id: int | None = None):
        self.L, self.pad, self.eos = seq_length, pad_token_id, eos_token_id
        self.cur: list[dict] = []
        self.used = 0

    def _prep(self, row):
        ids = list(row["input_ids"])[: self.L]
        if self.eos is not None and (not ids or ids[-1] != self.eos) and len(ids) < self.L:
            ids.append(self.eos)
        lab = list(row.get("labels", ids))[: len(ids)]
        lab += ids[len(lab):]
        return {"input_ids": ids, "labels": lab}

    def add(self, row: dict) -> list[dict]:
        r = self._prep(row)
        out = []
        if self.used + len(r["input_ids"]) > self.L and self.cur:
            out.append(_emit(self.cur, self.L, self.pad))
            self.cur, self.used = [], 0
        self.cur.append(r)
        self.used += len(r["input_ids"])
        return out

    def flush(self) -> list[dict]:
        out = [_emit(self.cur, self.L, self.pad)] if self.cur else []
        self.cur, self.used = [], 0
        return out


class PoolPacker(GreedyPacker):
    """Keeps ``pool_size`` open rows and puts each example into the fullest row that still fits (``pack.py:212``)."""

    def __init__(self, seq_length, pad_token_id=0, eos_token_id=None, pool_size: int = 8):
        super().__init__(seq_length, pad_token_id, eos_token_id)
        self.pool: list[tuple[int, list[dict]]] = []
        self.pool_size = pool_size

    def add(self, row):
        r = self._prep(row)
        n = len(r["input_ids"])
        best = None
        for i, (used, _) in enumerate(self.pool):
            if used + n <= self.L and (best is None or used > self.pool[best][0]):
                best = i
        out = []
        if best is None:
            if len(self.pool) >= self.pool_size:
                j = max(range(len(self.pool)), key=lambda i: self.pool[i][0])
                out.append(_emit(self.pool.pop(j)[1], self.L, self.pad))
            self.pool.append((n, [r]))
        else:
            used, members = self.pool[best]
            members.append(r)
            self.pool[best] = (used + n, members)
        return out

    def flush(self):
        out = [_emit(m, self.L, self.pad) for _, m in self.pool]
        self.pool = []
        return out


class FirstFitPacker(GreedyPacker):
    """Buffers ``buffer_size`` examples, sorts them by length (descending) and first-fits them into rows
    (``pack.py:288-407``). The bin search runs in the native packer when it is built."""

    def __init__(self, seq_length, pad_token_id=0, eos_token_id=None, buffer_size: int = 1024):
        super().__init__(seq_length, pad_token_id, eos_token_id)
        self.buf: list[dict] = []
        self.buffer_size = buffer_size

    def _pack_buffer(self):
        from ..trainers.packer import _first_fit_decreasing

        bins = _first_fit_decreasing([len(r["input_ids"]) for r in self.buf], self.L)
        out = [_emit([self.buf[i] for i in b], self.L, self.pad) for b in bins]
        self.buf = []
        return out

    def add(self, row):
        self.buf.append(self._prep(row))
        return self._pack_buffer() if len(self.buf) >= self.buffer_size else []

    def flush(self):
        return self._pack_buffer() if self.buf else []


class PackedShardedSource(ShardedDataSource):
    """Packs the rows of every shard of ``base`` on the fly (``pack.py:410``). Resume restarts a shard's packing
    from its first row, so positions count emitted packed rows."""

    def __init__(self, base: ShardedDataSource, seq_length: int, strategy: str = "first_fit", pad_token_id: int = 0,
                 eos_token_id: int | None = None, **kw):
        self.base, self.L, self.strategy, self.pad, self.eos, self.kw = base, seq_length, strategy, pad_token_id, \
            eos_token_id, kw

    @property
    def shard_names(self):
        return self.base.shard_names

    def _packer(self):
        cls = {"greedy": GreedyPacker, "pool": PoolPacker, "first_fit": FirstFitPacker}[self.strategy]
        return cls(self.L, self.pad, self.eos, **self.kw)

    def open_shard_at_row(self, shard_name, row):
        p = self._packer()
        k = 0
        for r in self.base.open_shard_at_row(shard_name, 0):
            for packed in p.add(r):
                if k >= row:
                    yield packed
                k += 1
        for packed in p.flush():
            if k >= row:
                yield packed
            k += 1


# ------------------------------------------------------------------------------------------------ mixing
class MixtureSource(ShardedDataSource):
    """Samples rows from several sources with (optionally scheduled) weights (``mixture.py:42-481``).

    ``weights`` is a list of floats or a list of ``(start_step, weights)`` stages; ``block_size`` rows are drawn
    per decision so that the realised mixture is exact over every block. ``stop_strategy``: ``restart`` re-opens an
    exhausted source, ``first_exhausted`` ends the mixture, ``all_exhausted`` drops exhausted sources.
    """

    def __init__(self, sources: dict[str, ShardedDataSource] | tp.Sequence[ShardedDataSource],
                 weights: tp.Sequence[float] | tp.Sequence[tuple[int, tp.Sequence[float]]] | None = None,
                 seed: int = 0, block_size: int = 64, stop_strategy: str = "restart"):
        self.names = list(sources) if isinstance(sources, dict) else [str(i) for i in range(len(sources))]
        self.sources = list(sources.values()) if isinstance(sources, dict) else list(sources)
        n = len(self.sources)
        if weights is None:
            weights = [1.0 / n] * n
        self.stages = [(0, list(weights))] if not isinstance(weights[0], (tuple, list)) else \
            [(int(s), list(w)) for s, w in weights]
        self.seed, self.block, self.stop = seed, block_size, stop_strategy

    @property
    def shard_names(self):
        return ["mixture"]

    def weights_at(self, step: int) -> np.ndarray:
        w = self.stages[0][1]
        for s, ww in self.stages:
            if step >= s:
                w = ww
        w = np.asarray(w, dtype=np.float64)
        return w / w.sum()

    def open_shard_at_row(self, shard_name, row, rank: int = 0, world_size: int = 1):
        rng = np.random.default_rng(self.seed)
        iters = [iter(s.iterate(SourceState(), rank, world_size)) for s in self.sources]
        alive = [True] * len(iters)
        produced = 0
        while any(alive):
            w = self.weights_at(produced) * np.asarray(alive, dtype=np.float64)
            if w.sum() == 0:
                return
            w = w / w.sum()
            counts = np.floor(w * self.block).astype(int)
            for _ in range(self.block - counts.sum()):
                counts[rng.choice(len(w), p=w)] += 1
            order = np.repeat(np.arange(len(w)), counts)
            rng.shuffle(order)
            for i in order:
                try:
                    r = next(iters[i])
                except StopIteration:
                    if self.stop == "first_exhausted":
                        return
                    if self.stop == "all_exhausted":
                        alive[i] = False
                        continue
                    iters[i] = iter(self.sources[i].iterate(SourceState(), rank, world_size))
                    try:
                        r = next(iters[i])
                    except StopIteration:
                        alive[i] = False
                        continue
                if produced >= row:
                    r = dict(r)
                    r.setdefault("__source__", self.names[i])
                    yield r
                produced += 1

    def iterate(self, state=None, rank=0, world_size=1):
        state = state if state is not None else SourceState()
        for j, r in enumerate(self.open_shard_at_row("mixture", state.row, rank, world_size), start=state.row):
            state.row = j + 1
            yield r
