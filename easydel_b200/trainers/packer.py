"""Sequence packing for SFT (easydel/trainers/packer.py and sft_trainer.py:198-225).

``bfd``: best-fit-decreasing bin packing of whole examples into rows of ``seq_length`` tokens (no example is
split; rows carry ``segment_ids`` so attention and positions restart per example). ``wrapped``: greedy
concatenation of the token stream cut every ``seq_length`` tokens (examples may straddle rows).
The inner bin search runs in the native packer when the extension is built.
"""

from __future__ import annotations

import bisect


def _first_fit_decreasing(lengths: list[int], capacity: int) -> list[list[int]]:
    try:
        from ..data import _native

        if _native.available():
            return _native.pack_bfd(lengths, capacity)
    except Exception:
        pass
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: list[list[int]] = []
    space: list[int] = []          # remaining capacity, kept sorted ascending with parallel index list
    space_idx: list[int] = []
    for i in order:
        n = min(lengths[i], capacity)
        j = bisect.bisect_left(space, n)          # tightest bin that still fits (best fit)
        if j == len(space):
            bins.append([i])
            rem, b = capacity - n, len(bins) - 1
        else:
            b = space_idx.pop(j)
            rem = space.pop(j) - n
            bins[b].append(i)
        k = bisect.bisect_left(space, rem)
        space.insert(k, rem)
        space_idx.insert(k, b)
    return bins


def pack_sequences(rows: list[dict], seq_length: int, strategy: str = "bfd", pad_token_id: int = 0) -> list[dict]:
    out = []
    if strategy == "wrapped":
        ids, labels, seg = [], [], []
        sid = 1
        for r in rows:
            ids += list(r["input_ids"])
            labels += list(r.get("labels", r["input_ids"]))
            seg += [sid] * len(r["input_ids"])
            sid += 1
        for s in range(0, len(ids) - seq_length + 1, seq_length):
            sg = seg[s:s + seq_length]
            base = sg[0] - 1
            out.append({"input_ids": ids[s:s + seq_length], "labels": labels[s:s + seq_length],
                        "segment_ids": [x - base for x in sg], "attention_mask": [1] * seq_length})
        return out
    lengths = [len(r["input_ids"]) for r in rows]
    for members in _first_fit_decreasing(lengths, seq_length):
        ids, labels, seg = [], [], []
        for sid, i in enumerate(members, start=1):
            r = rows[i]
            t = list(r["input_ids"])[:seq_length - len(ids)]
            lab = list(r.get("labels", r["input_ids"]))[:len(t)]
            if lab:
                lab[0] = -100   # the first token of an example is never predicted from the previous example
            ids += t
            labels += lab
            seg += [sid] * len(t)
        pad = seq_length - len(ids)
        out.append({"input_ids": ids + [pad_token_id] * pad, "labels": labels + [-100] * pad,
                    "segment_ids": seg + [0] * pad, "attention_mask": [1] * len(ids) + [0] * pad})
    return out
