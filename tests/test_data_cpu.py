"""Data pipeline: sources round-trip through the writers, resume positions, packing strategies, mixtures."""

import json

import numpy as np
import pytest

from easydel_b200 import data as D


class Tok:
    pad_token_id, eos_token_id = 0, 2

    def __call__(self, text, add_special_tokens=True, **_):
        return {"input_ids": [3 + (ord(c) % 90) for c in text]}


def _rows(n):
    return [{"text": "x" * (1 + i % 7), "id": i} for i in range(n)]


@pytest.mark.parametrize("fmt", ["jsonl", "parquet", "arrow"])
def test_writer_reader_roundtrip_and_resume(tmp_path, fmt):
    files = D.save_source(_rows(25), str(tmp_path), fmt, rows_per_shard=10)
    assert len(files) == 3
    src = D.create_source(str(tmp_path))
    got = list(src)
    assert [r["id"] for r in got] == list(range(25))
    st = D.SourceState()
    it = src.iterate(st)
    first = [next(it)["id"] for _ in range(13)]
    assert first == list(range(13)) and (st.shard, st.row) == (1, 3)
    rest = [r["id"] for r in src.iterate(D.SourceState.from_dict(st.to_dict()))]
    assert rest == list(range(13, 25))
    # two ranks partition the shards
    a = [r["id"] for r in src.iterate(None, 0, 2)]
    b = [r["id"] for r in src.iterate(None, 1, 2)]
    assert sorted(a + b) == list(range(25)) and not set(a) & set(b)


def test_tokenize_and_pack_strategies():
    src = D.InMemorySource(_rows(40)).map(D.TokenizeTransform(Tok(), max_length=16))
    for strategy in ("greedy", "pool", "first_fit"):
        packed = list(D.PackedShardedSource(src, 16, strategy, pad_token_id=0, eos_token_id=2))
        assert all(len(r["input_ids"]) == 16 == len(r["segment_ids"]) for r in packed)
        n_tok = sum(sum(r["attention_mask"]) for r in packed)
        assert n_tok == sum(len(Tok()(r["text"])["input_ids"]) + 1 for r in _rows(40))
        for r in packed:   # every document start is masked out of the loss
            seg = r["segment_ids"]
            for i in range(16):
                if seg[i] and (i == 0 or seg[i] != seg[i - 1]):
                    assert r["labels"][i] == -100
    ff = list(D.PackedShardedSource(src, 16, "first_fit"))
    gr = list(D.PackedShardedSource(src, 16, "greedy"))
    assert len(ff) <= len(gr)


def test_mixture_weights_and_schedule():
    a = D.InMemorySource([{"v": "a"}] * 50)
    b = D.InMemorySource([{"v": "b"}] * 50)
    mix = D.MixtureSource({"a": a, "b": b}, weights=[(0, [0.75, 0.25]), (128, [0.0, 1.0])], block_size=32, seed=1)
    it = iter(mix)
    first = [next(it) for _ in range(128)]
    frac = np.mean([r["v"] == "a" for r in first])
    assert abs(frac - 0.75) < 1e-9            # exact over whole blocks
    later = [next(it)["v"] for _ in range(64)]
    assert set(later) == {"b"} and first[0]["__source__"] in ("a", "b")
    ended = list(D.MixtureSource([a, b], [0.5, 0.5], stop_strategy="first_exhausted", block_size=10))
    assert 90 <= len(ended) <= 100


def test_pipeline_from_config_feeds_batches(tmp_path):
    D.save_source(_rows(64), str(tmp_path / "d1"), "jsonl")
    D.save_source([{"messages": [{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}]}] * 8,
                  str(tmp_path / "d2"), "jsonl")

    class ChatTok(Tok):
        def apply_chat_template(self, msgs, tokenize=True, add_generation_prompt=False, **_):
            s = "".join(f"<{m['role']}>{m['content']}" for m in msgs) + ("<assistant>" if add_generation_prompt else "")
            return self(s)["input_ids"] if tokenize else s

    cfg = D.PipelineConfig(datasets=[D.DatasetConfig(str(tmp_path / "d1"), name="text", weight=0.8),
                                     D.DatasetConfig(str(tmp_path / "d2"), name="chat", messages_field="messages",
                                                     weight=0.2)],
                           seq_length=32, pack=True, pack_strategy="greedy", batch_size=4)
    loader = D.Pipeline.from_config(cfg, ChatTok()).loader(4, prefetch=0)
    it = iter(loader)
    batch = next(it)
    assert batch["input_ids"].shape == (4, 32) and batch["segment_ids"].shape == (4, 32)
    sd = loader.state_dict()
    assert sd["row"] == 4
    cache = D.TreeCache(str(tmp_path / "cache"))
    key = cache.fingerprint({"a": 1}, "tok-v1")
    assert cache.get_or_compute(key, lambda: [1, 2, 3]) == [1, 2, 3]
    assert D.TreeCache(str(tmp_path / "cache")).get(key) == [1, 2, 3]
