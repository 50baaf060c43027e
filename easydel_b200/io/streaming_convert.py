"""Hugging Face safetensors -> EasyDeL checkpoint layout, one tensor at a time.

The reference converts large checkpoints shard by shard so that a model never has to fit in host memory while it is
converted (easydel/infra/mixins/bridge.py:2269, ``StateDictConverter`` streaming path). Here the conversion rules of
``utils.parameters_transformation.hf_to_easydel`` are applied tensor by tensor: every safetensors shard is opened
lazily, each tensor is renamed / transposed and written as its own zarr array, and only the per-expert matrices of
one projection are held back until all experts of that projection have been seen (they are stored stacked). Peak
host memory is one tensor, or one stacked expert projection.
"""

from __future__ import annotations

import datetime
import json
import os
import typing as tp

import torch

from ..utils import parameters_transformation as PT
from . import checkpoint as CK
from . import zarr_store as Z


class LazySafetensors:
    """Read-only mapping over the tensors of a (sharded) safetensors checkpoint; tensors are read on access."""

    def __init__(self, path: str):
        self.path = path
        index = os.path.join(path, CK.SAFETENSORS_INDEX_NAME)
        single = os.path.join(path, CK.SAFETENSORS_NAME)
        self.where: dict[str, str] = {}
        if os.path.exists(index):
            with open(index, encoding="utf-8") as f:
                self.where = dict(json.load(f)["weight_map"])
        elif os.path.exists(single):
            from safetensors import safe_open

            with safe_open(single, framework="pt") as f:
                self.where = {k: CK.SAFETENSORS_NAME for k in f.keys()}
        else:
            raise FileNotFoundError(f"no safetensors weights under {path}")
        self._open: tuple[str, tp.Any] | None = None
        self.reads = 0

    def keys(self):
        return self.where.keys()

    def __len__(self) -> int:
        return len(self.where)

    def __contains__(self, key) -> bool:
        return key in self.where

    def __iter__(self):
        return iter(self.where)

    def files(self) -> list[str]:
        return sorted(set(self.where.values()))

    def keys_in_file_order(self) -> list[str]:
        """Keys grouped by shard (each shard is opened once)."""
        by_file: dict[str, list[str]] = {}
        for k, fn in self.where.items():
            by_file.setdefault(fn, []).append(k)
        return [k for fn in sorted(by_file) for k in by_file[fn]]

    def __getitem__(self, key: str) -> torch.Tensor:
        from safetensors import safe_open

        fn = self.where[key]
        if self._open is None or self._open[0] != fn:
            self.close()
            h = safe_open(os.path.join(self.path, fn), framework="pt")
            h.__enter__()
            self._open = (fn, h)
        self.reads += 1
        return self._open[1].get_tensor(key)

    def close(self) -> None:
        if self._open is not None:
            self._open[1].__exit__(None, None, None)
            self._open = None


def iter_easydel_leaves(hf_state, layernorm_names: tp.Sequence[str] = (), embedding_layer_names=None,
                        num_experts_hint: int | None = None):
    """Yields ``(easydel leaf name, tensor)`` for every tensor of ``hf_state`` (any mapping with
    ``keys_in_file_order`` or plain ``keys``), in the order the tensors are stored. Per-expert projection weights are
    collected and yielded stacked ``[E, in, out]`` once the last expert of a projection has been read."""
    emb = tuple(embedding_layer_names or PT.DEFAULT_EMBEDDING_NAMES)
    lns = tuple(layernorm_names or ())
    keys = hf_state.keys_in_file_order() if hasattr(hf_state, "keys_in_file_order") else list(hf_state.keys())
    # how many experts each (prefix, projection) has: known from the key set alone, before any tensor is read
    expected: dict[tuple[str, str], int] = {}
    for k in keys:
        m = PT._EXPERT_RE.match(k)
        if m:
            g = (m.group(1), m.group(3))
            expected[g] = max(expected.get(g, 0), int(m.group(2)) + 1)
    pending: dict[tuple[str, str], dict[int, torch.Tensor]] = {}
    for key in keys:
        m = PT._EXPERT_RE.match(key)
        if m:
            g = (m.group(1), m.group(3))
            got = pending.setdefault(g, {})
            got[int(m.group(2))] = hf_state[key]
            if len(got) == expected[g]:
                stacked = torch.stack([got[e] for e in range(expected[g])])
                del pending[g]
                yield f"{g[0]}experts.{g[1]}.kernel", stacked.permute(0, 2, 1)
            continue
        one = PT.hf_to_easydel({key: hf_state[key]}, embedding_layer_names=emb, layernorm_names=lns)
        yield from one.items()
    if pending:
        raise KeyError(f"incomplete expert sets in the checkpoint: {sorted(pending)[:4]}")


def stream_hf_to_easydel(source: str, out: str, dtype=None, task=None, verbose: bool = False) -> dict:
    """Converts the safetensors checkpoint in ``source`` into the EasyDeL layout in ``out`` without instantiating
    the model. Returns ``{"tensors": n, "bytes": b, "peak_tensor_bytes": p}``."""
    from ..infra.factory import TaskType, registry

    dtype = CK.coerce_dtype(dtype)
    cfg = CK.load_config(source)
    os.makedirs(out, exist_ok=True)
    task = TaskType(task) if task is not None and not isinstance(task, TaskType) else (task or TaskType.CAUSAL_LM)
    lns: tuple[str, ...] = ()
    try:
        reg = registry.get_module_registration(task, cfg.model_type)
        lns = tuple(reg.layernorm_names or ())
        cfg.architectures = [reg.module.__name__]
    except Exception:
        pass
    cfg.save_pretrained(out)
    gen = {k: getattr(cfg, k) for k in ("bos_token_id", "eos_token_id", "pad_token_id") if getattr(cfg, k, None) is not None}
    gen["_from_model_config"] = True
    CK._atomic_json(os.path.join(out, CK.GENERATION_CONFIG_NAME), gen)
    lazy = LazySafetensors(source)
    entries, total, peak = [], 0, 0
    try:
        for name, t in iter_easydel_leaves(lazy, layernorm_names=lns):
            if dtype is not None and t.is_floating_point():
                t = t.to(dtype)
            t = t.contiguous()
            nbytes = t.numel() * t.element_size()
            total += nbytes
            peak = max(peak, nbytes)
            rel = CK._leaf_path(CK.MODEL_PREFIX, name)
            info = Z.write_array(os.path.join(out, rel), t, per_expert=t.dim() == 3 and ".experts." in name)
            entries.append({"path": rel.replace(os.sep, "/"), "shape": info["shape"], "dtype": info["dtype"]})
            if verbose:
                print(f"[convert] {name} {tuple(t.shape)}")
            del t
    finally:
        lazy.close()
    CK._atomic_json(os.path.join(out, CK.TENSORSTORE_INDEX_NAME),
                    {"format": "tensorstore", "version": "easydel", "prefixes": {CK.MODEL_PREFIX: entries}})
    CK._atomic_json(os.path.join(out, CK.CHECKPOINT_METADATA_NAME),
                    {"timestamp": datetime.datetime.now().isoformat(), "custom_metadata": {"step": 0}})
    return {"tensors": len(entries), "bytes": total, "peak_tensor_bytes": peak}
