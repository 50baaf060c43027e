"""Model / training-state checkpoints in the reference's on-disk layout.

``save_pretrained`` / ``save_state`` produce (easydel/infra/mixins/bridge.py:600-728, 2641-2685;
easydel/infra/base_state.py:1197-1320)::

    <dir>/config.json                  diff-style config, sorted keys, dtype names, architectures=[Class]
    <dir>/generation_config.json       when the model can generate
    <dir>/README.md                    generated model card
    <dir>/tensorstore_index.json       {"format":"tensorstore","version":"easydel","prefixes":{"model":[...],"tx":[...]}}
    <dir>/model/<k0>/<k1>/.../<leaf>/  one zarr-v2 array per parameter, path = leaf key joined by "/"
    <dir>/tx/...                       optimizer state arrays (+ tx_structure.json describing the optimizer)
    <dir>/checkpoint_metadata.json     {"timestamp", "custom_metadata": {"step": N}}
    <dir>/metadata.json                {"step","timestamp","is_temporary","has_optimizer_state","has_resume_model"}

Leaves use the reference's naming (``kernel`` transposed to ``(in, out)``, ``embedding``, stacked
``(E, in, out)`` experts). Loading accepts that layout, ``model.safetensors`` (+ index) in Hugging
Face naming, and ``easydel-model.parameters`` safetensors files.
"""

from __future__ import annotations

import datetime
import json
import os
import shutil
import typing as tp

import torch

from ..infra.base_config import (CHECKPOINT_METADATA_NAME, CONFIG_NAME, GENERATION_CONFIG_NAME, LEGACY_PARAMS_NAME,
                                 MODEL_PREFIX, OPTIMIZER_PREFIX, SAFETENSORS_INDEX_NAME, SAFETENSORS_NAME,
                                 STATE_METADATA_NAME, TENSORSTORE_INDEX_NAME, coerce_dtype)
from ..utils import parameters_transformation as PT
from . import zarr_store as Z

TX_STRUCTURE_NAME = "tx_structure.json"


def _is_writer() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def _atomic_json(path: str, obj) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(obj, f, indent=2)
    os.replace(tmp, path)


def _leaf_path(prefix: str, key: str) -> str:
    return os.path.join(prefix, *key.split("."))


# ----------------------------------------------------------------------------- writing
def write_tree(root: str, prefix: str, tensors: dict[str, torch.Tensor], float_dtype=None) -> list[dict]:
    """Writes ``{dotted key: tensor}`` under ``root/prefix``; returns the index entries."""
    entries = []
    for key, t in tensors.items():
        if float_dtype is not None and t.is_floating_point():
            t = t.to(float_dtype)
        rel = _leaf_path(prefix, key)
        info = Z.write_array(os.path.join(root, rel), t, per_expert=t.dim() == 3 and ".experts." in key)
        entries.append({"path": rel.replace(os.sep, "/"), "shape": info["shape"], "dtype": info["dtype"]})
    return entries


def _model_card(model, step: int | None) -> str:
    cfg = model.config
    return (f"---\nlibrary_name: easydel_b200\ntags: [easydel, b200]\n---\n# {type(model).__name__}\n\n"
            f"* model_type: `{cfg.model_type}`\n* parameters: {sum(p.numel() for p in model.parameters()):,}\n"
            f"* dtype: {model.dtype}\n* step: {step if step is not None else 0}\n\n"
            "Saved in the EasyDeL checkpoint layout (config.json + tensorstore_index.json + zarr arrays).\n")


def save_model(model, save_directory: str, float_dtype=None, step: int | None = None, gather: bool = True,
               write_card: bool = True, **_) -> str:
    """``save_pretrained``: config, generation config, model card, index and parameter arrays."""
    float_dtype = coerce_dtype(float_dtype)
    fsdp = getattr(getattr(model, "model", None), "fsdp_layers", None)
    if fsdp is not None:       # parameter-sharded layers: assemble them for the duration of the save (a collective)
        fsdp.materialize()
        try:
            return save_model(_Unsharded(model), save_directory, float_dtype=float_dtype, step=step, gather=gather,
                              write_card=write_card)
        finally:
            fsdp.dematerialize()
    model = getattr(model, "_wrapped", model)
    # Tensor- / expert-parallel shards are all-gathered into full tensors first (a collective over those groups,
    # so every rank takes part); only the writer rank touches the disk.
    ed_state = PT.model_to_easydel_state(model) if (PT.is_model_parallel(model) or _is_writer()) else None
    if not _is_writer():
        return save_directory
    os.makedirs(save_directory, exist_ok=True)
    cfg = model.config
    cfg.architectures = [type(model).__name__]
    cfg.save_pretrained(save_directory)
    if model.can_generate():
        gen = {k: getattr(cfg, k) for k in ("bos_token_id", "eos_token_id", "pad_token_id")
               if getattr(cfg, k, None) is not None}
        gen["_from_model_config"] = True
        _atomic_json(os.path.join(save_directory, GENERATION_CONFIG_NAME), gen)
    if write_card:
        with open(os.path.join(save_directory, "README.md"), "w", encoding="utf-8") as f:
            f.write(_model_card(model, step))
    entries = write_tree(save_directory, MODEL_PREFIX, ed_state, float_dtype)
    index_path = os.path.join(save_directory, TENSORSTORE_INDEX_NAME)
    index = {"format": "tensorstore", "version": "easydel", "prefixes": {}}
    if os.path.exists(index_path):
        try:
            with open(index_path, encoding="utf-8") as f:
                index = json.load(f)
        except Exception:
            pass
    index.setdefault("prefixes", {})[MODEL_PREFIX] = entries
    _atomic_json(index_path, index)
    _atomic_json(os.path.join(save_directory, CHECKPOINT_METADATA_NAME),
                 {"timestamp": datetime.datetime.now().isoformat(), "custom_metadata": {"step": int(step or 0)}})
    return save_directory


class _Unsharded:
    """Marks a model whose parameter-sharded layers are currently materialised (see ``save_model``)."""

    def __init__(self, model):
        self._wrapped = model

    def __getattr__(self, name):
        if name == "model":      # hides ``model.fsdp_layers`` from the recursive call
            return None
        return getattr(self._wrapped, name)


def save_optimizer_state(state, save_directory: str) -> None:
    """Optimizer moments + fp32 master weights, named like the parameters they belong to."""
    flat = state.flat
    if flat is None:
        return
    tensors: dict[str, torch.Tensor] = {}
    gathered = _gather_flat_state(state)
    model_parallel = PT.is_model_parallel(state.model)
    mods = dict(state.model.named_modules()) if model_parallel else None
    for sname in sorted(gathered):
        for pname, view in flat.named_views(gathered[sname]):
            if model_parallel:  # same assembly as the parameter itself (a collective over the tp / ep group)
                view = PT.gather_tensor_from_ranks(state.model, pname, view, mods)
            tensors[f"{sname}.{pname}"] = view
    fsdp = getattr(state, "_fsdp", None)
    if fsdp is not None:       # master weights and moments of the parameter-sharded layers (a collective)
        for key, full in fsdp.named_state():
            tensors[key] = full.cpu() if _is_writer() else None
    if not _is_writer():
        return
    entries = write_tree(save_directory, OPTIMIZER_PREFIX, tensors)
    index_path = os.path.join(save_directory, TENSORSTORE_INDEX_NAME)
    index = {"format": "tensorstore", "version": "easydel", "prefixes": {}}
    if os.path.exists(index_path):
        with open(index_path, encoding="utf-8") as f:
            index = json.load(f)
    index.setdefault("prefixes", {})[OPTIMIZER_PREFIX] = entries
    _atomic_json(index_path, index)
    _atomic_json(os.path.join(save_directory, TX_STRUCTURE_NAME),
                 {"optimizer": state.tx.describe() if state.tx is not None else None, "step": state.step,
                  "state_names": sorted(gathered)})


def _gather_flat_state(state) -> dict[str, torch.Tensor]:
    """Full-size copies of master weights and moments (all-gathered over the sharding group when sharded)."""
    flat = state.flat
    bufs = {"master": flat.master, **flat.opt_state}
    if flat.world_size == 1:
        return {k: v for k, v in bufs.items()}
    import torch.distributed as dist

    out = {}
    group = state._dist.group if state._dist is not None else None
    for k, v in bufs.items():
        full = torch.empty(flat.numel, dtype=v.dtype, device=v.device)
        dist.all_gather_into_tensor(full, v.contiguous(), group=group)
        out[k] = full
    return out


def save_state(state, save_directory: str, float_dtype=None, save_optimizer: bool = True, step: int | None = None,
               is_temporary: bool = False, **_) -> str:
    """``EasyDeLState.save_state``: model + optimizer + metadata. ``metadata.json`` is written last, so a
    directory without it is an incomplete save."""
    step = state.step if step is None else step
    tmp_marker = os.path.join(save_directory, STATE_METADATA_NAME)
    if _is_writer() and os.path.exists(tmp_marker):
        os.remove(tmp_marker)
    save_model(state.model, save_directory, float_dtype=float_dtype, step=step)
    has_opt = bool(save_optimizer and state.flat is not None)
    if has_opt:
        save_optimizer_state(state, save_directory)
    if _is_writer():
        _atomic_json(tmp_marker, {"step": int(step), "timestamp": datetime.datetime.now().isoformat(),
                                  "is_temporary": bool(is_temporary), "has_optimizer_state": has_opt,
                                  "has_resume_model": False})
    return save_directory


# ----------------------------------------------------------------------------- reading
def is_easydel_checkpoint(path: str) -> bool:
    return os.path.exists(os.path.join(path, TENSORSTORE_INDEX_NAME)) or \
        os.path.exists(os.path.join(path, LEGACY_PARAMS_NAME))


def read_tree(root: str, prefix: str) -> dict[str, torch.Tensor]:
    with open(os.path.join(root, TENSORSTORE_INDEX_NAME), encoding="utf-8") as f:
        index = json.load(f)
    out = {}
    for ent in index.get("prefixes", {}).get(prefix, []):
        rel = ent["path"]
        key = ".".join(rel.split("/")[1:])
        out[key] = Z.read_array(os.path.join(root, rel))
    return out


def _read_safetensors(path: str) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    single = os.path.join(path, SAFETENSORS_NAME)
    index = os.path.join(path, SAFETENSORS_INDEX_NAME)
    if os.path.exists(index):
        with open(index, encoding="utf-8") as f:
            wm = json.load(f)["weight_map"]
        out = {}
        for fn in sorted(set(wm.values())):
            out.update(load_file(os.path.join(path, fn)))
        return out
    if os.path.exists(single):
        return load_file(single)
    legacy = os.path.join(path, LEGACY_PARAMS_NAME)
    if os.path.exists(legacy):
        return load_file(legacy)
    raise FileNotFoundError(f"no model weights found under {path}")


def _resolve_dir(path: str) -> str:
    """A checkpoint directory, or a training directory whose newest ``run-*`` is used."""
    if os.path.exists(os.path.join(path, CONFIG_NAME)):
        return path
    from ..trainers.base_trainer import find_latest_checkpoint

    latest = find_latest_checkpoint(path)
    if latest is None:
        raise FileNotFoundError(f"{path} holds neither a config.json nor run-* checkpoints")
    return latest


def load_config(path: str, config_kwargs: dict | None = None, **overrides):
    from ..infra.factory import _ensure_models_imported, registry

    _ensure_models_imported()
    with open(os.path.join(path, CONFIG_NAME), encoding="utf-8") as f:
        d = json.load(f)
    mtype = d.pop("model_type")
    for k in ("architectures", "transformers_version", "torch_dtype", "dtype"):
        d.pop(k, None) if k != "architectures" else None
    arch = d.pop("architectures", None)
    cls = registry.get_config(mtype)
    cfg = cls(**d)
    cfg.architectures = arch
    kw = dict(config_kwargs or {})
    kw.update({k: v for k, v in overrides.items() if v is not None})
    if kw:
        cfg.add_basic_configurations(**kw)
    return cfg


def load_weights_into(model, path: str, strict: bool = True) -> None:
    fsdp = getattr(getattr(model, "model", None), "fsdp_layers", None)
    if fsdp is not None and fsdp._materialized is None:
        fsdp.materialize()          # full parameters to load into, then back into the shards
        try:
            return load_weights_into(model, path, strict=strict)
        finally:
            fsdp.dematerialize(reshard=True)
    if os.path.exists(os.path.join(path, TENSORSTORE_INDEX_NAME)):
        PT.load_easydel_state(model, read_tree(path, MODEL_PREFIX), strict=strict)
        return
    sd = _read_safetensors(path)
    if any(k.endswith((".kernel", ".embedding")) for k in sd):
        PT.load_easydel_state(model, sd, strict=strict)
    else:
        PT.load_hf_state(model, sd, strict=strict)


def load_model(cls, path: str, dtype=torch.bfloat16, param_dtype=None, sharding_axis_dims=None,
               sharding_axis_names=None, sharding_dcn_axis_dims=None, partition_axis=None, config_kwargs=None,
               auto_shard_model: bool = True, quantization_config=None, apply_quantization: bool = False,
               from_torch: bool | None = None, device=None, strict: bool = True, **_):
    """``from_pretrained`` for a concrete model class."""
    path = _resolve_dir(path)
    cfg = load_config(path, config_kwargs, sharding_axis_dims=sharding_axis_dims,
                      sharding_axis_names=sharding_axis_names, sharding_dcn_axis_dims=sharding_dcn_axis_dims,
                      partition_axis=partition_axis)
    dtype = coerce_dtype(dtype, torch.bfloat16)
    param_dtype = coerce_dtype(param_dtype, dtype)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
    model = cls(cfg, dtype=dtype, param_dtype=param_dtype)
    load_weights_into(model, path, strict=strict)
    model.to(device)
    if quantization_config is not None and apply_quantization:
        model.quantize(quantization_config)
    if auto_shard_model and cfg.mesh.is_distributed:
        model.shard_model()
    model.eval()
    return model


def load_optimizer_state(state, path: str, tx_template=None) -> None:
    flat = state.flat
    if flat is None:
        if tx_template is None and state.tx is None:
            raise ValueError("loading optimizer state needs an optimizer (tx_template)")
        state.init_tx(tx_template or state.tx)
        flat = state.flat
    tree = read_tree(path, OPTIMIZER_PREFIX)
    names = {"master": flat.master, **flat.opt_state}
    lo, hi = flat.shard_lo, flat.shard_hi
    model_parallel = PT.is_model_parallel(state.model)
    mods = dict(state.model.named_modules()) if model_parallel else None
    for sname, buf in names.items():
        for pname, off, sz, shape, _ in flat.entries:
            key = f"{sname}.{pname}"
            if key not in tree:
                continue
            a, b = max(off, lo), min(off + sz, hi)
            if a >= b:
                continue
            full = tree[key]
            if model_parallel:  # the checkpoint holds full tensors; keep this rank's tensor-/expert-parallel piece
                full = PT.shard_tensor_for_rank(state.model, pname, full, mods).contiguous()
            src = full.reshape(-1)[a - off:b - off]
            buf[a - lo:b - lo].copy_(src.to(buf.dtype))
    fsdp = getattr(state, "_fsdp", None)
    if fsdp is not None:
        fsdp.load_named_state(tree)
    sp = os.path.join(path, TX_STRUCTURE_NAME)
    if os.path.exists(sp):
        with open(sp, encoding="utf-8") as f:
            state.step = int(json.load(f).get("step", state.step))


def load_state_into(state, path: str, tx=None, load_optimizer: bool = True) -> None:
    """Restores weights, step and (optionally) optimizer state into an existing ``EasyDeLState``."""
    load_weights_into(state.model, path)
    with open(os.path.join(path, STATE_METADATA_NAME), encoding="utf-8") as f:
        meta = json.load(f)
    state.step = int(meta.get("step", 0))
    if tx is not None and state.flat is None:
        state.init_tx(tx)
    elif state.flat is not None:
        state.flat.sync_master_from_work()
    if load_optimizer and meta.get("has_optimizer_state") and state.flat is not None:
        load_optimizer_state(state, path)
        # master weights are authoritative: refresh the working copy from them
        if not state.flat.master_is_work:
            state.flat.work[state.flat.shard_lo:state.flat.shard_hi].copy_(state.flat.master)
        state.step = int(meta.get("step", state.step))


def load_state(cls, path: str, model_class=None, tx_template=None, dtype=torch.bfloat16, param_dtype=None,
               device=None, config_kwargs=None, load_optimizer: bool = True, **kw):
    path = _resolve_dir(path)
    if model_class is None:
        from ..modules.auto import resolve_model_class

        model_class = resolve_model_class(path)
    model = load_model(model_class, path, dtype=dtype, param_dtype=param_dtype, device=device,
                       config_kwargs=config_kwargs, **kw)
    state = cls.create(model=model)
    with open(os.path.join(path, STATE_METADATA_NAME), encoding="utf-8") as f:
        meta = json.load(f)
    state.step = int(meta.get("step", 0))
    if tx_template is not None:
        state.init_tx(tx_template)
        if load_optimizer and meta.get("has_optimizer_state"):
            load_optimizer_state(state, path)
            if not state.flat.master_is_work:
                state.flat.work[state.flat.shard_lo:state.flat.shard_hi].copy_(state.flat.master)
            state.step = int(meta.get("step", 0))
    return state
