"""Parameter name / layout conversion between three conventions.

1. **internal**: this framework's module tree. Torch layout ``[out, in]``, fused projections
   (``qkv_proj``, ``gate_up_proj``), stacked experts ``[E, out, in]``.
2. **hf**: Hugging Face transformers names (``q_proj.weight`` ... per-expert modules).
3. **easydel**: the reference's checkpoint leaves (easydel/utils/parameters_transformation.py:187-279):
   ``embed*.weight -> .embedding``; LayerNorm ``.weight -> .scale`` for registered layer-norm names;
   every other ``.weight -> .kernel`` with 2-D tensors transposed to ``(in, out)``; experts stacked as
   ``experts.<proj>.kernel`` of shape ``(E, in, out)``; 1-D weights (RMSNorm) keep their shape as ``.kernel``.

``StateDictConverter`` offers the reference's entry points on top of these maps.
"""

from __future__ import annotations

import re
import typing as tp

import torch

FUSED_SPLITS: dict[str, tuple[str, ...]] = {
    "qkv_proj": ("q_proj", "k_proj", "v_proj"),
    "gate_up_proj": ("gate_proj", "up_proj"),
}

_EXPERT_RE = re.compile(r"^(.*\.)experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")


def _module_of(model, name: str):
    mod = model
    for part in name.split("."):
        mod = getattr(mod, part) if not part.isdigit() else mod[int(part)]
    return mod


# ----------------------------------------------------------------------------- internal <-> hf
def internal_to_hf(model, state: dict[str, torch.Tensor] | None = None,
                   full_shapes: bool = False) -> dict[str, torch.Tensor]:
    """Splits fused projections and unstacks experts; applies the family's ``hf_rename_out`` hook if present.
    ``full_shapes``: ``state`` holds gathered (tensor-parallel size 1) tensors, so merged outputs are split at
    their global widths rather than at this rank's."""
    state = state if state is not None else {k: v for k, v in model.state_dict().items()}
    out: dict[str, torch.Tensor] = {}
    for name, t in state.items():
        parts = name.split(".")
        leaf, mod_name = parts[-1], parts[-2] if len(parts) > 1 else ""
        prefix = ".".join(parts[:-2])
        pre = prefix + "." if prefix else ""
        keeps = getattr(model, "hf_keeps_fused", ())
        # "prefix." keeps every fused matrix under that parameter-name prefix, "prefix.:module" only that module's
        kept = mod_name in keeps or any(
            (":" in e and name.startswith(e.split(":")[0]) and mod_name == e.split(":")[1])
            or (":" not in e and "." in e and name.startswith(e)) for e in keeps)
        if mod_name in FUSED_SPLITS and t.dim() <= 2 and not kept and \
                hasattr(_module_of(model, ".".join(parts[:-1])), "local_out_splits"):
            mod = _module_of(model, ".".join(parts[:-1]))
            widths = (mod.out_splits or (t.shape[0],)) if full_shapes else mod.local_out_splits()
            for sub, chunk in zip(FUSED_SPLITS[mod_name], torch.split(t, list(widths), dim=0)):
                out[f"{pre}{sub}.{leaf}"] = chunk
        elif t.dim() == 3 and mod_name in ("gate_up_proj", "down_proj") and leaf == "weight" and \
                "experts" not in getattr(model, "hf_keeps_fused", ()):
            E = t.shape[0]
            if mod_name == "gate_up_proj":
                F = t.shape[1] // 2
                for e in range(E):
                    out[f"{pre}experts.{e}.gate_proj.weight"] = t[e, :F]
                    out[f"{pre}experts.{e}.up_proj.weight"] = t[e, F:]
            else:
                for e in range(E):
                    out[f"{pre}experts.{e}.down_proj.weight"] = t[e]
        else:
            out[name] = t
    hook = getattr(model, "hf_rename_out", None)
    if hook is not None:
        out = hook(out)
    return out


def hf_to_internal(model, hf_state: dict[str, torch.Tensor], strict: bool = True) -> dict[str, torch.Tensor]:
    """Inverse of :func:`internal_to_hf`: concatenates q/k/v and gate/up, stacks experts."""
    hook = getattr(model, "hf_rename_in", None)
    if hook is not None:
        hf_state = hook(dict(hf_state))
    target = model.state_dict()
    out: dict[str, torch.Tensor] = {}
    missing = []
    for name, ref in target.items():
        parts = name.split(".")
        leaf, mod_name = parts[-1], parts[-2] if len(parts) > 1 else ""
        prefix = ".".join(parts[:-2])
        pre = prefix + "." if prefix else ""
        if name in hf_state:
            out[name] = hf_state[name]
        elif mod_name in FUSED_SPLITS and ref.dim() <= 2:
            keys = [f"{pre}{sub}.{leaf}" for sub in FUSED_SPLITS[mod_name]]
            if all(k in hf_state for k in keys):
                out[name] = torch.cat([hf_state[k] for k in keys], dim=0)
            elif f"{pre}{mod_name}.{leaf}" in hf_state:
                out[name] = hf_state[f"{pre}{mod_name}.{leaf}"]
            else:
                missing.append(name)
        elif ref.dim() == 3 and mod_name in ("gate_up_proj", "down_proj"):
            # all experts are assembled here; an expert-parallel model keeps its own slice afterwards
            try:
                block = _module_of(model, prefix) if prefix else model
            except (AttributeError, IndexError):
                block = None
            E = ref.shape[0] * max(1, getattr(block, "ep_size", 1))
            try:
                if mod_name == "gate_up_proj":
                    out[name] = torch.stack([torch.cat([hf_state[f"{pre}experts.{e}.gate_proj.weight"],
                                                        hf_state[f"{pre}experts.{e}.up_proj.weight"]], dim=0)
                                             for e in range(E)])
                else:
                    out[name] = torch.stack([hf_state[f"{pre}experts.{e}.down_proj.weight"] for e in range(E)])
            except KeyError:
                # HF checkpoints with already-fused expert tensors [E, in, 2F] / [E, F, out]
                fused_key = f"{pre}experts.{mod_name}"
                if fused_key in hf_state:
                    t = hf_state[fused_key]
                    transposed = getattr(model, "hf_fused_experts_transposed", None)
                    if transposed is None:
                        transposed = tuple(t.shape[1:]) != tuple(ref.shape[1:])
                    out[name] = t.transpose(1, 2) if transposed else t
                else:
                    missing.append(name)
        else:
            missing.append(name)
    if missing and strict:
        raise KeyError(f"checkpoint is missing parameters: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    return out


# ----------------------------------------------------------------------------- hf <-> easydel
def _is_embedding(key: str, embedding_layer_names: tp.Sequence[str]) -> bool:
    return any(n in key for n in embedding_layer_names)


DEFAULT_EMBEDDING_NAMES = ("embed_tokens", "embed_positions", "wte", "wpe", "word_embeddings", "embed_in")


def hf_to_easydel(hf_state: dict[str, torch.Tensor], embedding_layer_names: tp.Sequence[str] | None = None,
                  layernorm_names: tp.Sequence[str] | None = None) -> dict[str, torch.Tensor]:
    """Applies the leaf renaming / transposition rules and stacks per-expert weights."""
    emb = tuple(embedding_layer_names or DEFAULT_EMBEDDING_NAMES)
    lns = tuple(layernorm_names or ())
    out: dict[str, torch.Tensor] = {}
    experts: dict[tuple[str, str], dict[int, torch.Tensor]] = {}
    for key, t in hf_state.items():
        m = _EXPERT_RE.match(key)
        if m:
            experts.setdefault((m.group(1), m.group(3)), {})[int(m.group(2))] = t
            continue
        if key.endswith(".weight") and _is_embedding(key, emb):
            out[key[: -len(".weight")] + ".embedding"] = t
        elif key.endswith(".weight") and any(n in key for n in lns):
            out[key[: -len(".weight")] + ".scale"] = t
        elif key.endswith(".weight"):
            nk = key[: -len(".weight")] + ".kernel"
            if t.dim() == 2:
                t = t.t()
            elif t.dim() == 3:
                t = t.permute(2, 1, 0)
            elif t.dim() == 4:
                t = t.permute(2, 3, 1, 0)
            out[nk] = t
        else:
            out[key] = t
    for (pre, proj), byidx in experts.items():
        E = max(byidx) + 1
        stacked = torch.stack([byidx[e] for e in range(E)])  # (E, out, in)
        out[f"{pre}experts.{proj}.kernel"] = stacked.permute(0, 2, 1)  # (E, in, out)
    return out


def easydel_to_hf(ed_state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for key, t in ed_state.items():
        m = re.match(r"^(.*\.)experts\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.kernel$", key)
        if m and t.dim() == 3:
            for e in range(t.shape[0]):
                out[f"{m.group(1)}experts.{e}.{m.group(2)}.weight"] = t[e].t()
            continue
        if key.endswith(".embedding"):
            out[key[: -len(".embedding")] + ".weight"] = t
        elif key.endswith(".scale"):
            out[key[: -len(".scale")] + ".weight"] = t
        elif key.endswith(".kernel"):
            nk = key[: -len(".kernel")] + ".weight"
            if t.dim() == 2:
                t = t.t()
            elif t.dim() == 3:
                t = t.permute(2, 1, 0)
            elif t.dim() == 4:
                t = t.permute(3, 2, 0, 1)
            out[nk] = t
        else:
            out[key] = t
    return out


def model_to_easydel_state(model) -> dict[str, torch.Tensor]:
    """Internal module tree -> reference checkpoint leaves (what ``save_pretrained`` writes)."""
    reg_ln = _layernorm_names(model)
    if is_model_parallel(model):  # a collective: every rank assembles the full tensors
        return hf_to_easydel(internal_to_hf(model, gather_internal_state(model), full_shapes=True),
                             layernorm_names=reg_ln)
    return hf_to_easydel(internal_to_hf(model), layernorm_names=reg_ln)


def load_easydel_state(model, ed_state: dict[str, torch.Tensor], strict: bool = True) -> None:
    load_hf_state(model, easydel_to_hf(ed_state), strict=strict)


def load_hf_state(model, hf_state: dict[str, torch.Tensor], strict: bool = True) -> None:
    internal = hf_to_internal(model, hf_state, strict=strict)
    if is_model_parallel(model):
        internal = shard_internal_state_for_tp(model, internal)
    with torch.no_grad():
        own = dict(model.named_parameters())
        own.update(dict(model.named_buffers()))
        for k, v in internal.items():
            if k not in own:
                continue
            if own[k].shape != v.shape:
                raise ValueError(f"shape mismatch for {k}: model {tuple(own[k].shape)} vs checkpoint {tuple(v.shape)}")
            own[k].copy_(v.to(own[k].dtype))


def _layernorm_names(model) -> tuple[str, ...]:
    from ..infra.factory import registry

    task = getattr(model, "_model_task", None)
    mtype = getattr(model, "_model_type", None)
    try:
        reg = registry.get_module_registration(task, mtype)
        return tuple(reg.layernorm_names or ())
    except Exception:
        return ()


_EXPERT_ALIASES = (("gate_proj", "up_proj", "down_proj"), ("w1", "w3", "w2"))


def _adapt_to_hf_module_names(sd: dict[str, torch.Tensor], expected: dict[str, torch.Tensor]):
    """Checkpoint-format names -> the in-memory names of the installed ``transformers`` version.

    Recent ``transformers`` keeps MoE experts as stacked ``experts.gate_up_proj`` / ``experts.down_proj``
    tensors (and renames Mixtral's ``block_sparse_moe`` to ``mlp``) while checkpoints on disk keep the
    per-expert modules; ``from_pretrained`` converts on load, ``load_state_dict`` does not.
    """
    out = dict(sd)
    for key, ref in expected.items():
        if key in out:
            continue
        alt = key.replace(".mlp.", ".block_sparse_moe.")
        if alt in out:
            out[key] = out.pop(alt)
            continue
        if not (key.endswith("experts.gate_up_proj") or key.endswith("experts.down_proj")):
            continue
        base = key.rsplit(".", 1)[0]
        for prefix in (base, base.replace(".mlp.", ".block_sparse_moe.")):
            for g, u, d in _EXPERT_ALIASES:
                if f"{prefix}.0.{d}.weight" not in out:
                    continue
                E = ref.shape[0]
                if key.endswith("gate_up_proj"):
                    t = torch.stack([torch.cat([out.pop(f"{prefix}.{e}.{g}.weight"),
                                                out.pop(f"{prefix}.{e}.{u}.weight")], 0) for e in range(E)])
                else:
                    t = torch.stack([out.pop(f"{prefix}.{e}.{d}.weight") for e in range(E)])
                out[key] = t if tuple(t.shape) == tuple(ref.shape) else t.transpose(1, 2).contiguous()
                break
            if key in out:
                break
    return out


class StateDictConverter:
    """Reference-named facade (easydel/utils/parameters_transformation.py:117-700)."""

    @staticmethod
    def huggingface_to_easydel(state_dict, *, embedding_layer_names=None, layernorm_names=None, **_):
        return hf_to_easydel(state_dict, embedding_layer_names, layernorm_names)

    @staticmethod
    def easydel_to_huggingface(state_dict, **_):
        return easydel_to_hf(state_dict)


class ModelConverter:
    @staticmethod
    def easydel_to_huggingface(model, base_hf_auto_class=None, dtype=torch.float32, **_):
        """Builds the matching ``transformers`` model on CPU and loads the converted weights into it."""
        import transformers

        hf_cfg_cls = transformers.CONFIG_MAPPING[model.config.model_type]
        hf_defaults = hf_cfg_cls().to_dict()
        own_keys = set(getattr(model.config, "hf_config_keys", ())) | {"rope_scaling", "head_dim", "rope_theta"}
        cfg_dict = {k: v for k, v in model.config.to_dict().items()
                    if (k in hf_defaults or k in own_keys) and not (v is None and k not in hf_defaults)}
        spec = getattr(model, "spec", None)
        if getattr(model.config, "layer_types", None):
            cfg_dict["layer_types"] = list(model.config.layer_types)      # the family's own vocabulary
        elif "layer_types" in hf_defaults and spec is not None and spec.layer_types is not None:
            cfg_dict["layer_types"] = [{"sliding": "sliding_attention", "linear": "linear_attention"}.get(
                t, "full_attention") for t in spec.layer_types]
        hf_cfg = hf_cfg_cls(**cfg_dict)
        auto = base_hf_auto_class or transformers.AutoModelForCausalLM
        hf_model = auto.from_config(hf_cfg).to(dtype)
        sd = {k: v.detach().to("cpu", dtype) for k, v in internal_to_hf(model).items()}
        sd = _adapt_to_hf_module_names(sd, hf_model.state_dict())
        missing, unexpected = hf_model.load_state_dict(sd, strict=False)
        bad = [m for m in missing if "rotary" not in m and "inv_freq" not in m and not
               (m == "lm_head.weight" and getattr(hf_cfg, "tie_word_embeddings", False))]
        if bad:
            raise KeyError(f"conversion left HF parameters unset: {bad[:8]}")
        return hf_model

    @staticmethod
    def huggingface_to_easydel(hf_model, model_class, config=None, dtype=torch.bfloat16, param_dtype=None, device=None):
        from ..infra.factory import registry

        cfg = config
        if cfg is None:
            cfg_cls = registry.get_config(hf_model.config.model_type)
            cfg = cfg_cls(**{k: v for k, v in hf_model.config.to_dict().items()
                             if k not in ("architectures", "model_type", "transformers_version", "dtype",
                                          "torch_dtype")})
        model = model_class(cfg, dtype=dtype, param_dtype=param_dtype or dtype)
        load_hf_state(model, hf_model.state_dict())
        if device is not None:
            model.to(device)
        return model


class TensorConverter:
    @staticmethod
    def convert_pytorch_to_numpy(t: torch.Tensor):
        import numpy as np

        if t.dtype == torch.bfloat16:
            import ml_dtypes

            return t.detach().cpu().view(torch.int16).numpy().view(ml_dtypes.bfloat16)
        return t.detach().cpu().numpy()


def _parallel_owner(model, name: str, mods: dict | None = None):
    """(module, leaf, kind) for a parameter name: kind is "column" / "row" (tensor-parallel linear of size > 1),
    "ep" (per-rank expert weights) or None (replicated)."""
    mods = mods if mods is not None else dict(model.named_modules())
    mod_name, _, leaf = name.rpartition(".")
    mod = mods.get(mod_name)
    if mod is None:
        return None, leaf, None
    style = getattr(mod, "parallel_style", None)
    if getattr(mod, "tp_size", 1) > 1 and style in ("column", "row"):
        return mod, leaf, style
    param = getattr(mod, leaf, None)
    if getattr(param, "_ep_local", False):
        block = mods.get(mod_name.rpartition(".")[0])
        if block is not None and getattr(block, "ep_size", 1) > 1:
            return block, leaf, "ep"
    return mod, leaf, None


def shard_tensor_for_rank(model, name: str, t: torch.Tensor, mods: dict | None = None) -> torch.Tensor:
    """The piece of a full (tp = ep = 1) tensor that this rank's parameter ``name`` holds."""
    mod, leaf, kind = _parallel_owner(model, name, mods)
    if kind is None:
        return t
    if kind == "ep":
        n = mod.num_local_experts
        return t[mod.ep_rank * n:(mod.ep_rank + 1) * n]
    tp_size, r = mod.tp_size, mod.tp_rank
    if kind == "row":
        if leaf == "weight":
            c = t.shape[1] // tp_size
            return t[:, r * c:(r + 1) * c]
        return t
    local = mod.local_out_splits()
    if len(local) == 1:
        c = t.shape[0] // tp_size
        return t[r * c:(r + 1) * c]
    # merged outputs: infer the full widths from the tensor (q is exact; k / v may be replicated)
    q_full = local[0] * tp_size
    rest = (t.shape[0] - q_full) // (len(local) - 1)
    full_widths = [q_full] + [rest] * (len(local) - 1)
    pieces, o = [], 0
    for lw, fw in zip(local, full_widths):
        chunk = t[o:o + fw]
        if fw == lw * tp_size:
            pieces.append(chunk[r * lw:(r + 1) * lw])
        else:  # fewer KV heads than ranks: pick the head group this rank's queries use
            n_groups = fw // lw
            gi = r * n_groups // tp_size
            pieces.append(chunk[gi * lw:(gi + 1) * lw])
        o += fw
    out = torch.cat(pieces, dim=0)
    assert out.shape[0] == sum(local)
    return out


def gather_tensor_from_ranks(model, name: str, t: torch.Tensor, mods: dict | None = None) -> torch.Tensor:
    """Inverse of :func:`shard_tensor_for_rank`: the full tensor, assembled from the tensor- / expert-parallel
    group's shards. A collective: every rank of that group must call it for the same names in the same order."""
    import torch.distributed as dist

    mod, leaf, kind = _parallel_owner(model, name, mods)
    if kind is None or (kind == "row" and leaf != "weight"):
        return t
    group = mod.ep_group if kind == "ep" else mod.tp_group
    world = mod.ep_size if kind == "ep" else mod.tp_size
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous(), group=group)
    if kind == "ep":
        return torch.cat(parts, dim=0)
    if kind == "row":
        return torch.cat(parts, dim=1)
    local = mod.local_out_splits()
    if len(local) == 1:
        return torch.cat(parts, dim=0)
    pieces, o = [], 0
    for lw in local:  # each merged output is contiguous over the ranks in the full tensor
        pieces.extend(part[o:o + lw] for part in parts)
        o += lw
    return torch.cat(pieces, dim=0)


def is_model_parallel(model) -> bool:
    """True when some parameter of the model is a tensor- or expert-parallel shard."""
    for mod in model.modules():
        if getattr(mod, "tp_size", 1) > 1 and getattr(mod, "parallel_style", None) in ("column", "row"):
            return True
        if getattr(mod, "ep_size", 1) > 1:
            return True
    return False


def gather_internal_state(model, state: dict[str, torch.Tensor] | None = None) -> dict[str, torch.Tensor]:
    """The model's state dict with every tensor- / expert-parallel shard replaced by the full tensor
    (a collective over those groups; the result is identical on every rank)."""
    state = state if state is not None else dict(model.state_dict())
    if not is_model_parallel(model):
        return state
    mods = dict(model.named_modules())
    return {k: gather_tensor_from_ranks(model, k, v, mods) for k, v in state.items()}


def shard_internal_state_for_tp(model, full_state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Cuts a full (tensor- and expert-parallel size 1) internal state dict down to what this rank's model holds.

    Column-parallel weights keep this rank's rows of every merged output (q / k / v, gate / up), row-parallel
    weights keep this rank's input columns, expert stacks keep this rank's experts. When there are fewer KV
    heads than ranks, every rank keeps the KV head its query heads belong to.
    """
    mods = dict(model.named_modules())
    return {name: shard_tensor_for_rank(model, name, t, mods) for name, t in full_state.items()}
