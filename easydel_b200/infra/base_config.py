"""``EasyDeLBaseConfig``: a Hugging Face ``PretrainedConfig`` with the framework's runtime fields.

The JSON this class reads and writes is the reference's ``config.json``
(easydel/infra/base_config.py:468-2947): HF model fields plus sharding axis
dims/names, attention-mechanism selection, activation-checkpoint policy, MoE
execution knobs, quantization and KV-cache settings. dtypes are stored as name
strings (``"bfloat16"``), accepted as torch dtypes, jnp-style names or short
aliases (``"bf16"``).

What differs is what the fields *drive*: the 5-axis ``(dp, fsdp, ep, tp, sp)``
description is not handed to an SPMD partitioner; it is resolved into a
:class:`easydel_b200.parallel.mesh.DeviceMesh` of process groups over one
process per GPU, and the fused kernels implement the collectives each axis implies.
"""

from __future__ import annotations

import copy
import json
import os
import typing as tp
import warnings

import torch
from transformers.configuration_utils import PretrainedConfig

from .etils import (
    DEFAULT_ATTENTION_MECHANISM,
    DEFAULT_MLA_ATTENTION_MECHANISM,
    EasyDeLGradientCheckPointers,
)

# file names of the on-disk layout (easydel/infra/base_config.py:135-178, base_state.py:117-129)
CONFIG_NAME = "config.json"
GENERATION_CONFIG_NAME = "generation_config.json"
TENSORSTORE_INDEX_NAME = "tensorstore_index.json"
CHECKPOINT_METADATA_NAME = "checkpoint_metadata.json"
STATE_METADATA_NAME = "metadata.json"
MODEL_PREFIX = "model"
OPTIMIZER_PREFIX = "tx"
SAFETENSORS_NAME = "model.safetensors"
SAFETENSORS_INDEX_NAME = "model.safetensors.index.json"
LEGACY_PARAMS_NAME = "easydel-model.parameters"
TRAINING_ARGS_NAME = "easydel-training-arguments.json"
RESUME_MODEL_DIR = "_resume_model"

DEFAULT_AXIS_NAMES = ("dp", "fsdp", "ep", "tp", "sp")
DEFAULT_AXIS_DIMS = (1, -1, 1, 1, 1)

_DTYPE_ALIASES: dict[str, torch.dtype] = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "torch.bfloat16": torch.bfloat16,
    "fp16": torch.float16, "f16": torch.float16, "float16": torch.float16, "half": torch.float16,
    "torch.float16": torch.float16,
    "fp32": torch.float32, "f32": torch.float32, "float32": torch.float32, "float": torch.float32,
    "torch.float32": torch.float32,
    "fp64": torch.float64, "f64": torch.float64, "float64": torch.float64, "double": torch.float64,
    "fp8": torch.float8_e4m3fn, "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2,
    "e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2,
    "int8": torch.int8, "uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64,
}

_DTYPE_FIELDS = ("attn_dtype", "kvdtype", "attn_softmax_dtype", "mla_attn_dtype", "mla_attn_softmax_dtype")


def coerce_dtype(spec: tp.Any, default: torch.dtype | None = None) -> torch.dtype | None:
    """Accepts torch dtypes, numpy/jax-style objects with a ``name`` and strings / aliases."""
    if spec is None:
        return default
    if isinstance(spec, torch.dtype):
        return spec
    name = getattr(spec, "name", None) or getattr(spec, "__name__", None) or str(spec)
    name = name.strip().lower().replace("jnp.", "").replace("jax.numpy.", "").replace("numpy.", "").replace("np.", "")
    if name in _DTYPE_ALIASES:
        return _DTYPE_ALIASES[name]
    raise ValueError(f"unknown dtype specification {spec!r}")


def dtype_name(dt: torch.dtype | None) -> str | None:
    return None if dt is None else str(dt).replace("torch.", "")


class PartitionAxis:
    """Names the mesh axes that each *semantic* tensor dimension is split over.

    Equivalent of ``eformer.escale.PartitionAxis`` as used by the reference
    (README.md:852-857, easydel/layers/attention/_flexible.py:861-866): batch over
    ``(fsdp, dp)``, sequence over ``sp``, heads / hidden over ``tp``, experts over ``ep``.
    Generation-mode variants cover decode, where the query sequence axis is not split.
    """

    _FIELDS = {
        "data_parallel_axis": "dp",
        "fully_sharded_data_parallel_axis": "fsdp",
        "tensor_parallel_axis": "tp",
        "sequence_parallel_axis": "sp",
        "expert_parallel_axis": "ep",
        "batch_axis": ("fsdp", "dp"),
        "sequence_axis": "sp",
        "query_sequence_axis": "sp",
        "head_axis": "tp",
        "kv_head_axis": "tp",
        "key_sequence_axis": "sp",
        "hidden_state_axis": "tp",
        "mlp_intermediate_axis": "tp",
        "vocab_axis": "tp",
        "expert_axis": "ep",
        "expert_gate_axis": None,
        "attention_dim_axis": None,
        "attention_kv_dim_axis": None,
        "bias_head_sequence_axis": None,
        "bias_key_sequence_axis": None,
        "decode_batch_axis": ("fsdp", "dp"),
        "decode_query_sequence_axis": None,
        "decode_head_axis": "tp",
        "decode_kv_head_axis": "tp",
        "decode_key_sequence_axis": "sp",
        "decode_attention_dim_axis": None,
        "decode_attention_kv_dim_axis": None,
    }
    _registered: dict[str, tuple[tp.Any, tp.Any]] = {}

    def __init__(self, **kw):
        for k, v in self._FIELDS.items():
            val = kw.pop(k, v)
            setattr(self, k, tuple(val) if isinstance(val, list) else val)
        if kw:
            raise TypeError(f"unknown PartitionAxis fields: {sorted(kw)}")

    @classmethod
    def register(cls, name: str, rule, generation_axis_rule=None) -> None:
        """Registers an extra semantic axis (the reference adds ``ATTN_DP`` this way, easydel/axis.py:24-98)."""
        cls._registered[name] = (rule, generation_axis_rule if generation_axis_rule is not None else rule)

    def resolve_axis(self, axes: tp.Sequence[str | None], mode: str = "train") -> tuple:
        """Maps semantic axis names (``"batch"``, ``"head"``...) to mesh axis names for ``mode``."""
        out = []
        gen = mode in ("decode", "generation", "insert")
        for a in axes:
            if a is None or a == "_":
                out.append(None)
                continue
            if a in self._registered:
                out.append(self._registered[a][1 if gen else 0])
                continue
            key = a if a.endswith("_axis") else f"{a}_axis"
            if gen and hasattr(self, f"decode_{key}"):
                key = f"decode_{key}"
            if not hasattr(self, key):
                raise KeyError(f"unknown semantic axis {a!r}")
            out.append(getattr(self, key))
        return tuple(out)

    def to_dict(self) -> dict:
        return {k: (list(getattr(self, k)) if isinstance(getattr(self, k), tuple) else getattr(self, k))
                for k in self._FIELDS}

    def __eq__(self, other):
        return isinstance(other, PartitionAxis) and self.to_dict() == other.to_dict()

    def __repr__(self):
        return f"PartitionAxis({self.to_dict()})"


def resolve_axis_dims(dims: tp.Sequence[int], world_size: int) -> tuple[int, ...]:
    """Replaces a single ``-1`` by whatever makes the product equal ``world_size``.

    On one device every axis collapses to 1 (easydel/infra/base_config.py:1047-1059).
    """
    dims = [int(d) for d in dims]
    if world_size == 1:
        return tuple(1 for _ in dims)
    neg = [i for i, d in enumerate(dims) if d == -1]
    if len(neg) > 1:
        raise ValueError(f"at most one -1 allowed in sharding_axis_dims, got {dims}")
    known = 1
    for d in dims:
        if d != -1:
            if d <= 0:
                raise ValueError(f"axis dims must be positive or -1, got {dims}")
            known *= d
    if neg:
        if world_size % known:
            raise ValueError(f"axis dims {dims} do not divide world size {world_size}")
        dims[neg[0]] = world_size // known
    elif known != world_size:
        raise ValueError(f"product of axis dims {dims} is {known}, world size is {world_size}")
    return tuple(dims)


class EasyDeLBaseConfig(PretrainedConfig):
    """Base of every model config. See the module docstring."""

    model_type = "easydel-base"
    #: config attribute names holding layer counts etc. are declared by subclasses

    def __init__(
        self,
        sharding_axis_dims: tp.Sequence[int] = DEFAULT_AXIS_DIMS,
        sharding_dcn_axis_dims: tp.Sequence[int] | None = None,
        sharding_axis_names: tp.Sequence[str] = DEFAULT_AXIS_NAMES,
        attn_mechanism: str = DEFAULT_ATTENTION_MECHANISM,
        decode_attn_mechanism: str | None = None,
        mla_attn_mechanism: str = DEFAULT_MLA_ATTENTION_MECHANISM,
        mla_attn_dtype=None,
        mla_attn_softmax_dtype=None,
        blocksize_k: int = 512,
        blocksize_q: int = 512,
        blocksize_b: int = 1,
        moe_tiling_size_batch: int = 4,
        moe_tiling_size_seqlen: int = 128,
        moe_tiling_size_dim: int = 128,
        partition_axis: PartitionAxis | dict | None = None,
        use_sharded_kv_caching: bool = False,
        use_sharding_constraint: bool = False,
        backend: str | None = None,
        platform: str | None = None,
        easy_method: str = "train",
        bits: int | None = None,
        scan_ring_attention: bool = True,
        scan_attention_layers: bool = False,
        use_scan_mlp: bool = False,
        scan_mlp_chunk_size: int = 1024,
        sequence_axis_name: str = "sp",
        gradient_checkpointing: str = EasyDeLGradientCheckPointers.NONE.value,
        gradient_checkpointing_targets: list[str] | None = None,
        precompute_masks: bool = True,
        lmhead_chunksize: int | None = None,
        kv_cache_quantization_config=None,
        quantization_config=None,
        use_qmm_best_config: bool = False,
        qmm_platform_override: str | None = None,
        qmm_tpu_path_override: str | None = None,
        kv_cache_sharding_sequence_axis_name: str | tuple[str, ...] = "sp",
        flash_attention_backward_pass_impl: str = "triton",
        attn_dtype=torch.bfloat16,
        kvdtype=None,
        attn_softmax_dtype=torch.float32,
        fcm_max_ratio: float = 0.0,
        fcm_min_ratio: float = 0.0,
        hardware_abstraction: bool = False,
        pallas_m_block_size: int = 128,
        pallas_k_block_size: int = 128,
        pallas_n_block_size: int = 128,
        moe_method: str = "fused_moe",
        moe_force_xla_gmm: bool = False,
        use_expert_tensor_mode: bool = False,
        use_ring_of_experts: bool = False,
        fsdp_is_ep_bound: bool = True,
        sp_is_ep_bound: bool = True,
        operation_configs: dict | None = None,
        fsdp_parameter_sharding: str = "auto",
        tp_sequence_parallel: bool = True,
        ring_attention_layout: str = "zigzag",
        ring_attention_impl: str = "auto",
        **kwargs,
    ):
        self.sharding_axis_dims = tuple(getattr(self, "sharding_axis_dims", None) or sharding_axis_dims)
        self.sharding_dcn_axis_dims = getattr(self, "sharding_dcn_axis_dims", None) or sharding_dcn_axis_dims
        if self.sharding_dcn_axis_dims is not None:
            self.sharding_dcn_axis_dims = tuple(self.sharding_dcn_axis_dims)
        self.sharding_axis_names = tuple(getattr(self, "sharding_axis_names", None) or sharding_axis_names)
        # one backend: accepted and recorded, never dispatched on
        self.backend = backend if backend is not None else ("gpu" if torch.cuda.is_available() else "cpu")
        self.platform = platform if platform is not None else ("cuda" if self.backend == "gpu" else "jax")
        self.easy_method = easy_method
        self.attn_mechanism = attn_mechanism
        self.decode_attn_mechanism = decode_attn_mechanism
        self.mla_attn_mechanism = mla_attn_mechanism
        self.blocksize_b, self.blocksize_k, self.blocksize_q = blocksize_b, blocksize_k, blocksize_q
        self.moe_tiling_size_batch = moe_tiling_size_batch
        self.moe_tiling_size_seqlen = moe_tiling_size_seqlen
        self.moe_tiling_size_dim = moe_tiling_size_dim
        if partition_axis is None:
            partition_axis = PartitionAxis()
        elif isinstance(partition_axis, dict):
            partition_axis = PartitionAxis(**partition_axis)
        self.partition_axis = partition_axis
        self.bits = bits
        self.scan_attention_layers = scan_attention_layers
        self.scan_ring_attention = scan_ring_attention
        self.use_sharded_kv_caching = use_sharded_kv_caching
        self.use_scan_mlp = use_scan_mlp
        self.scan_mlp_chunk_size = scan_mlp_chunk_size
        self.use_sharding_constraint = use_sharding_constraint
        self.sequence_axis_name = sequence_axis_name
        self.kv_cache_sharding_sequence_axis_name = kv_cache_sharding_sequence_axis_name
        self.gradient_checkpointing = str(getattr(gradient_checkpointing, "value", gradient_checkpointing) or "")
        self.gradient_checkpointing_targets = gradient_checkpointing_targets
        self.precompute_masks = precompute_masks
        if lmhead_chunksize is not None:
            if isinstance(lmhead_chunksize, bool) or not isinstance(lmhead_chunksize, int):
                raise TypeError(f"`lmhead_chunksize` must be an int when provided, got {lmhead_chunksize!r}")
            if lmhead_chunksize <= 0:
                raise ValueError("`lmhead_chunksize` must be positive when provided.")
        self.lmhead_chunksize = lmhead_chunksize
        self.kv_cache_quantization_config = kv_cache_quantization_config
        self.quantization_config = quantization_config
        self.use_qmm_best_config = bool(use_qmm_best_config)
        self.qmm_platform_override = qmm_platform_override
        self.qmm_tpu_path_override = qmm_tpu_path_override
        self.flash_attention_backward_pass_impl = flash_attention_backward_pass_impl
        self.attn_dtype = coerce_dtype(attn_dtype, torch.bfloat16)
        self.kvdtype = coerce_dtype(kvdtype, self.attn_dtype)
        self.attn_softmax_dtype = coerce_dtype(attn_softmax_dtype, torch.float32)
        self.mla_attn_dtype = coerce_dtype(mla_attn_dtype, self.attn_dtype)
        self.mla_attn_softmax_dtype = coerce_dtype(mla_attn_softmax_dtype, self.attn_softmax_dtype)
        self.fcm_max_ratio, self.fcm_min_ratio = fcm_max_ratio, fcm_min_ratio
        self.hardware_abstraction = hardware_abstraction
        self.pallas_m_block_size = pallas_m_block_size
        self.pallas_k_block_size = pallas_k_block_size
        self.pallas_n_block_size = pallas_n_block_size
        self.moe_method = moe_method
        self.moe_force_xla_gmm = moe_force_xla_gmm
        self.use_ring_of_experts = use_ring_of_experts
        self.use_expert_tensor_mode = use_expert_tensor_mode
        self.fsdp_is_ep_bound = fsdp_is_ep_bound
        self.sp_is_ep_bound = sp_is_ep_bound
        self.operation_configs = operation_configs
        # "sharded": every rank of the dp x fsdp group keeps 1/N of each decoder layer's parameters and layers are
        # gathered one at a time (parallel.fsdp); "hoisted": full bf16 weights on every rank, only the optimizer
        # state is sharded (parallel.dist_optim); "auto": hoisted while the replicas fit in device memory.
        if str(fsdp_parameter_sharding).lower() not in ("auto", "sharded", "hoisted"):
            raise ValueError(f"fsdp_parameter_sharding must be auto / sharded / hoisted, got {fsdp_parameter_sharding!r}")
        self.fsdp_parameter_sharding = str(fsdp_parameter_sharding).lower()
        # tensor-parallel dense stacks keep the residual stream sharded by token rows between their linears
        self.tp_sequence_parallel = bool(tp_sequence_parallel)
        # attn_mechanism="ring" with sp > 1: how the sequence is laid over the sp ranks (zigzag balances causal work,
        # contiguous keeps rank r's tokens adjacent) and which exchange serves it (gather = all keys / values
        # gathered, peer = remote key blocks read in place by the flash kernel, auto = peer when it applies)
        if ring_attention_layout not in ("zigzag", "contiguous"):
            raise ValueError(f"ring_attention_layout must be zigzag or contiguous, got {ring_attention_layout!r}")
        if ring_attention_impl not in ("auto", "gather", "peer"):
            raise ValueError(f"ring_attention_impl must be auto, gather or peer, got {ring_attention_impl!r}")
        self.ring_attention_layout, self.ring_attention_impl = ring_attention_layout, ring_attention_impl
        self.pretraining_tp = 1
        if self.kv_cache_quantization_config is not None and self.use_sharded_kv_caching:
            warnings.warn("`kv_cache_quantization_config` and `use_sharded_kv_caching` can't be used together "
                          "at the moment.", stacklevel=1)
        self._mesh = None
        rp = kwargs.get("rope_parameters")
        if isinstance(rp, dict) and rp.get("rope_theta") is not None and "rope_theta" in self.__dict__:
            # newer checkpoint configs keep the rotary base inside ``rope_parameters`` and have no top-level field
            self.rope_theta = rp["rope_theta"]
        super().__init__(**kwargs)

    # ------------------------------------------------------------------ mesh
    @property
    def mesh(self):
        """The process-group mesh built from ``sharding_axis_dims`` (created lazily, cached)."""
        if self.__dict__.get("_mesh") is None:
            from ..parallel.mesh import DeviceMesh

            self._mesh = DeviceMesh.from_config(self)
        return self._mesh

    def set_model_mesh(self, mesh) -> None:
        self._mesh = mesh

    def get_mesh(self):
        return self.mesh

    @staticmethod
    def create_mesh(sharding_axis_dims=DEFAULT_AXIS_DIMS, sharding_axis_names=DEFAULT_AXIS_NAMES,
                    sharding_dcn_axis_dims=None, world_size: int | None = None, **_):
        from ..parallel.mesh import DeviceMesh

        return DeviceMesh.create(sharding_axis_dims, sharding_axis_names, world_size=world_size)

    def get_partition_rules(self, *args, **kwargs):
        """``None`` = derive the rules from the layers themselves (column / row / replicated)."""
        return None

    def add_basic_configurations(self, **kw):
        """Overrides runtime fields after load (``config_kwargs`` of ``from_pretrained``)."""
        for k, v in kw.items():
            if v is None:
                continue
            if k in _DTYPE_FIELDS:
                v = coerce_dtype(v)
            if k == "partition_axis" and isinstance(v, dict):
                v = PartitionAxis(**v)
            if k in ("sharding_axis_dims", "sharding_axis_names", "sharding_dcn_axis_dims") and v is not None:
                v = tuple(v)
                self._mesh = None
            setattr(self, k, v)
        return self

    # ------------------------------------------------------------------ helpers used by models
    def get_basic_rope(self, dtype, head_size: int, rotary_dim: int | None = None, is_neox_style: bool = True,
                       base: float | None = None):
        from ..layers.rotary import get_rope

        return get_rope(head_size=head_size, rotary_dim=rotary_dim or head_size,
                        max_position=getattr(self, "max_position_embeddings", 4096),
                        base=base if base is not None else getattr(self, "rope_theta", 10000.0),
                        is_neox_style=is_neox_style, rope_scaling=getattr(self, "rope_scaling", None), dtype=dtype)

    def get_basic_causal_mask(self, length: int | None = None, device=None):
        n = length or getattr(self, "max_position_embeddings", 4096)
        return torch.ones(n, n, dtype=torch.bool, device=device).tril_()

    @property
    def granted_mask_max_position_embedding(self) -> int:
        return getattr(self, "mask_max_position_embeddings", getattr(self, "max_position_embeddings", 4096))

    @property
    def granted_freq_max_position_embedding(self) -> int:
        return getattr(self, "freq_max_position_embeddings", getattr(self, "max_position_embeddings", 4096))

    # ------------------------------------------------------------------ serialisation
    def to_dict(self) -> dict:
        # the mesh holds process groups, which cannot be deep-copied: take it out while the base class copies
        mesh = self.__dict__.pop("_mesh", None)
        try:
            d = super().to_dict()
        finally:
            self.__dict__["_mesh"] = mesh
        d.pop("_mesh", None)
        for f in _DTYPE_FIELDS:
            if f in d:
                d[f] = dtype_name(coerce_dtype(d[f])) if d[f] is not None else None
        pa = d.get("partition_axis")
        if isinstance(pa, PartitionAxis):
            d["partition_axis"] = pa.to_dict()
        for k in ("quantization_config", "kv_cache_quantization_config"):
            q = d.get(k)
            if q is not None and hasattr(q, "to_dict"):
                d[k] = q.to_dict()
        for k in ("sharding_axis_dims", "sharding_axis_names", "sharding_dcn_axis_dims"):
            if d.get(k) is not None:
                d[k] = list(d[k])
        if isinstance(d.get("operation_configs"), dict):
            d["operation_configs"] = {k: (v.to_dict() if hasattr(v, "to_dict") else v)
                                      for k, v in d["operation_configs"].items()}
        return d

    def to_diff_dict(self) -> dict:
        """Only the fields that differ from a default-constructed config of the same class."""
        full = self.to_dict()
        default = type(self)().to_dict() if self._can_default_construct() else {}
        out = {k: v for k, v in full.items() if k not in default or v != default[k]}
        out["model_type"] = self.model_type
        if full.get("architectures"):
            out["architectures"] = full["architectures"]
        return out

    def _can_default_construct(self) -> bool:
        try:
            type(self)()
            return True
        except Exception:
            return False

    def to_json_string(self, use_diff: bool = True) -> str:
        d = self.to_diff_dict() if use_diff else self.to_dict()
        # runtime dtypes of the attention op are not persisted (easydel/infra/mixins/bridge.py:618-622)
        d.pop("attn_dtype", None)
        d.pop("attn_softmax_dtype", None)
        return json.dumps(_jsonable(d), indent=2, sort_keys=True) + "\n"

    def save_pretrained(self, save_directory: str | os.PathLike, push_to_hub: bool = False, **kwargs):
        os.makedirs(save_directory, exist_ok=True)
        path = os.path.join(save_directory, CONFIG_NAME)
        tmp = path + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            f.write(self.to_json_string(use_diff=True))
        os.replace(tmp, path)
        return [path]

    def __deepcopy__(self, memo):
        mesh, self._mesh = self._mesh, None
        try:
            cls = self.__class__
            new = cls.__new__(cls)
            memo[id(self)] = new
            for k, v in self.__dict__.items():
                setattr(new, k, copy.deepcopy(v, memo))
        finally:
            self._mesh = mesh
        new._mesh = mesh
        return new


def _jsonable(x):
    if isinstance(x, dict):
        return {str(k): _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    if isinstance(x, torch.dtype):
        return dtype_name(x)
    if isinstance(x, PartitionAxis):
        return x.to_dict()
    if hasattr(x, "to_dict") and callable(x.to_dict):
        return _jsonable(x.to_dict())
    if hasattr(x, "value") and isinstance(getattr(x, "value"), (str, int, float)):
        return x.value
    return x


class EasyDeLBaseConfigDict(tp.TypedDict, total=False):
    """Typed view of the runtime overrides accepted through ``config_kwargs`` (base_config.py:401-465)."""

    sharding_axis_dims: tp.Sequence[int]
    sharding_dcn_axis_dims: tp.Sequence[int] | None
    sharding_axis_names: tp.Sequence[str]
    attn_mechanism: str
    decode_attn_mechanism: str | None
    blocksize_k: int
    blocksize_q: int
    blocksize_b: int
    partition_axis: PartitionAxis
    use_sharded_kv_caching: bool
    backend: str | None
    platform: str | None
    easy_method: str
    bits: int | None
    scan_ring_attention: bool
    scan_attention_layers: bool
    use_scan_mlp: bool
    scan_mlp_chunk_size: int
    sequence_axis_name: str
    gradient_checkpointing: str
    gradient_checkpointing_targets: list[str] | None
    lmhead_chunksize: int | None
    kv_cache_quantization_config: tp.Any
    quantization_config: tp.Any
    attn_dtype: tp.Any
    kvdtype: tp.Any
    attn_softmax_dtype: tp.Any
    moe_method: str
    use_expert_tensor_mode: bool
    use_ring_of_experts: bool
    fsdp_is_ep_bound: bool
    sp_is_ep_bound: bool
    operation_configs: dict | None
    freq_max_position_embeddings: int
    mask_max_position_embeddings: int
    hardware_abstraction: bool
