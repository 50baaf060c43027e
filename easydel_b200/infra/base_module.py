"""``EasyDeLBaseModule``: the ``torch.nn.Module`` base every model derives from.

Public behaviour follows easydel/infra/base_module.py:179-3091 where it makes sense outside a
tracing compiler: config + dtype bookkeeping, ``compute_loss``, ``flops_per_token``, LoRA
apply / merge / unwrap, quantisation hook, shard / gather through the parallel runtime,
``lazy_init`` (shape-only construction on the meta device), ``to_state``. Saving / loading
lives in :class:`easydel_b200.infra.mixins.bridge.EasyBridgeMixin`, generation in
:class:`easydel_b200.infra.mixins.generation.EasyGenerationMixin`.
"""

from __future__ import annotations

import contextlib
import re
import typing as tp

import torch
from torch import nn

from .base_config import EasyDeLBaseConfig, coerce_dtype
from .loss_utils import LossConfig, LossMetrics
from .mixins.bridge import EasyBridgeMixin
from .mixins.generation import EasyGenerationMixin
from .mixins.operation_cache import OperationCacheMixin


class EasyDeLBaseModule(nn.Module, EasyBridgeMixin, EasyGenerationMixin, OperationCacheMixin):
    config_class: type[EasyDeLBaseConfig] = EasyDeLBaseConfig
    base_model_prefix: str = "model"
    _model_task: str | None = None
    _model_type: str | None = None
    loss_type: str | None = None

    def __init__(self, config: EasyDeLBaseConfig, dtype: tp.Any = torch.bfloat16, param_dtype: tp.Any = None,
                 precision: tp.Any = None, rngs: tp.Any = None):
        super().__init__()
        self.config = config
        self.dtype = coerce_dtype(dtype, torch.bfloat16)
        self.param_dtype = coerce_dtype(param_dtype, self.dtype)
        self.precision = precision
        self._seed = _seed_from(rngs)

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def lazy_init(cls, config, dtype=torch.bfloat16, param_dtype=None, **kw):
        """Builds the module on the meta device: shapes and dtypes only, no storage."""
        with torch.device("meta"):
            return cls(config=config, dtype=dtype, param_dtype=param_dtype, **kw)

    @classmethod
    def sequential_init(cls, config, dtype=torch.bfloat16, param_dtype=None, device=None, seed: int = 0, **kw):
        """Random-initialises directly on ``device`` (used by the benchmarks: no checkpoint, no network)."""
        gen_state = torch.random.get_rng_state()
        torch.manual_seed(seed)
        try:
            ctx = torch.device(device) if device is not None else contextlib.nullcontext()
            with ctx:
                model = cls(config=config, dtype=dtype, param_dtype=param_dtype, **kw)
        finally:
            torch.random.set_rng_state(gen_state)
        return model

    # ------------------------------------------------------------------ introspection
    @property
    def model_task(self) -> str | None:
        return self._model_task

    @property
    def model_type(self) -> str | None:
        return self._model_type or getattr(self.config, "model_type", None)

    @property
    def mesh(self):
        return self.config.mesh

    @property
    def parameters_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    @property
    def device(self) -> torch.device:
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")

    def half(self, change_runtime_dtype: bool = True):
        self.to(torch.float16)
        if change_runtime_dtype:
            self.dtype = torch.float16
        return self

    def float(self, change_runtime_dtype: bool = True):
        self.to(torch.float32)
        if change_runtime_dtype:
            self.dtype = torch.float32
        return self

    def flops_per_token(self, sequence_length: int | None = None, include_loss: bool = True,
                        include_backward: bool = False) -> float:
        """Analytic FLOPs per token: 2 * (matmul params) + attention score/value terms
        (the model of easydel/infra/base_module.py:2564-2639)."""
        cfg = self.config
        L = getattr(cfg, "num_hidden_layers", 0)
        H = getattr(cfg, "hidden_size", 0)
        heads = getattr(cfg, "num_attention_heads", 1)
        hd = getattr(cfg, "head_dim", None) or (H // max(heads, 1))
        T = sequence_length or getattr(cfg, "max_position_embeddings", 2048)
        embed = 0
        for n, p in self.named_parameters():
            if "embed_tokens" in n or "wte" in n or "wpe" in n:
                embed += p.numel()
        tied = getattr(cfg, "tie_word_embeddings", False)
        matmul_params = self.parameters_count - embed
        if tied and include_loss:
            matmul_params += getattr(cfg, "vocab_size", 0) * H
        k = getattr(cfg, "num_experts_per_tok", None)
        E = getattr(cfg, "num_experts", None) or getattr(cfg, "num_local_experts", None) or \
            getattr(cfg, "n_routed_experts", None)
        if k and E:
            expert_params = sum(p.numel() for n, p in self.named_parameters()
                                if ".experts." in n or ("mlp.gate_up_proj" in n and p.dim() == 3)
                                or ("mlp.down_proj" in n and p.dim() == 3))
            matmul_params -= expert_params * (1 - k / E)
        flops = 2.0 * matmul_params + 4.0 * L * heads * hd * T * 0.5
        if include_backward:
            flops *= 3.0
        return float(flops)

    # ------------------------------------------------------------------ loss
    def compute_loss(self, *, labels: torch.Tensor | None = None, loss_config: LossConfig | None = None,
                     loss_kwargs: dict | None = None, loss_scale: float = 1.0, **batch):
        """Runs the model and its task loss; returns ``(outputs, LossMetrics)``.

        Batch keys the model's ``forward`` does not accept are dropped, as the reference does
        (easydel/infra/base_module.py:2757-2761).
        """
        import inspect

        sig = inspect.signature(self.forward).parameters
        accepts_kw = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.values())
        call = {k: v for k, v in batch.items() if accepts_kw or k in sig}
        if labels is None:
            labels = batch.get("input_ids")
        return self._compute_task_loss(labels, loss_config or LossConfig(), loss_scale, call, loss_kwargs or {})

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        raise NotImplementedError(f"{type(self).__name__} does not define a task loss")

    # ------------------------------------------------------------------ activation checkpointing
    def gradient_checkpointing_policy(self) -> str:
        return str(getattr(self.config, "gradient_checkpointing", "") or "")

    def remat_policy(self):
        """The activation save policy of this model's layers (``ops.remat.SavePolicy``), from
        ``config.gradient_checkpointing`` and, for the name-based policies, ``config.gradient_checkpointing_targets``
        (the names to save, or to exclude for the ``..._except_these_names`` policies)."""
        from ..ops import remat

        key = (self.gradient_checkpointing_policy(), tuple(getattr(self.config, "gradient_checkpointing_targets",
                                                                   None) or ()))
        cached = getattr(self, "_remat_policy", None)
        if cached is None or cached[0] != key:
            targets = list(key[1]) or None
            cached = (key, remat.get_policy(key[0], save_names=targets, exclude_names=targets))
            object.__setattr__(self, "_remat_policy", cached)
        return cached[1]

    # ------------------------------------------------------------------ parallel runtime hooks
    def shard_model(self, partition_rules=None, mesh=None, **_):
        """Places parameters according to the mesh. With one rank this is a no-op; with several the
        FSDP / TP / EP runtime in :mod:`easydel_b200.parallel` owns the placement."""
        from ..parallel.runtime import place_model

        return place_model(self, mesh or self.config.mesh)

    def gather_model(self, **_):
        from ..parallel.runtime import gather_model

        return gather_model(self)

    fully_shard = shard_model
    fully_gather = gather_model

    def resolve_shardings_automatically(self) -> tuple[tuple[str, tuple], ...]:
        """Partition rules ``(regex, spec)`` derived from each layer's parallel style: column kernels
        ``("fsdp","tp")``, row kernels ``("tp","fsdp")``, stacked experts led by ``"ep"``, everything
        else replicated; layer indices generalised to ``\\d+`` and a catch-all appended
        (easydel/infra/base_module.py:1181-1286)."""
        rules: dict[str, tuple] = {}
        for mod_name, mod in self.named_modules():
            style = getattr(mod, "parallel_style", None)
            if style is None or not hasattr(mod, "weight"):
                continue
            pat = re.sub(r"\.\d+\.", r".\\d+.", mod_name)
            w = getattr(mod, "weight")
            if w is None:
                continue
            if w.dim() == 3:
                spec = ("ep", "fsdp", "tp") if style == "column" else ("ep", "tp", "fsdp")
            elif style == "column":
                spec = ("fsdp", "tp")
            elif style == "row":
                spec = ("tp", "fsdp")
            else:
                spec = ()
            rules[pat + r"\.(weight|kernel|embedding)"] = spec
            if getattr(mod, "bias", None) is not None:
                rules[pat + r"\.bias"] = ("tp",) if style == "column" else ()
        out = tuple(rules.items()) + ((".*", ()),)
        return out

    # ------------------------------------------------------------------ state
    def to_state(self, state_class=None, **kw):
        from .base_state import EasyDeLState

        return (state_class or EasyDeLState).create(model=self, **kw)

    # ------------------------------------------------------------------ LoRA
    def apply_lora_to_layers(self, lora_rank: int, lora_pattern: str | None = None, lora_alpha: float | None = None,
                             lora_dropout: float = 0.0, verbose: bool = False, **_):
        """Wraps every linear whose qualified name matches ``lora_pattern`` (regex) in an ``eLoRA``."""
        from ..layers.linears import ParallelLinear, eLoRA

        pat = re.compile(lora_pattern or ".*(qkv_proj|o_proj|gate_up_proj|down_proj).*")
        for p in self.parameters():
            p.requires_grad_(False)
        n = 0
        for parent_name, parent in list(self.named_modules()):
            for child_name, child in list(parent.named_children()):
                full = f"{parent_name}.{child_name}" if parent_name else child_name
                if isinstance(child, ParallelLinear) and pat.search(full):
                    setattr(parent, child_name, eLoRA(child, lora_rank, lora_alpha, lora_dropout))
                    n += 1
        if n == 0:
            raise ValueError(f"lora_pattern {lora_pattern!r} matched no linear layer")
        return self

    def merge_lora_params(self):
        from ..layers.linears import eLoRA

        for parent in list(self.modules()):
            for child_name, child in list(parent.named_children()):
                if isinstance(child, eLoRA):
                    setattr(parent, child_name, child.merge())
        return self

    def unwrap_lora_to_layers(self, verbose: bool = False):
        from ..layers.linears import eLoRA

        for parent in list(self.modules()):
            for child_name, child in list(parent.named_children()):
                if isinstance(child, eLoRA):
                    setattr(parent, child_name, child.unwrap())
        return self

    def split_lora_params(self) -> dict[str, torch.Tensor]:
        return {n: p for n, p in self.named_parameters() if ".lora_a" in n or ".lora_b" in n}

    # ------------------------------------------------------------------ quantisation
    def quantize(self, quantization_config=None, apply_quantization: bool = True, verbose: bool = False, **kw):
        if quantization_config is None or not apply_quantization:
            return self
        from ..layers.quantization import EasyQuantizer

        return EasyQuantizer(quantization_config).apply_quantization(self, verbose=verbose)

    # ------------------------------------------------------------------ torch interop
    def to_torch(self, **kw):
        """Instantiates the matching Hugging Face model and copies the weights into it."""
        from ..utils.parameters_transformation import ModelConverter

        return ModelConverter.easydel_to_huggingface(self, **kw)

    def __repr__(self):
        base = super().__repr__()
        return base


def _seed_from(rngs) -> int:
    if rngs is None:
        return 0
    if isinstance(rngs, int):
        return rngs
    for attr in ("seed", "default"):
        v = getattr(rngs, attr, None)
        if isinstance(v, int):
            return v
    return 0
