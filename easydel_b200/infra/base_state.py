"""``EasyDeLState``: model + optimizer + step, with the optimizer step and (de)serialisation.

Counterpart of easydel/infra/base_state.py:253-1929. ``tx`` is a
:class:`easydel_b200.optimizers.FlatOptimizer`; ``opt_state`` lives in flat fp32 buffers owned by
:class:`easydel_b200.parallel.flat.FlatParams`. ``apply_gradients`` consumes the gradients that
the backward pass accumulated into ``param.main_grad``: global-norm computation, clipping,
non-finite guard, the optimizer update, the bf16 working-copy refresh and gradient zeroing are
a handful of kernel launches over the flat buffers (one fused launch per buffer for AdamW). With
more than one rank the same call runs the fused reduce-scatter + update + all-gather path of
:mod:`easydel_b200.parallel.dist_optim`.
"""

from __future__ import annotations

import os
import typing as tp

import torch

from ..optimizers import FlatOptimizer
from ..parallel.flat import FlatParams


class EasyDeLState:
    def __init__(self, model, step: int = 0, tx: FlatOptimizer | None = None, flat: FlatParams | None = None):
        self.model = model
        self.step = int(step)
        self.tx = tx
        self.flat = flat
        self._sumsq = None
        self.last_grad_norm: torch.Tensor | None = None
        self._dist = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, model, tx: FlatOptimizer | None = None, step: int = 0, init_opt_state: bool = False, **_):
        st = cls(model=model, step=step)
        if tx is not None and init_opt_state:
            st.init_tx(tx)
        elif tx is not None:
            st.tx = tx
        return st

    def init_tx(self, tx: FlatOptimizer, partition_rules=None, no_decay_patterns: tp.Sequence[str] = ()):
        """Creates the flat storage and the optimizer state for ``tx`` (sharded when the mesh says so)."""
        self.tx = tx
        mesh = getattr(self.model.config, "mesh", None)
        world = mesh.axis_size(("dp", "fsdp")) if mesh is not None and mesh.is_distributed else 1
        self._fsdp = None
        if world > 1:
            from ..parallel.dist_optim import DistributedFlat

            param_filter = None
            if self._wants_sharded_parameters(world):
                # the decoder layers keep 1/world of their parameters per rank (parallel.fsdp); embeddings, final
                # norm and LM head stay with the optimizer-sharded flat storage below
                from ..parallel.fsdp import ShardedLayers

                backbone = self.model.model
                self._fsdp = ShardedLayers(backbone.layers, mesh, prefix="model.layers",
                                           no_decay_patterns=no_decay_patterns)
                backbone.fsdp_layers = self._fsdp
                self._fsdp.opt_state = tx.init_state(self._fsdp.master)
                param_filter = lambda n, p: not n.startswith("model.layers.")  # noqa: E731
            self._dist = DistributedFlat(self.model, mesh, no_decay_patterns=no_decay_patterns,
                                         param_filter=param_filter)
            self.flat = self._dist.flat
        else:
            self.flat = FlatParams(self.model, no_decay_patterns=no_decay_patterns)
        self.flat.opt_state = tx.init_state(self.flat.master)
        return self

    def _wants_sharded_parameters(self, world: int) -> bool:
        """``config.fsdp_parameter_sharding``: "sharded" keeps 1/N of every decoder layer per rank and gathers
        layer by layer, "hoisted" keeps full bf16 weights and fp32 gradients on every rank and shards only the
        optimizer state, "auto" (default) takes "hoisted" while those replicas fit comfortably in device memory."""
        cfg = getattr(self.model, "config", None)
        mode = str(getattr(cfg, "fsdp_parameter_sharding", "auto")).lower()
        layers = getattr(getattr(self.model, "model", None), "layers", None)
        if mode == "hoisted" or layers is None or len(layers) == 0 or not hasattr(self.model.model, "_run_layer"):
            return False
        if mode == "sharded":
            return True
        n = sum(p.numel() for p in self.model.parameters())
        replicas = n * (2 + 4)                       # bf16 weights + fp32 gradient buffer on every rank
        dev = next(self.model.parameters()).device
        if dev.type != "cuda":
            return False
        total = torch.cuda.get_device_properties(dev).total_memory
        return replicas + n * 12 // world > 0.6 * total

    @property
    def opt_state(self):
        return None if self.flat is None else self.flat.opt_state

    @property
    def size(self) -> int:
        n = sum(p.numel() * p.element_size() for p in self.model.parameters())
        if self.flat is not None:
            n += sum(t.numel() * t.element_size() for t in self.flat.opt_state.values())
        return n

    @property
    def graphstate(self):
        return dict(self.model.named_parameters())

    # ------------------------------------------------------------------ the optimizer step
    @torch.no_grad()
    def apply_gradients(self, *, grad_scale: float = 1.0, zero_grad: bool = True):
        """One optimizer update from the accumulated ``main_grad`` buffers.

        ``grad_scale`` multiplies the gradients first (``1/accumulation`` when the loss was not
        pre-scaled). Returns the (device) global gradient norm after scaling, before clipping.
        """
        if self.flat is None or self.tx is None:
            raise RuntimeError("call init_tx(tx) before apply_gradients")
        flat, tx = self.flat, self.tx
        flat.fold_param_grads()
        self.step += 1
        lr = tx.lr_at(self.step - 1)
        if getattr(self.model, "sp_partial_grads", False):
            # the backward ran on sequence-sharded activations (see parallel.tp): complete the partial gradients
            mesh = self._model_mesh()
            if mesh is not None and mesh.tp > 1:
                flat.sync_partial_grads_over_tp(mesh.get_group("tp"))
            self.model.sp_partial_grads = False
        if getattr(self.model, "cp_partial_grads", False):
            # the batch's sequence dimension was sharded over the ``sp`` axis: every gradient is a partial sum
            mesh = self._model_mesh()
            if mesh is not None and mesh.sp > 1:
                if self._fsdp is not None:
                    raise NotImplementedError("sequence-sharded batches with parameter-sharded layers")
                import torch.distributed as dist

                dist.all_reduce(flat.grad, group=mesh.get_group("sp"))
            self.model.cp_partial_grads = False
        ep_group, ep = self._expert_parallel()
        if ep > 1:
            # replicated parameters: sum over the ranks' different tokens; then everything is the gradient of the
            # sum of the per-rank mean losses, so one factor 1/ep turns it into the global mean
            flat.sync_replicated_grads(ep_group)
            grad_scale = grad_scale / ep
        if self._dist is not None:
            extra = None
            if self._fsdp is not None:
                extra = self._sharded_layers_sumsq()
            norm = self._dist.step(tx, step=self.step, lr=lr, grad_scale=grad_scale, zero_grad=zero_grad,
                                   extra_sumsq=extra)
            if self._fsdp is not None:
                coef, skip, gscale = self._dist.last_clip
                self._fsdp.update(tx, step=self.step, lr=lr, gscale=gscale, coef=coef, skip=skip)
            self.last_grad_norm = norm
            return norm
        g = flat.grad_shard
        coef = skip = None
        if g.is_cuda:
            from ..ops import kernels as K

            if self._sumsq is None:
                self._sumsq = torch.zeros(1, dtype=torch.float32, device=g.device)
            self._sumsq.zero_()
            K.sumsq_(self._sumsq, g)
            # every rank of the tensor- / expert-parallel groups must clip with the same global norm
            self._sumsq.copy_(flat.global_sumsq(self._sumsq, g, flat.shard_lo, self._model_mesh()))
            norm, coef, skip = K.clip_coef(self._sumsq, grad_scale, tx.clip_grad or 0.0)
        else:
            sq = flat.global_sumsq(g.float().pow(2).sum().reshape(1), g, flat.shard_lo, self._model_mesh())
            norm = sq.sqrt().reshape(()) * grad_scale
            skip = (~torch.isfinite(norm)).to(torch.int32).reshape(1)
            if tx.clip_grad:
                coef = torch.clamp(tx.clip_grad / (norm + 1e-6), max=1.0).reshape(1)
        for lo, hi, decay in flat.decay_ranges():
            state = {k: v[lo:hi] for k, v in flat.opt_state.items()}
            work = None if flat.master_is_work else flat.work_shard[lo:hi]
            tx.update(flat.master[lo:hi], work, g[lo:hi], state, step=self.step, lr=lr, gscale=grad_scale,
                      gscale_tensor=coef, skip_tensor=skip, decay=decay, zero_grad=zero_grad)
        self.last_grad_norm = norm
        return norm

    def _sharded_layers_sumsq(self) -> torch.Tensor:
        """Sum of squared gradients of the layer-sharded parameters over the whole model (one float, on device)."""
        import torch.distributed as dist

        rt = self._fsdp
        parts = rt.finish_reduction().clone()          # [tensor-parallel shards, the rest] of this rank's slices
        dist.all_reduce(parts, group=rt.group)         # the slices of all ranks make up the layers
        mesh = self._model_mesh()
        if mesh is not None and mesh.tp > 1 and rt._tp_mask_ranges():
            dist.all_reduce(parts[0:1], group=mesh.get_group("tp"))
        return parts.sum().reshape(1)

    def _model_mesh(self):
        mesh = getattr(getattr(self.model, "config", None), "mesh", None)
        return mesh if (mesh is not None and getattr(mesh, "is_distributed", False)) else None

    def _expert_parallel(self):
        mesh = getattr(getattr(self.model, "config", None), "mesh", None)
        if mesh is None or getattr(mesh, "ep", 1) <= 1:
            return None, 1
        return mesh.get_group("ep"), mesh.ep

    def zero_grad(self) -> None:
        if self.flat is not None:
            self.flat.zero_grad()
        for p in self.model.parameters():
            p.grad = None

    # ------------------------------------------------------------------ sharding API (kept for parity)
    def shard_state(self, **_):
        return self

    def gather_state(self, **_):
        return self

    def shard_model(self, **kw):
        self.model.shard_model(**kw)
        return self

    def gather_model(self, **kw):
        self.model.gather_model(**kw)
        return self

    # ------------------------------------------------------------------ persistence
    def save_state(self, save_directory: str | os.PathLike, float_dtype=None, save_optimizer: bool = True,
                   step: int | None = None, is_temporary: bool = False, **kw):
        from ..io.checkpoint import save_state

        return save_state(self, str(save_directory), float_dtype=float_dtype, save_optimizer=save_optimizer,
                          step=self.step if step is None else step, is_temporary=is_temporary, **kw)

    @classmethod
    def load_state(cls, load_directory: str | os.PathLike, model_class=None, tx_template: FlatOptimizer | None = None,
                   dtype=torch.bfloat16, param_dtype=None, device=None, config_kwargs: dict | None = None,
                   load_optimizer: bool = True, **kw):
        from ..io.checkpoint import load_state

        return load_state(cls, str(load_directory), model_class=model_class, tx_template=tx_template, dtype=dtype,
                          param_dtype=param_dtype, device=device, config_kwargs=config_kwargs,
                          load_optimizer=load_optimizer, **kw)

    def save_optimizer(self, save_directory: str):
        from ..io.checkpoint import save_optimizer_state

        return save_optimizer_state(self, save_directory)

    def load_optimizer(self, load_directory: str, tx_template: FlatOptimizer | None = None):
        from ..io.checkpoint import load_optimizer_state

        return load_optimizer_state(self, load_directory, tx_template)

    def __repr__(self):
        return f"EasyDeLState(step={self.step}, model={type(self.model).__name__}, tx={getattr(self.tx, 'name', None)})"
