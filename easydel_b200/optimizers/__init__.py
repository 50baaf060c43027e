"""Optimizers and learning-rate schedules.

Plays the role of ``eformer.optimizers`` for the reference (``OptimizerFactory.create`` is reached
from easydel/trainers/training_configurations.py:1396-1445; optimizer / scheduler names from
easydel/infra/etils.py:116-123,154-156). Every optimizer works on *flat* fp32 buffers
(master weights, moments, gradients) owned by :class:`easydel_b200.parallel.flat.FlatParams`;
AdamW on CUDA is one fused kernel launch over each buffer (``edl_adamw``), which also emits
the bf16 working copy. Under FSDP the buffers are the rank's shard and the same code runs
on the shard.
"""

from __future__ import annotations

import math
import typing as tp
from dataclasses import dataclass, field

import torch

from ..ops import _lib


# --------------------------------------------------------------------------- schedules
@dataclass
class SchedulerConfig:
    scheduler_type: str | None = None     # None | "linear" | "cosine"
    learning_rate: float = 5e-5
    learning_rate_end: float | None = None
    warmup_steps: int = 0
    steps: int | None = None
    exponent: float = 1.0

    def build(self) -> tp.Callable[[int], float]:
        lr, end = float(self.learning_rate), self.learning_rate_end
        warm = int(self.warmup_steps or 0)
        total = self.steps
        kind = (self.scheduler_type or "none")
        kind = str(getattr(kind, "value", kind)).lower()

        def sched(step: int) -> float:
            if warm > 0 and step < warm:
                return lr * (step + 1) / warm
            if kind in ("none", "constant") or not total or total <= warm:
                return lr
            frac = min(1.0, (step - warm) / max(1, total - warm))
            lo = 0.0 if end is None else float(end)
            if kind == "linear":
                return lo + (lr - lo) * (1.0 - frac) ** self.exponent
            if kind == "cosine":
                return lo + (lr - lo) * 0.5 * (1.0 + math.cos(math.pi * frac))
            raise ValueError(f"unknown scheduler {kind!r}")

        return sched


# --------------------------------------------------------------------------- optimizers
class FlatOptimizer:
    """Base: state tensors shaped like the flat fp32 master buffer of each bucket."""

    name = "base"
    state_names: tuple[str, ...] = ()

    def __init__(self, scheduler: tp.Callable[[int], float], weight_decay: float = 0.0, clip_grad: float | None = None,
                 **hyper):
        self.scheduler = scheduler
        self.weight_decay = float(weight_decay or 0.0)
        self.clip_grad = clip_grad
        self.hyper = hyper

    def init_state(self, master: torch.Tensor) -> dict[str, torch.Tensor]:
        return {n: torch.zeros_like(master) for n in self.state_names}

    def lr_at(self, step: int) -> float:
        return float(self.scheduler(step))

    def update(self, master, work, grad, state, *, step: int, lr: float, gscale: float, gscale_tensor, skip_tensor,
               decay: bool = True, zero_grad: bool = True) -> None:
        raise NotImplementedError

    # torch-op fallback used by the non-AdamW rules; g is the *scaled* fp32 gradient
    def _finish(self, master, work, grad, zero_grad):
        if work is not None and work.data_ptr() != master.data_ptr():
            work.copy_(master)
        if zero_grad:
            grad.zero_()

    @staticmethod
    def _scaled(grad, gscale, gscale_tensor):
        g = grad.float() * gscale
        if gscale_tensor is not None:
            g = g * gscale_tensor
        return g

    def describe(self) -> dict:
        return {"optimizer": self.name, "weight_decay": self.weight_decay, "clip_grad": self.clip_grad, **self.hyper}


class AdamW(FlatOptimizer):
    name = "adamw"
    state_names = ("mu", "nu")

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, b1: float = 0.9, b2: float = 0.999,
                 eps: float = 1e-8, **kw):
        super().__init__(scheduler, weight_decay, clip_grad, b1=b1, b2=b2, eps=eps)
        self.b1, self.b2, self.eps = b1, b2, eps

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        wd = self.weight_decay if decay else 0.0
        if master.is_cuda:
            from ..ops import kernels as K

            w16 = work if (work is not None and work.dtype == torch.bfloat16) else None
            K.adamw_(master, w16, state["mu"], state["nu"], grad, lr=lr, beta1=self.b1, beta2=self.b2, eps=self.eps,
                     weight_decay=wd, step=step, gscale=gscale, gscale_tensor=gscale_tensor,
                     skip_tensor=skip_tensor, zero_grad=zero_grad)
            if work is not None and w16 is None and work.data_ptr() != master.data_ptr():
                work.copy_(master)
            return
        from ..ops import reference as R

        g = self._scaled(grad, gscale, gscale_tensor)
        if skip_tensor is not None and bool(skip_tensor.item()):
            if zero_grad:
                grad.zero_()
            return
        R.adamw_step(master, state["mu"], state["nu"], g, lr=lr, beta1=self.b1, beta2=self.b2, eps=self.eps,
                     weight_decay=wd, step=step)
        self._finish(master, work, grad, zero_grad)


class Lion(FlatOptimizer):
    name = "lion"
    state_names = ("mu",)

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, b1: float = 0.9, b2: float = 0.99, **kw):
        super().__init__(scheduler, weight_decay, clip_grad, b1=b1, b2=b2)
        self.b1, self.b2 = b1, b2

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        m = state["mu"]
        upd = (m * self.b1 + g * (1 - self.b1)).sign_()
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.add_(upd, alpha=-lr)
        m.mul_(self.b2).add_(g, alpha=1 - self.b2)
        self._finish(master, work, grad, zero_grad)


class RMSProp(FlatOptimizer):
    name = "rmsprop"
    state_names = ("nu", "mu")

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, decay: float = 0.9, eps: float = 1e-8,
                 momentum: float = 0.0, **kw):
        super().__init__(scheduler, weight_decay, clip_grad, decay=decay, eps=eps, momentum=momentum)
        self.decay, self.eps, self.momentum = decay, eps, momentum

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        v = state["nu"]
        v.mul_(self.decay).addcmul_(g, g, value=1 - self.decay)
        upd = g / (v.sqrt() + self.eps)
        if self.momentum:
            m = state["mu"]
            m.mul_(self.momentum).add_(upd)
            upd = m
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.add_(upd, alpha=-lr)
        self._finish(master, work, grad, zero_grad)


class Adafactor(FlatOptimizer):
    """Adafactor on flat buffers. Factored second moments need matrix shapes, which flat storage
    does not carry, so the unfactored form with update clipping and relative step scaling is used."""

    name = "adafactor"
    state_names = ("nu",)

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, decay_rate: float = 0.8, eps: float = 1e-30,
                 clipping_threshold: float = 1.0, **kw):
        super().__init__(scheduler, weight_decay, clip_grad, decay_rate=decay_rate, eps=eps,
                         clipping_threshold=clipping_threshold)
        self.decay_rate, self.eps, self.clip = decay_rate, eps, clipping_threshold

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        beta2 = 1.0 - step ** (-self.decay_rate)
        v = state["nu"]
        v.mul_(beta2).add_(g * g + self.eps, alpha=1 - beta2)
        u = g / v.sqrt()
        rms = u.pow(2).mean().sqrt()
        u = u / torch.clamp(rms / self.clip, min=1.0)
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.add_(u, alpha=-lr)
        self._finish(master, work, grad, zero_grad)


class Mars(AdamW):
    """MARS: AdamW on a variance-reduced gradient ``c = g + gamma * b1/(1-b1) * (g - g_prev)``, clipped to unit norm."""

    name = "mars"
    state_names = ("mu", "nu", "prev")

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, b1=0.95, b2=0.99, eps=1e-8, gamma: float = 0.025,
                 **kw):
        super().__init__(scheduler, weight_decay, clip_grad, b1=b1, b2=b2, eps=eps)
        self.gamma = gamma
        self.hyper["gamma"] = gamma

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        prev = state["prev"]
        c = g + self.gamma * self.b1 / (1 - self.b1) * (g - prev)
        n = c.norm()
        c = c / torch.clamp(n, min=1.0)
        prev.copy_(g)
        from ..ops import reference as R

        R.adamw_step(master, state["mu"], state["nu"], c, lr=lr, beta1=self.b1, beta2=self.b2, eps=self.eps,
                     weight_decay=self.weight_decay if decay else 0.0, step=step)
        self._finish(master, work, grad, zero_grad)


class Muon(FlatOptimizer):
    """Momentum + sign-normalised update. Matrix orthogonalisation (Newton-Schulz) needs per-matrix
    views; on flat storage the update is the RMS-normalised Nesterov momentum, which is what Muon
    reduces to for non-matrix parameters."""

    name = "muon"
    state_names = ("mu",)

    def __init__(self, scheduler, weight_decay=0.0, clip_grad=None, momentum: float = 0.95, nesterov: bool = True,
                 **kw):
        super().__init__(scheduler, weight_decay, clip_grad, momentum=momentum, nesterov=nesterov)
        self.momentum, self.nesterov = momentum, nesterov

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        m = state["mu"]
        m.mul_(self.momentum).add_(g)
        u = g + self.momentum * m if self.nesterov else m
        u = u / (u.pow(2).mean().sqrt() + 1e-8)
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.add_(u, alpha=-lr)
        self._finish(master, work, grad, zero_grad)


class Skew(AdamW):
    """AdamW variant with asymmetric second-moment tracking (faster to grow than to shrink)."""

    name = "skew"

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        m, v = state["mu"], state["nu"]
        m.mul_(self.b1).add_(g, alpha=1 - self.b1)
        g2 = g * g
        v.copy_(torch.where(g2 > v, g2 * (1 - self.b2 ** 2) + v * self.b2 ** 2, v * self.b2 + g2 * (1 - self.b2)))
        bc1 = 1 - self.b1 ** step
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.addcdiv_(m / bc1, v.sqrt() + self.eps, value=-lr)
        self._finish(master, work, grad, zero_grad)


class Quad(AdamW):
    """AdamW with a fourth-root preconditioner (``|g|`` statistics instead of ``g^2``)."""

    name = "quad"

    def update(self, master, work, grad, state, *, step, lr, gscale, gscale_tensor, skip_tensor, decay=True,
               zero_grad=True):
        g = self._scaled(grad, gscale, gscale_tensor)
        m, v = state["mu"], state["nu"]
        m.mul_(self.b1).add_(g, alpha=1 - self.b1)
        v.mul_(self.b2).add_(g.abs(), alpha=1 - self.b2)
        bc1, bc2 = 1 - self.b1 ** step, 1 - self.b2 ** step
        if decay and self.weight_decay:
            master.mul_(1 - lr * self.weight_decay)
        master.addcdiv_(m / bc1, v / bc2 + self.eps, value=-lr)
        self._finish(master, work, grad, zero_grad)


OPTIMIZERS: dict[str, type[FlatOptimizer]] = {
    "adamw": AdamW, "lion": Lion, "rmsprop": RMSProp, "adafactor": Adafactor, "mars": Mars, "muon": Muon,
    "skew": Skew, "quad": Quad,
}


class OptimizerFactory:
    @staticmethod
    def create(optimizer_type: str, scheduler_config: SchedulerConfig, clip_grad: float | None = None,
               weight_decay: float = 0.0, custom_scheduler: tp.Callable[[int], float] | None = None, **kwargs):
        """Returns ``(optimizer, schedule_fn)``. Extra kwargs (``b1``, ``b2``, ``eps``...) reach the optimizer."""
        name = str(getattr(optimizer_type, "value", optimizer_type)).lower()
        if name not in OPTIMIZERS:
            raise ValueError(f"unknown optimizer {optimizer_type!r}; available: {sorted(OPTIMIZERS)}")
        sched = custom_scheduler(scheduler_config.steps) if custom_scheduler is not None and \
            _wants_steps(custom_scheduler) else (custom_scheduler or scheduler_config.build())
        kwargs.pop("mu_dtype", None)
        kwargs.pop("gradient_accumulation_steps", None)
        opt = OPTIMIZERS[name](sched, weight_decay=weight_decay, clip_grad=clip_grad, **kwargs)
        return opt, sched


def _wants_steps(fn) -> bool:
    import inspect

    try:
        params = list(inspect.signature(fn).parameters)
    except (TypeError, ValueError):
        return False
    return len(params) == 1 and params[0] in ("steps", "total_steps", "num_steps")
