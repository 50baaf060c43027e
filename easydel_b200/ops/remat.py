"""Activation recomputation with named save policies.

The reference selects what a checkpointed layer keeps with ``jax.checkpoint`` policies over named intermediates
(easydel/infra/utils.py:180-267: ``nothing_saveable``, ``dots_saveable``, ``save_only_these_names`` ...). The
kernels here are opaque autograd nodes, so the same choice is made at the op level: a layer runs as a
:class:`RecomputeUnit` (forward without a graph, recomputed in backward), and the expensive ops inside it
(linear layers = "dots", the flash-attention kernel) carry a name. When the policy says a name is saved, the op's
output of the first forward is kept, and during the recompute the op hands that output back instead of running its
kernel, while still recording what its own backward needs (inputs and weights). Element-wise work, norms and
rotary embeddings are always recomputed.

Names follow the reference's: ``attn_qkv`` (also matches ``attn_query`` / ``attn_key`` / ``attn_value``),
``attn_core`` (the attention kernel itself), ``attn_output`` (output projection), ``mlp_gate_up`` (also
``mlp_gate`` / ``mlp_up``), ``mlp_down`` (also ``mlp_output``).
"""

from __future__ import annotations

import re
import threading
import typing as tp

import torch

_ALIASES = {
    "attn_qkv": ("attn_qkv", "attn_query", "attn_key", "attn_value"),
    "attn_core": ("attn_core",),
    "attn_output": ("attn_output",),
    "mlp_gate_up": ("mlp_gate_up", "mlp_gate", "mlp_up"),
    "mlp_down": ("mlp_down", "mlp_output"),
}
KNOWN_NAMES = tuple(_ALIASES)


class SavePolicy:
    """``saves(name, kind)``: keep the output of the op called ``name`` (kind "dot" or "attn")?"""

    def __init__(self, label: str, fn: tp.Callable[[str | None, str], bool], full: bool = False, none: bool = False):
        self.label, self._fn = label, fn
        self.recompute_everything = full      # nothing saved: plain full recompute
        self.save_everything = none           # no checkpointing at all

    def saves(self, name: str | None, kind: str) -> bool:
        return self._fn(name, kind)

    def __repr__(self):
        return f"SavePolicy({self.label})"


def _matches(name: str | None, wanted: tp.Iterable[str]) -> bool:
    if name is None:
        return False
    al = _ALIASES.get(name, (name,))
    return any(w in al for w in wanted)


def get_policy(name: str | None, save_names: tp.Sequence[str] | None = None,
               exclude_names: tp.Sequence[str] | None = None) -> SavePolicy:
    """Policy by the reference's name (``EasyDeLGradientCheckPointers`` values)."""
    name = str(getattr(name, "value", name) or "")
    if name in ("", "everything_saveable"):
        return SavePolicy(name or "everything_saveable", lambda n, k: True, none=True)
    if name == "nothing_saveable":
        return SavePolicy(name, lambda n, k: False, full=True)
    if name in ("dots_saveable", "checkpoint_dots", "dots_with_no_batch_dims_saveable",
                "checkpoint_dots_with_no_batch_dims"):
        return SavePolicy(name, lambda n, k: k == "dot")
    if name == "save_only_these_names":
        if not save_names:
            raise ValueError("save_names must be provided when using 'save_only_these_names' policy")
        wanted = tuple(save_names)
        return SavePolicy(f"{name}{wanted}", lambda n, k: _matches(n, wanted))
    if name in ("save_anything_except_these_names", "save_any_names_but_these"):
        if exclude_names is None:
            raise ValueError("exclude_names must be provided when using exclude-based policies")
        ex = tuple(exclude_names)
        return SavePolicy(f"{name}{ex}", lambda n, k: n is not None and not _matches(n, ex))
    pats = {"mlp_notsaveable": [r"^mlp_"], "attn_notsaveable": [r"^attn_"], "mlp_attn_notsaveable": [r"^mlp_", r"^attn_"]}
    if name in pats:
        rx = [re.compile(p) for p in pats[name]]
        return SavePolicy(name, lambda n, k: n is not None and not any(r.search(n) for r in rx))
    if name == "save_from_both_policies":
        a = get_policy("dots_saveable")
        b = get_policy("save_only_these_names", save_names or KNOWN_NAMES)
        return SavePolicy(name, lambda n, k: a.saves(n, k) or b.saves(n, k))
    raise KeyError(f"Unknown checkpoint policy: {name}")


class _Tape(threading.local):
    def __init__(self):
        self.mode: str | None = None        # None | "record" | "replay"
        self.policy: SavePolicy | None = None
        self.store: list = []
        self.cursor = 0


_tape = _Tape()


def saved_output(name: str | None, kind: str):
    """For an op about to run: ``(hit, value)``. ``hit`` is True during the recompute of a unit whose policy kept
    this op's output; ``value`` is then what the op returned in the first forward."""
    t = _tape
    if t.mode == "replay" and t.policy.saves(name, kind):
        v = t.store[t.cursor]
        t.cursor += 1
        return True, v
    return False, None


def keep_output(name: str | None, kind: str, value) -> None:
    """For an op that just ran in the first forward of a unit: keeps ``value`` if the policy saves it."""
    t = _tape
    if t.mode == "record" and t.policy.saves(name, kind):
        t.store.append(value)


class _Unit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, policy, hooks, n_tensors, *args):
        tensors, rest = args[:n_tensors], args[n_tensors:]
        prev = (_tape.mode, _tape.policy, _tape.store, _tape.cursor)
        _tape.mode, _tape.policy, _tape.store, _tape.cursor = "record", policy, [], 0
        try:
            if hooks is not None:
                hooks.before_forward()
            with torch.no_grad():
                outs = fn(*tensors, *rest)
            if hooks is not None:
                hooks.after_forward()
            ctx.kept = _tape.store
        finally:
            _tape.mode, _tape.policy, _tape.store, _tape.cursor = prev
        ctx.fn, ctx.policy, ctx.hooks, ctx.rest = fn, policy, hooks, rest
        ctx.save_for_backward(*[t if isinstance(t, torch.Tensor) else None for t in tensors])
        ctx.is_tensor = [isinstance(t, torch.Tensor) for t in tensors]
        ctx.raw = [None if isinstance(t, torch.Tensor) else t for t in tensors]
        single = isinstance(outs, torch.Tensor)
        outs = (outs,) if single else tuple(outs)
        ctx.out_none = [o is None for o in outs]
        ctx.single = single
        ref = next(o for o in outs if o is not None)
        return tuple(o if o is not None else ref.new_empty(0) for o in outs)

    @staticmethod
    def backward(ctx, *gouts):
        saved = ctx.saved_tensors
        ins = []
        for i, is_t in enumerate(ctx.is_tensor):
            if is_t:
                t = saved[i]
                ins.append(t.detach().requires_grad_(t.requires_grad) if t.is_floating_point() else t)
            else:
                ins.append(ctx.raw[i])
        prev = (_tape.mode, _tape.policy, _tape.store, _tape.cursor)
        _tape.mode, _tape.policy, _tape.store, _tape.cursor = "replay", ctx.policy, ctx.kept, 0
        try:
            if ctx.hooks is not None:
                ctx.hooks.before_backward()
            with torch.enable_grad():
                outs = ctx.fn(*ins, *ctx.rest)
            outs = (outs,) if isinstance(outs, torch.Tensor) else tuple(outs)
            sel_o, sel_g = [], []
            for o, g in zip(outs, gouts):
                if o is not None and o.requires_grad and g is not None and g.numel():
                    sel_o.append(o)
                    sel_g.append(g)
            torch.autograd.backward(sel_o, sel_g)
            if ctx.hooks is not None:
                ctx.hooks.after_backward()
        finally:
            _tape.mode, _tape.policy, _tape.store, _tape.cursor = prev
        ctx.kept = None
        grads = [t.grad if (isinstance(t, torch.Tensor) and t.is_floating_point() and t.requires_grad) else None
                 for t in ins]
        return (None, None, None, None, *grads, *([None] * len(ctx.rest)))


class UnitHooks:
    """Callbacks around the two passes of a unit (the parameter-sharded runtime gathers weights and launches the
    gradient reduction from here)."""

    def before_forward(self): ...
    def after_forward(self): ...
    def before_backward(self): ...
    def after_backward(self): ...


def recompute_unit(fn: tp.Callable, policy: SavePolicy, tensors: tp.Sequence, rest: tp.Sequence = (),
                   hooks: UnitHooks | None = None) -> tuple:
    """Runs ``fn(*tensors, *rest)`` as a recompute unit under ``policy`` and returns its outputs as a tuple.
    ``tensors`` may contain ``None``; gradients flow to its floating-point tensors. An output that is ``None``
    stays ``None`` (real outputs must not be empty tensors)."""
    outs = _Unit.apply(fn, policy, hooks, len(tensors), *tensors, *rest)
    return tuple(None if o.numel() == 0 else o for o in outs)
