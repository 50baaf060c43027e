"""Parameter-sharded data parallelism for a stack of identical layers (the ``fsdp`` axis as ZeRO-3).

What the reference expresses as parameters *and* optimizer state sharded over ``fsdp`` with XLA-inserted
all-gathers and reduce-scatters (easydel/infra/base_config.py:793-795, easydel/infra/base_state.py:575-666)
is carried out here explicitly, one decoder layer at a time:

* every rank keeps ``1/N`` of each layer's bf16 weights (in symmetric memory, so that peers can read it), the
  fp32 master copy and optimizer moments of that slice, and an fp32 accumulator for the slice's gradients;
* a layer's full weights are assembled into one of three rotating buffers by this framework's gather kernel
  (``edl_fsdp_gather``: peer loads over NVLink) on a side stream while the previous layer computes: layer
  *l + 1* during the forward sweep, layer *l - 1* during the backward sweep;
* the layer runs as a recompute unit (forward without saved activations, recomputed in backward), its weight
  gradients accumulate into one of two rotating fp32 layer buffers, and as soon as the layer's backward is done
  the side stream sums every rank's buffer slice into the owner's accumulator (``edl_fsdp_reduce_acc``) while the
  compute stream already runs the backward of the next layer;
* the optimizer step then touches only the local slices (fused AdamW writing the bf16 shard in place).

On CPU ranks (gloo) the same schedule runs synchronously through ``torch.distributed`` collectives, which is what
the multi-process tests use. Embeddings, final norm and LM head are not handled here: they stay with the
optimizer-sharded flat storage (``parallel.dist_optim``).
"""

from __future__ import annotations

import ctypes as C
import re
import typing as tp

import torch
import torch.distributed as dist
from torch import nn

from ..ops import _lib

_lib.register("edl_fsdp_gather", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i64, _lib.vp, _lib.i32, _lib.vp])
_lib.register("edl_fsdp_reduce_acc", _lib.i32, [_lib.vp, _lib.i32, _lib.i32, _lib.i64, _lib.vp, _lib.i32, _lib.vp])

ALIGN = 128
W_SLOTS = 3   # rotating full-weight buffers: the layer in use, the one being prefetched, the one just used
G_SLOTS = 2   # rotating layer-gradient buffers: the layer in backward, the one being reduced


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _LayerHooks:
    """Connects a recompute unit (``ops.remat``) to the runtime: weights are gathered before each pass of the
    layer and released after it; the gradient buffer is claimed before the backward pass and reduced after it."""

    def __init__(self, rt: "ShardedLayers", idx: int):
        self.rt, self.idx = rt, idx

    def before_forward(self):
        self.rt.acquire_weights(self.idx, +1)

    def after_forward(self):
        self.rt.release_weights(self.idx)

    def before_backward(self):
        self.rt.acquire_weights(self.idx, -1)
        self.rt.acquire_grad_buffer(self.idx)

    def after_backward(self):
        self.rt.release_weights(self.idx)
        self.rt.reduce_layer_grads(self.idx)


class ShardedLayers:
    def __init__(self, layers: tp.Sequence[nn.Module], mesh, prefix: str = "model.layers",
                 no_decay_patterns: tp.Sequence[str] = (), use_peer_kernels: bool | None = None):
        axes = ("dp", "fsdp")
        self.mesh = mesh
        self.group = mesh.get_group(axes)
        self.world = mesh.axis_size(axes)
        self.rank = mesh.axis_index(axes)
        self.layers = list(layers)
        self.prefix = prefix
        L = len(self.layers)
        first = next(self.layers[0].parameters())
        self.device, self.dtype = first.device, first.dtype
        dev = self.device
        self.peer = bool(dev.type == "cuda" and _lib.available()) if use_peer_kernels is None else use_peer_kernels
        nd = [re.compile(x) for x in no_decay_patterns]
        # ---- layout of one layer's flat buffer (the same for every layer of a uniform stack)
        self.entries: list[list[tuple[str, nn.Parameter, int, int, tuple, bool]]] = []
        sizes = []
        for li, layer in enumerate(self.layers):
            off, ents = 0, []
            for n, p in layer.named_parameters():
                if not p.requires_grad:
                    continue
                if p.dtype != self.dtype:
                    raise ValueError("all sharded parameters must share one dtype")
                full_name = f"{prefix}.{li}.{n}"
                ents.append((full_name, p, off, p.numel(), tuple(p.shape), not any(r.search(full_name) for r in nd)))
                off = _round_up(off + p.numel(), ALIGN)
            self.entries.append(ents)
            sizes.append(off)
        self.S = _round_up(max(sizes), ALIGN * self.world)
        self.per = self.S // self.world
        S, per = self.S, self.per
        # ---- persistent, per rank
        self._symm = []
        self.wshard = self._alloc_symm(L * per, self.dtype)
        self.master = torch.zeros(L * per, dtype=torch.float32, device=dev)
        self.gshard = torch.zeros(L * per, dtype=torch.float32, device=dev)
        self.opt_state: dict[str, torch.Tensor] = {}
        # ---- rotating
        self.wfull = [torch.zeros(S, dtype=self.dtype, device=dev) for _ in range(W_SLOTS)]
        self.gfull = [self._alloc_symm(S, torch.float32) for _ in range(G_SLOTS)]
        self.resident = [-1] * W_SLOTS
        self._sumsq = torch.zeros(2, dtype=torch.float32, device=dev)
        if self.peer:
            self.comm = torch.cuda.Stream(device=dev)
            self.ev_gathered = [torch.cuda.Event() for _ in range(W_SLOTS)]
            self.ev_wfree = [torch.cuda.Event() for _ in range(W_SLOTS)]
            self.ev_gfree = [torch.cuda.Event() for _ in range(G_SLOTS)]
            self.ev_bwd = [torch.cuda.Event() for _ in range(G_SLOTS)]
            cur = torch.cuda.current_stream(dev)
            for e in (*self.ev_wfree, *self.ev_gfree):
                e.record(cur)
            self._rendezvous()
        # ---- take the weights over: rank 0's values are authoritative
        src = dist.get_global_rank(self.group, 0) if self.world > 1 else 0
        with torch.no_grad():
            stage = self.wfull[0]
            for li, ents in enumerate(self.entries):
                stage.zero_()
                for _, p, off, n, shape, _ in ents:
                    stage[off:off + n].copy_(p.data.reshape(-1))
                if self.world > 1:
                    dist.broadcast(stage, src=src, group=self.group)
                self.wshard[li * per:(li + 1) * per].copy_(stage[self.rank * per:(self.rank + 1) * per])
            self.master.copy_(self.wshard.float())
            placeholder = torch.empty(0, dtype=self.dtype, device=dev)
            for ents in self.entries:
                for _, p, _, _, _, _ in ents:
                    p.data = placeholder   # the full weights exist only while a layer is resident
                    p.grad = None
        self._barrier()
        self._shards_published()
        self._last = -1
        self._materialized: torch.Tensor | None = None

    def _shards_published(self) -> None:
        """Call after this rank's shards changed and the group barrier behind the change has been enqueued on the
        compute stream: gathers (side stream) issued from now on wait for that point."""
        if self.peer:
            self.comm.wait_stream(torch.cuda.current_stream(self.device))

    # ------------------------------------------------------------------ symmetric memory
    def _alloc_symm(self, n: int, dtype) -> torch.Tensor:
        if self.peer and self.world > 1:
            import torch.distributed._symmetric_memory as symm

            t = symm.empty(n, dtype=dtype, device=self.device)
            t.zero_()
            self._symm.append(t)
            return t
        return torch.zeros(n, dtype=dtype, device=self.device)

    def _rendezvous(self) -> None:
        self._w_ptrs = self._g_ptrs = None
        self._handle = None
        if self.world == 1:
            self._w_base = [self.wshard.data_ptr()]
            self._g_base = [[g.data_ptr()] for g in self.gfull]
            return
        import torch.distributed._symmetric_memory as symm

        def ptrs(t):
            h = symm.rendezvous(t, self.group)
            off = int(getattr(h, "offset", 0))
            base = [int(p) + off for p in h.buffer_ptrs]
            if base[self.rank] != t.data_ptr():
                raise RuntimeError("symmetric-memory handle does not address this rank's own buffer")
            return h, base

        self._handle, self._w_base = ptrs(self.wshard)
        self._g_base = [ptrs(g)[1] for g in self.gfull]
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _barrier(self, channel: int = 0) -> None:
        """Device-side barrier over the group on the current stream (host barrier on CPU ranks)."""
        if self.world == 1:
            return
        if self.peer:
            self._handle.barrier(channel=channel)
        else:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ weights
    def _point_params(self, idx: int, wbuf: torch.Tensor) -> None:
        for _, p, off, n, shape, _ in self.entries[idx]:
            p.data = wbuf[off:off + n].view(shape)

    def _gather(self, idx: int) -> None:
        """Assembles layer ``idx`` into its weight slot (on the side stream when peer kernels are in use)."""
        slot = idx % W_SLOTS
        per, S = self.per, self.S
        dst = self.wfull[slot]
        if self.peer:
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(self.ev_wfree[slot])    # the layer that last used this slot is done with it
                elt = dst.element_size()
                ptrs = (C.c_ulonglong * self.world)(*[b + idx * per * elt for b in self._w_base])
                _lib.call("edl_fsdp_gather", C.cast(ptrs, C.c_void_p), self.world, self.rank, per, dst.data_ptr(), 0,
                          self.comm.cuda_stream)
                self.ev_gathered[slot].record(self.comm)
        elif self.world > 1:
            dist.all_gather_into_tensor(dst, self.wshard[idx * per:(idx + 1) * per].contiguous(), group=self.group)
        else:
            dst.copy_(self.wshard[idx * per:(idx + 1) * per])
        self.resident[slot] = idx

    def acquire_weights(self, idx: int, direction: int) -> None:
        if self._materialized is not None:
            return
        slot = idx % W_SLOTS
        if self.resident[slot] != idx:
            self._gather(idx)
        if self.peer:
            torch.cuda.current_stream(self.device).wait_event(self.ev_gathered[slot])
        self._point_params(idx, self.wfull[slot])
        nxt = idx + direction
        if 0 <= nxt < len(self.layers) and self.resident[nxt % W_SLOTS] != nxt:
            self._gather(nxt)     # in flight while this layer computes
        self._last = idx

    def release_weights(self, idx: int) -> None:
        if self.peer and self._materialized is None:
            self.ev_wfree[idx % W_SLOTS].record(torch.cuda.current_stream(self.device))

    # ------------------------------------------------------------------ gradients
    def acquire_grad_buffer(self, idx: int) -> None:
        slot = idx % G_SLOTS
        if self.peer:
            torch.cuda.current_stream(self.device).wait_event(self.ev_gfree[slot])   # reduced and zeroed
        gbuf = self.gfull[slot]
        for _, p, off, n, shape, _ in self.entries[idx]:
            p.main_grad = gbuf[off:off + n].view(shape)
            p.grad = None

    def reduce_layer_grads(self, idx: int) -> None:
        """Sums the layer's gradient buffer over the ranks into the owners' accumulators and clears it."""
        slot = idx % G_SLOTS
        gbuf = self.gfull[slot]
        per = self.per
        for _, p, _, _, _, _ in self.entries[idx]:   # gradients that autograd delivered as .grad (norm scales)
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
        acc = self.gshard[idx * per:(idx + 1) * per]
        if self.peer:
            cur = torch.cuda.current_stream(self.device)
            self.ev_bwd[slot].record(cur)
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(self.ev_bwd[slot])
                self._barrier(0)        # every rank's gradients of this layer are complete
                ptrs = (C.c_ulonglong * self.world)(*self._g_base[slot])
                _lib.call("edl_fsdp_reduce_acc", C.cast(ptrs, C.c_void_p), self.world, self.rank, per,
                          acc.data_ptr(), 0, self.comm.cuda_stream)
                self._barrier(1)        # every rank has read this buffer: it may be cleared
                gbuf.zero_()
                self.ev_gfree[slot].record(self.comm)
        else:
            if self.world > 1:
                dist.all_reduce(gbuf, group=self.group)
            acc.add_(gbuf[self.rank * per:(self.rank + 1) * per])
            gbuf.zero_()

    # ------------------------------------------------------------------ running a layer
    def run(self, idx: int, layer: nn.Module, x, pending, positions, segment_ids, policy=None):
        """Runs layer ``idx`` with its weights gathered for the duration of the call (and of its backward). Under
        autograd the layer is a recompute unit: its weights leave after the forward pass, so its activations are
        rebuilt in backward (``policy`` may keep the outputs of named ops, see ``ops.remat``)."""
        if torch.is_grad_enabled():
            from ..ops import remat

            if policy is None or policy.save_everything:
                policy = remat.get_policy("nothing_saveable")
            return remat.recompute_unit(lambda a, b, c, d: layer(a, b, c, d, None, None), policy,
                                        (x, pending, positions, segment_ids), hooks=_LayerHooks(self, idx))
        self.acquire_weights(idx, +1)
        out = layer(x, pending, positions, segment_ids, None, None)
        self.release_weights(idx)
        return out

    # ------------------------------------------------------------------ optimizer step
    def decay_ranges(self) -> list[tuple[int, int, bool]]:
        """Maximal runs of this rank's shard storage ``[L * per]`` with one weight-decay flag."""
        lo_r, hi_r = self.rank * self.per, (self.rank + 1) * self.per
        runs: list[tuple[int, int, bool]] = []
        for li, ents in enumerate(self.entries):
            base = li * self.per - lo_r
            cur = lo_r
            for i, (_, _, off, n, _, decay) in enumerate(ents):
                end = ents[i + 1][2] if i + 1 < len(ents) else self.S
                a, b = max(off, lo_r), min(end, hi_r)
                if a >= b:
                    continue
                a, b = a + base, b + base
                if runs and runs[-1][2] == decay and runs[-1][1] == a:
                    runs[-1] = (runs[-1][0], b, decay)
                else:
                    runs.append((a, b, decay))
                cur = b
        return runs

    def finish_reduction(self) -> torch.Tensor:
        """Waits for the gradient reductions in flight and returns ``[sum of squares of tensor-parallel shards,
        sum of squares of the rest]`` of this rank's accumulated gradient slices (device tensor of two floats)."""
        if self.peer:
            torch.cuda.current_stream(self.device).wait_stream(self.comm)
        self._sumsq.zero_()
        tp_kinds = self._tp_mask_ranges()
        g = self.gshard
        if not tp_kinds:
            self._sumsq[1] = g.float().pow(2).sum()
        else:
            total = g.float().pow(2).sum()
            tp_part = sum(g[a:b].float().pow(2).sum() for a, b in tp_kinds)
            self._sumsq[0] = tp_part
            self._sumsq[1] = total - tp_part
        return self._sumsq

    def _tp_mask_ranges(self) -> list[tuple[int, int]]:
        """Ranges of the shard storage that hold tensor-parallel (column / row) parameters."""
        if getattr(self, "_tp_ranges", None) is not None:
            return self._tp_ranges
        owner = set()
        for layer in self.layers:
            for mod in layer.modules():
                style = getattr(mod, "parallel_style", None)
                if getattr(mod, "tp_size", 1) > 1 and style in ("column", "row"):
                    for leaf, p in mod.named_parameters(recurse=False):
                        if not (style == "row" and leaf == "bias"):
                            owner.add(id(p))
        lo_r, hi_r = self.rank * self.per, (self.rank + 1) * self.per
        out = []
        for li, ents in enumerate(self.entries):
            base = li * self.per - lo_r
            for _, p, off, n, _, _ in ents:
                if id(p) in owner:
                    a, b = max(off, lo_r), min(off + n, hi_r)
                    if a < b:
                        out.append((a + base, b + base))
        self._tp_ranges = out
        return out

    @torch.no_grad()
    def update(self, tx, *, step: int, lr: float, gscale: float, coef, skip) -> None:
        """Optimizer update of the local slices (``coef`` / ``skip``: the shared clip factor and non-finite flag)."""
        for lo, hi, decay in self.decay_ranges():
            state = {k: v[lo:hi] for k, v in self.opt_state.items()}
            tx.update(self.master[lo:hi], self.wshard[lo:hi], self.gshard[lo:hi], state, step=step, lr=lr,
                      gscale=gscale, gscale_tensor=coef, skip_tensor=skip, decay=decay, zero_grad=False)
        self.gshard.zero_()
        self.resident = [-1] * W_SLOTS      # every gathered copy is stale now
        self._barrier(2)                    # nobody gathers before every rank has written its new shard
        self._shards_published()
        if self._materialized is not None:
            self._fill_materialized()

    # ------------------------------------------------------------------ whole-model views (checkpoints, export)
    def _fill_materialized(self) -> None:
        L, S, per = len(self.layers), self.S, self.per
        full = self._materialized
        for li in range(L):
            dst = full[li * S:(li + 1) * S]
            if self.world > 1:
                dist.all_gather_into_tensor(dst, self.wshard[li * per:(li + 1) * per].contiguous(), group=self.group)
            else:
                dst.copy_(self.wshard[li * per:(li + 1) * per])
            self._point_params(li, dst)

    def materialize(self) -> None:
        """Gathers every layer into one full buffer and points the parameters at it (a collective). Used around
        ``state_dict`` / checkpoint writing and by inference on a training model."""
        if self._materialized is None:
            if self.peer:
                torch.cuda.synchronize(self.device)
            self._materialized = torch.empty(len(self.layers) * self.S, dtype=self.dtype, device=self.device)
            self._fill_materialized()

    def dematerialize(self, reshard: bool = False) -> None:
        """Drops the full buffer; ``reshard=True`` first takes the (possibly loaded) parameter values back into
        the shards and the master copy."""
        if self._materialized is None:
            return
        S, per = self.S, self.per
        if reshard:
            with torch.no_grad():
                for li in range(len(self.layers)):
                    src = self._materialized[li * S:(li + 1) * S]
                    self.wshard[li * per:(li + 1) * per].copy_(src[self.rank * per:(self.rank + 1) * per])
                self.master.copy_(self.wshard.float())
        placeholder = torch.empty(0, dtype=self.dtype, device=self.device)
        for ents in self.entries:
            for _, p, *_ in ents:
                p.data = placeholder
        self._materialized = None
        self.resident = [-1] * W_SLOTS
        self._barrier(2)
        self._shards_published()

    def named_state(self) -> tp.Iterator[tuple[str, torch.Tensor]]:
        """``(state name . parameter name, full tensor)`` of master weights and moments (a collective)."""
        L, S, per = len(self.layers), self.S, self.per
        for sname, buf in {"master": self.master, **self.opt_state}.items():
            for li in range(L):
                piece = buf[li * per:(li + 1) * per].contiguous()
                if self.world > 1:
                    full = torch.empty(S, dtype=buf.dtype, device=buf.device)
                    dist.all_gather_into_tensor(full, piece, group=self.group)
                else:
                    full = piece
                for name, _, off, n, shape, _ in self.entries[li]:
                    yield f"{sname}.{name}", full[off:off + n].view(shape)

    def load_named_state(self, tree: dict[str, torch.Tensor]) -> None:
        """Inverse of :meth:`named_state`: keeps this rank's slice of every tensor found in ``tree``."""
        per = self.per
        lo_r, hi_r = self.rank * per, (self.rank + 1) * per
        for sname, buf in {"master": self.master, **self.opt_state}.items():
            for li, ents in enumerate(self.entries):
                for name, _, off, n, _, _ in ents:
                    key = f"{sname}.{name}"
                    if key not in tree:
                        continue
                    a, b = max(off, lo_r), min(off + n, hi_r)
                    if a < b:
                        src = tree[key].reshape(-1)[a - off:b - off]
                        buf[li * per + a - lo_r:li * per + b - lo_r].copy_(src.to(buf.dtype))

    def memory_bytes(self) -> dict[str, int]:
        e = self.wshard.element_size()
        L = len(self.layers)
        return {"weight_shards": L * self.per * e, "master_and_grad_shards": 2 * L * self.per * 4,
                "optimizer_moments": sum(v.numel() * v.element_size() for v in self.opt_state.values()),
                "rotating_weight_buffers": W_SLOTS * self.S * e, "rotating_grad_buffers": G_SLOTS * self.S * 4}
