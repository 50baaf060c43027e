"""Process-group mesh over one process per GPU.

The reference describes parallelism as a 5-axis device mesh
``("dp","fsdp","ep","tp","sp")`` handed to the XLA SPMD partitioner
(easydel/infra/base_config.py:974-1071). Here the same description becomes a
grid of ranks; every axis owns one ``torch.distributed`` process group per line
of the grid (NCCL on GPUs, gloo on CPU ranks), and the runtime (FSDP buckets,
tensor-parallel linears, expert dispatch, ring attention) addresses peers through
those groups or through the symmetric heap built on top of them.

Rank order is row-major over the axis tuple with the last axis fastest, so the
``tp`` / ``sp`` peers of a rank are its nearest neighbours in rank space.
"""

from __future__ import annotations

import math
import os
import typing as tp

import torch
import torch.distributed as dist

from ..infra.base_config import DEFAULT_AXIS_DIMS, DEFAULT_AXIS_NAMES, resolve_axis_dims


class DeviceMesh:
    def __init__(self, dims: tp.Sequence[int], names: tp.Sequence[str], rank: int = 0, world_size: int = 1):
        self.names = tuple(names)
        self.dims = tuple(int(d) for d in dims)
        if len(self.names) != len(self.dims):
            raise ValueError("axis names and dims differ in length")
        if math.prod(self.dims) != world_size:
            raise ValueError(f"mesh {dict(zip(self.names, self.dims))} does not cover world size {world_size}")
        self.rank = rank
        self.world_size = world_size
        self.shape = dict(zip(self.names, self.dims))
        self._groups: dict[tuple[str, ...], tp.Any] = {}
        self._group_ranks: dict[tuple[str, ...], list[int]] = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, dims=DEFAULT_AXIS_DIMS, names=DEFAULT_AXIS_NAMES, world_size: int | None = None,
               rank: int | None = None) -> "DeviceMesh":
        if world_size is None:
            world_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        return cls(resolve_axis_dims(dims, world_size), names, rank=rank, world_size=world_size)

    @classmethod
    def from_config(cls, config) -> "DeviceMesh":
        return cls.create(config.sharding_axis_dims, config.sharding_axis_names)

    # ------------------------------------------------------------------ coordinates
    def coords_of(self, rank: int) -> dict[str, int]:
        out, r = {}, rank
        for name, d in zip(reversed(self.names), reversed(self.dims)):
            out[name] = r % d
            r //= d
        return {n: out[n] for n in self.names}

    def rank_of(self, coords: dict[str, int]) -> int:
        r = 0
        for name, d in zip(self.names, self.dims):
            r = r * d + coords[name]
        return r

    @property
    def coords(self) -> dict[str, int]:
        return self.coords_of(self.rank)

    def axis_size(self, axis: str | tp.Sequence[str]) -> int:
        axes = (axis,) if isinstance(axis, str) else tuple(axis)
        return math.prod(self.shape[a] for a in axes)

    def axis_index(self, axis: str | tp.Sequence[str]) -> int:
        """Index of this rank inside its group over ``axis`` (row-major over the listed axes)."""
        axes = (axis,) if isinstance(axis, str) else tuple(axis)
        c = self.coords
        idx = 0
        for a in axes:
            idx = idx * self.shape[a] + c[a]
        return idx

    def group_ranks(self, axis: str | tp.Sequence[str], rank: int | None = None) -> list[int]:
        """Global ranks that share every coordinate with ``rank`` except those of ``axis``."""
        axes = (axis,) if isinstance(axis, str) else tuple(axis)
        base = self.coords_of(self.rank if rank is None else rank)
        ranks = []

        def rec(i, cur):
            if i == len(axes):
                ranks.append(self.rank_of(cur))
                return
            for v in range(self.shape[axes[i]]):
                nxt = dict(cur)
                nxt[axes[i]] = v
                rec(i + 1, nxt)

        rec(0, base)
        return ranks

    # ------------------------------------------------------------------ process groups
    def get_group(self, axis: str | tp.Sequence[str]):
        """Process group over one axis (or a tuple of axes folded together). ``None`` when trivial."""
        axes = (axis,) if isinstance(axis, str) else tuple(axis)
        if self.axis_size(axes) == 1 or self.world_size == 1:
            return None
        if axes in self._groups:
            return self._groups[axes]
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("torch.distributed is not initialised but the mesh has more than one rank")
        # every rank must create every group of the family, in the same order
        seen: set[tuple[int, ...]] = set()
        mine = None
        for r in range(self.world_size):
            ranks = tuple(self.group_ranks(axes, r))
            if ranks in seen:
                continue
            seen.add(ranks)
            g = dist.new_group(list(ranks))
            if self.rank in ranks:
                mine = g
                self._group_ranks[axes] = list(ranks)
        self._groups[axes] = mine
        return mine

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    def __repr__(self):
        return f"DeviceMesh({self.shape}, rank={self.rank}/{self.world_size})"

    # convenience accessors
    @property
    def dp(self) -> int:
        return self.shape.get("dp", 1)

    @property
    def fsdp(self) -> int:
        return self.shape.get("fsdp", 1)

    @property
    def ep(self) -> int:
        return self.shape.get("ep", 1)

    @property
    def tp(self) -> int:
        return self.shape.get("tp", 1)

    @property
    def sp(self) -> int:
        return self.shape.get("sp", 1)

    def expert_mesh_dims(self, fsdp_is_ep_bound: bool = True, sp_is_ep_bound: bool = True) -> dict[str, int]:
        """Folds fsdp / sp into the expert axis the way the reference's expert mesh does
        (easydel/infra/base_config.py:226-275): returns the ``(dp, ep, tp)`` sizes experts are laid out on."""
        ep = self.ep
        dp = self.dp
        if fsdp_is_ep_bound:
            ep *= self.fsdp
        else:
            dp *= self.fsdp
        if sp_is_ep_bound:
            ep *= self.sp
        else:
            dp *= self.sp
        return {"dp": dp, "ep": ep, "tp": self.tp}


def init_distributed(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int, int]:
    """Initialises ``torch.distributed`` from the torchrun environment. Returns (rank, local_rank, world)."""
    import datetime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, local, world
