"""Model placement helpers used by ``model.shard_model`` / ``gather_model``.

With the explicit runtime there is nothing to "shard" after construction: tensor- and expert-parallel
layers are built with their local shapes from the mesh in the config, and the data-parallel / FSDP
sharding of master weights and optimizer state happens in ``EasyDeLState.init_tx``. ``place_model``
therefore only moves the module to this rank's device and makes replicated parameters identical
across the tensor-parallel group.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def place_model(model, mesh):
    if torch.cuda.is_available():
        dev = torch.device("cuda", torch.cuda.current_device())
        if model.device != dev:
            model.to(dev)
    if mesh is not None and mesh.is_distributed and mesh.tp > 1:
        group = mesh.get_group("tp")
        src = dist.get_global_rank(group, 0)
        for name, mod in model.named_modules():
            style = getattr(mod, "parallel_style", None)
            for pname, p in mod.named_parameters(recurse=False):
                sharded = style in ("column", "row") and getattr(mod, "tp_size", 1) > 1 and \
                    not (style == "row" and pname == "bias")
                if not sharded:
                    dist.broadcast(p.data, src=src, group=group)
    return model


def gather_model(model):
    return model
