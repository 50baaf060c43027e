"""``RayDistributedTrainer``: build model + trainer inside worker processes from a scaling index
(easydel/trainers/ray_scaler/distributed_trainer.py).

The reference launches its workers through Ray actors. Ray is not a dependency here: workers are one process per
GPU started with ``torch.multiprocessing`` (the same rendezvous ``torchrun`` sets up), and when ``ray`` happens
to be importable the same worker function is submitted as Ray tasks instead. The scaling logic is identical:
``scaling_index`` multiplies the width / depth fields named in ``RayDistributedConfig.scaling_fields``.
"""

from __future__ import annotations

import copy
import os
import typing as tp
from dataclasses import dataclass, field

import torch


@dataclass
class RayDistributedConfig:
    pretrained_model_name_or_path: str | None = None
    model_type: str = "llama"
    model_task: str = "causal-language-model"
    base_config: dict = field(default_factory=dict)
    scaling_fields: dict[str, float] = field(default_factory=lambda: {"hidden_size": 1.0, "intermediate_size": 1.0,
                                                                      "num_hidden_layers": 1.0})
    round_to: int = 128
    num_workers: int = 1
    sharding_axis_dims: tuple[int, ...] = (1, -1, 1, 1, 1)
    trainer_type: str = "base"
    master_port: int = 29610

    def scaled_config(self, scaling_index: int) -> dict:
        cfg = copy.deepcopy(self.base_config)
        for k, rate in self.scaling_fields.items():
            if k not in cfg:
                continue
            v = cfg[k] * (1 + rate * scaling_index)
            cfg[k] = int(round(v)) if k.startswith("num_") else int(-(-v // self.round_to) * self.round_to)
        return cfg


def _worker(rank: int, world: int, cfg: RayDistributedConfig, scaling_index: int, arguments, dataset_fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(cfg.master_port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from ..infra.factory import registry
    from ..parallel.mesh import init_distributed
    from . import get_trainer_class

    if world > 1:
        init_distributed()
    from ..infra.factory import TaskType

    cfg_cls = registry.get_config(cfg.model_type)
    mcfg = cfg_cls(**cfg.scaled_config(scaling_index), sharding_axis_dims=cfg.sharding_axis_dims)
    reg = registry.get_module_registration(TaskType(cfg.model_task), cfg.model_type)
    dev_dtype = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    model = reg.module(mcfg, dtype=dev_dtype, param_dtype=dev_dtype)
    if torch.cuda.is_available():
        model = model.to(torch.device("cuda", rank))
    trainer = get_trainer_class(cfg.trainer_type)(arguments=arguments, model=model, dataset_train=dataset_fn())
    out = trainer.train()
    if rank == 0 and ret is not None:
        ret.put([m for m in out.metrics_history][-1:] or [{}])


class RayDistributedTrainer:
    def __init__(self, config: RayDistributedConfig, arguments, dataset_fn: tp.Callable[[], tp.Any]):
        self.config, self.arguments, self.dataset_fn = config, arguments, dataset_fn

    def train(self, scaling_index: int = 0):
        cfg = self.config
        world = cfg.num_workers
        if world == 1:
            import queue

            q = queue.Queue()
            _worker(0, 1, cfg, scaling_index, self.arguments, self.dataset_fn, q)
            return q.get()
        import torch.multiprocessing as mp

        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_worker, args=(r, world, cfg, scaling_index, self.arguments, self.dataset_fn, q))
                 for r in range(world)]
        for p in procs:
            p.start()
        res = q.get(timeout=3600)
        for p in procs:
            p.join(timeout=120)
        return res
