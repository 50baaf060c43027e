"""Expert parallelism on 2 GPUs: peer-memory all-gather / reduce-scatter around the grouped expert GEMMs agree
with the single-GPU MoE block (forward and gradients)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from easydel_b200.layers.moe import MoEBlock
        from easydel_b200.ops import _lib
        from easydel_b200.parallel import ep as EP

        torch.manual_seed(0)
        H, F, E, k, T = 256, 128, 8, 2, 192
        full = MoEBlock(H, F, E, k, dtype=torch.bfloat16).to(dev)
        ep = MoEBlock(H, F, E, k, dtype=torch.bfloat16, ep_size=world, ep_rank=rank,
                      ep_group=dist.group.WORLD).to(dev)
        El = E // world
        with torch.no_grad():
            for p in full.parameters():
                dist.broadcast(p, src=0)
            ep.gate.weight.copy_(full.gate.weight)
            ep.gate_up_proj.weight.copy_(full.gate_up_proj.weight[rank * El:(rank + 1) * El])
            ep.down_proj.weight.copy_(full.down_proj.weight[rank * El:(rank + 1) * El])
        xs = torch.randn(world, 1, T, H, device=dev, dtype=torch.bfloat16)
        dist.broadcast(xs, src=0)
        errs = {}
        for it in range(2):     # two rounds: the exchange slots alternate
            x_full = xs.reshape(1, world * T, H).clone().requires_grad_(True)
            y_full, _ = full(x_full)
            y_full.float().square().sum().backward()
            x = xs[rank].clone().requires_grad_(True)
            y, _ = ep(x)
            y.float().square().sum().backward()
            sl = slice(rank * T, (rank + 1) * T)
            rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))  # noqa: E731
            errs[f"y{it}"] = rel(y, y_full[:, sl])
            errs[f"dx{it}"] = rel(x.grad, x_full.grad[:, sl])
            g_ep = ep.gate_up_proj.weight.main_grad if hasattr(ep.gate_up_proj.weight, "main_grad") \
                else ep.gate_up_proj.weight.grad
            g_full = full.gate_up_proj.weight.main_grad if hasattr(full.gate_up_proj.weight, "main_grad") \
                else full.gate_up_proj.weight.grad
            if g_ep is not None and g_full is not None:
                errs[f"dw{it}"] = rel(g_ep, g_full[rank * El:(rank + 1) * El])
            for m in (ep, full):
                m.zero_grad(set_to_none=True)
        assert EP._EXCHANGES, "the peer-memory exchange was not used"
        torch.cuda.synchronize()
        _lib.check_status(dev)
        out_q.put((rank, errs))
    except Exception:  # noqa: BLE001
        import traceback

        out_q.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_gpus():
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in results:
        assert isinstance(errs, dict), errs
        for k, v in errs.items():
            assert v < 4e-2, (rank, k, v)
