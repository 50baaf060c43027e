"""Context-parallel attention on 2 GPUs: forward and gradients against dense attention over the gathered
sequence (one process per GPU; keys / values are read from the peer's memory by the attention kernel)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from easydel_b200.ops import _lib
        from easydel_b200.parallel.context_parallel import (ContextParallelAttention,
                                                            context_parallel_attention_reference)

        T, Hq, Hkv, D = 384, 8, 2, 128
        cp = ContextParallelAttention(dist.group.WORLD, T, Hkv, D, dev)
        errs = {}
        for causal in (True, False):
            torch.manual_seed(10 + rank)
            q = torch.randn(T, Hq, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
            k = torch.randn(T, Hkv, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
            v = torch.randn(T, Hkv, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
            w = torch.randn(T, Hq, D, device=dev, dtype=torch.bfloat16)
            o = cp(q, k, v, causal=causal)
            (o.float() * w.float()).sum().backward()
            got = (o.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone())
            # oracle: gather the full sequence on every rank, differentiate the dense computation
            qs = [torch.empty_like(q) for _ in range(world)]
            ks = [torch.empty_like(k) for _ in range(world)]
            vs = [torch.empty_like(v) for _ in range(world)]
            ws = [torch.empty_like(w) for _ in range(world)]
            for dst, src in ((qs, q), (ks, k), (vs, v), (ws, w)):
                dist.all_gather(dst, src.detach().contiguous())
            qf = torch.cat(qs).float().requires_grad_(True)
            kf = torch.cat(ks).float().requires_grad_(True)
            vf = torch.cat(vs).float().requires_grad_(True)
            from easydel_b200.ops import reference as R

            of = R.attention(qf[None], kf[None], vf[None], causal=causal)[0]
            (of * torch.cat(ws).float()).sum().backward()
            sl = slice(rank * T, (rank + 1) * T)
            ref = (of[sl].detach(), qf.grad[sl], kf.grad[sl], vf.grad[sl])
            for name, a, b in zip(("o", "dq", "dk", "dv"), got, ref):
                errs[f"{name}_{'causal' if causal else 'full'}"] = float(
                    (a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))
        torch.cuda.synchronize()
        _lib.check_status(dev)
        q_out.put((rank, errs))
    except Exception as e:  # noqa: BLE001
        import traceback

        q_out.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


def test_context_parallel_attention_two_gpus():
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 200)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in results:
        assert isinstance(errs, dict), errs
        for k, v in errs.items():
            assert v < 3e-2, (rank, k, v)
