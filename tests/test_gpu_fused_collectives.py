"""GEMM fused with reduce-scatter / all-gather (csrc/gemm_collective.cu).

One-rank cases run the whole kernel path (tile pipeline, peer-store epilogue, flags, shard reduction,
copier ring) on a single GPU; the multi-GPU cases spawn one process per GPU and compare against
torch.distributed collectives around an fp32 matmul.
"""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)).item()


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1024, 1000, 1152), (128, 264, 64)])
def test_gemm_reduce_scatter_one_rank(M, N, K):
    from easydel_b200.parallel.fused import GemmReduceScatter

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
    op = GemmReduceScatter(None, M, N, dev)
    for it in range(3):   # alternates slots, epochs grow
        out = op(a, w, residual=res if it else None, bias=bias if it == 2 else None)
        ref = a.float() @ w.float().t()
        if it:
            ref = ref + res.float()
        if it == 2:
            ref = ref + bias.float()
        assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("Ms,N,K", [(256, 512, 256), (1024, 520, 1024)])
def test_allgather_gemm_one_rank(Ms, N, K):
    from easydel_b200.parallel.fused import AllGatherGemm

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    a = torch.randn(Ms, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    op = AllGatherGemm(None, Ms, K, dev, n_copy=4)
    op.gathered.fill_(7.0)
    c, g = op(a, w, copy_own=True)
    assert _rel_err(c, a.float() @ w.float().t()) < 1e-2
    assert torch.equal(g, a)   # the copier ring moved every byte


def test_fused_collectives_mn_major_weight_one_rank():
    """The data-gradient forms: the second operand is stored [K, N] (a linear layer's weight read as dY @ W)."""
    from easydel_b200.parallel.fused import AllGatherGemm, GemmReduceScatter

    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    M, N, K = 512, 768, 384
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w_kn = torch.randn(K, N, device=dev, dtype=torch.bfloat16) * 0.05
    out = GemmReduceScatter(None, M, N, dev)(a, w_kn, b_mn=True)
    assert _rel_err(out, a.float() @ w_kn.float()) < 1e-2
    c, g = AllGatherGemm(None, M, K, dev)(a, w_kn, b_mn=True)
    assert _rel_err(c, a.float() @ w_kn.float()) < 1e-2
    assert torch.equal(g, a)


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from easydel_b200.ops import _lib
        from easydel_b200.parallel.fused import (AllGatherGemm, GemmReduceScatter, allgather_gemm_reference,
                                                 gemm_reduce_scatter_reference)

        group = dist.group.WORLD
        errs = {}
        # GEMM -> reduce-scatter
        M, N, Kr = 256 * world, 1024, 512
        torch.manual_seed(100 + rank)
        a = torch.randn(M, Kr, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, Kr, device=dev, dtype=torch.bfloat16) * 0.05
        res = torch.randn(M // world, N, device=dev, dtype=torch.bfloat16)
        op = GemmReduceScatter(group, M // world, N, dev)
        for it in range(4):
            out = op(a, w, residual=res)
            ref = gemm_reduce_scatter_reference(a, w, group, residual=res)
            errs[f"rs{it}"] = _rel_err(out, ref)
            a = a * 0.5 + 0.1
        # all-gather -> GEMM
        Ms, K = 384, 1024
        a_sh = torch.randn(Ms, K, device=dev, dtype=torch.bfloat16)
        w2 = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
        ag = AllGatherGemm(group, Ms, K, dev, n_copy=8)
        for it in range(3):
            c, g = ag(a_sh, w2)
            cref, gref = allgather_gemm_reference(a_sh, w2, group)
            errs[f"ag{it}"] = _rel_err(c, cref)
            errs[f"ag_gather{it}"] = float(not torch.equal(g, gref))
            a_sh = a_sh * 0.5 - 0.2
        torch.cuda.synchronize()
        _lib.check_status(dev)
        out_q.put((rank, errs))
    except Exception as e:  # noqa: BLE001
        out_q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_collectives_multi_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in results:
        assert isinstance(errs, dict), errs
        for k, v in errs.items():
            assert v < 1.5e-2, (rank, k, v)
