"""Expert parallelism: the token exchange kernels on one GPU (a rank exchanging with itself), and on 2 / 4 / 8 GPUs the
all-to-all and the all-gather forms around the grouped expert GEMMs against the single-GPU MoE block (forward and
gradients)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_q, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), EP_DISPATCH=mode)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from easydel_b200.layers.moe import MoEBlock
        from easydel_b200.ops import _lib
        from easydel_b200.parallel import ep as EP

        torch.manual_seed(0)
        H, F, E, k, T = 256, 128, 2 * world if world > 4 else 8, 2, 192
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
        used = EP._TOKEN_EXCHANGES if mode == "alltoall" else EP._EXCHANGES
        assert used, "the peer-memory exchange was not used"
        if mode == "alltoall":
            assert all(ex.native for ex in used.values())
            EP.release_token_exchanges()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        out_q.put((rank, errs))
    except Exception:  # noqa: BLE001
        import traceback

        out_q.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["alltoall", "allgather"])
def test_expert_parallel_multi_gpu(world, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in results:
        assert isinstance(errs, dict), errs
        for k, v in errs.items():
            assert v < 4e-2, (rank, k, v)


def test_token_exchange_kernels_one_rank():
    """Plan, dispatch, wait, return and sum on one GPU: every token with a valid expert id travels to the (only)
    rank in token order, rows of unused capacity carry expert id -1, and the returned rows come back to their
    tokens."""
    from easydel_b200.ops import _lib
    from easydel_b200.parallel import ep as EP

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    T, H, k, E = 300, 256, 4, 8
    ex = EP.TokenExchange(None, dev, cap=320, hidden=H, k=k)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx = torch.randint(0, E, (T, k), device=dev)
    idx[::7] = -1                                      # tokens without any expert are not sent
    w = torch.rand(T, k, device=dev)
    for it in range(3):                                # call numbers grow, flags are reused
        plan = ex.plan(idx, E)
        sent = (idx >= 0).any(1)
        n = int(sent.sum())
        assert int(plan.send_count[0]) == n
        assert torch.equal(plan.send_tok[0, :n].long(), sent.nonzero()[:, 0])
        aux = torch.zeros(T, ex.a_bytes // 4, dtype=torch.int32, device=dev)
        aux[:, :k] = w.view(torch.int32)
        aux[:, k:2 * k] = idx.to(torch.int32)
        x_recv, a_recv = ex.dispatch(x, aux, plan, mask_k=k)
        assert int(plan.recv_count[0]) == n
        assert torch.equal(x_recv[:n], x[sent])
        assert torch.equal(a_recv[:n, :k].contiguous().view(torch.float32), w[sent])
        assert torch.equal(a_recv[:n, k:2 * k].long(), idx[sent])
        assert bool((a_recv[n:ex.cap, k:2 * k] == -1).all())
        y = (x_recv.float() * 2).to(torch.bfloat16)
        dw = torch.zeros(ex.cap, ex.ra_bytes // 4, device=dev)
        dw[:, :k] = a_recv[:, :k].contiguous().view(torch.float32) + 1.0
        out, out_aux = ex.ret(y, dw, plan, aux_floats=k)
        assert torch.equal(out[sent], y[:n]) and float(out[~sent].abs().max()) == 0.0
        assert torch.allclose(out_aux[sent], w[sent] + 1.0) and float(out_aux[~sent].abs().max()) == 0.0
    torch.cuda.synchronize()
    _lib.check_status(dev)


def test_alltoall_expert_ffn_one_rank_matches_local_block():
    """The whole all-to-all expert FFN (dispatch -> grouped GEMMs -> return, and its backward) with one rank
    against the same block without any exchange."""
    from easydel_b200.layers.moe import MoEBlock
    from easydel_b200.ops import _lib
    from easydel_b200.parallel import ep as EP

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    H, F, E, k, T = 256, 128, 8, 2, 200
    block = MoEBlock(H, F, E, k, dtype=torch.bfloat16).to(dev)
    x = torch.randn(1, T, H, device=dev).to(torch.bfloat16)
    xa = x.clone().requires_grad_(True)
    ya, _ = block(xa)
    ya.float().square().sum().backward()
    ga = {n: p.grad.clone() if p.grad is not None else p.main_grad.clone() for n, p in block.named_parameters()}
    block.zero_grad(set_to_none=True)
    for p in block.parameters():
        if hasattr(p, "main_grad"):
            p.main_grad.zero_()
    xb = x.clone().requires_grad_(True)
    x2 = xb.reshape(-1, H)
    logits = block.gate(x2)
    w, idx, _ = block.route(logits)
    yb = EP.expert_parallel_ffn_alltoall(block, x2, w, idx).view(1, T, H)
    yb.float().square().sum().backward()
    rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))  # noqa: E731
    assert rel(yb, ya) < 2e-2
    assert rel(xb.grad, xa.grad) < 4e-2
    for n, p in block.named_parameters():
        g = p.grad if p.grad is not None else p.main_grad
        assert rel(g, ga[n]) < 4e-2, n
    torch.cuda.synchronize()
    _lib.check_status(dev)
    EP.release_token_exchanges()
