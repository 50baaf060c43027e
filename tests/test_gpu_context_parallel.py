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


def _spawn(target, world, *args):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 200)
    procs = [ctx.Process(target=target, args=(r, world, port, q, *args)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return results


@pytest.mark.parametrize("world", [2, 4, 8])
def test_context_parallel_attention_multi_gpu(world):
    for rank, errs in _spawn(_worker, world):
        assert isinstance(errs, dict), errs
        for k, v in errs.items():
            assert v < 3e-2, (rank, k, v)


def _model_worker(rank, world, port, q_out, layout, impl):
    """A Llama block stack with the sequence sharded over the sp axis (attn_mechanism="ring") against the same model
    on the whole sequence: loss and the gradient of the embedding table."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
        from easydel_b200.ops import _lib
        from easydel_b200.parallel import context_parallel as CP
        from easydel_b200.parallel.mesh import DeviceMesh

        kw = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=64, max_position_embeddings=4096)
        one = LlamaConfig(**kw)
        one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
        torch.manual_seed(3)
        full = LlamaForCausalLM(one, dtype=torch.bfloat16, param_dtype=torch.bfloat16).to(dev)
        cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, 1, world), attn_mechanism="ring", ring_attention_layout=layout,
                          ring_attention_impl=impl, **kw)
        model = LlamaForCausalLM(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16).to(dev)
        model.load_state_dict(full.state_dict())
        T = 256 * world
        ids = torch.randint(0, 512, (1, T), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
        dist.broadcast(ids, src=0)
        _, m_full = full.compute_loss(input_ids=ids, labels=ids)
        m_full.loss.backward()
        _, m_cp = model.compute_loss(input_ids=ids, labels=ids)
        m_cp.loss.backward()

        def grad(m, name):
            p = dict(m.named_parameters())[name]
            return (p.main_grad if getattr(p, "main_grad", None) is not None else p.grad).float().clone()

        errs = {"loss": abs(float(m_full.loss) - float(m_cp.loss)) / max(1.0, abs(float(m_full.loss)))}
        for name in ("model.embed_tokens.weight", "model.layers.0.self_attn.qkv_proj.weight"):
            g = grad(model, name)
            dist.all_reduce(g)          # every rank holds the partial gradient of its tokens
            ref = grad(full, name)
            errs[name] = float((g - ref).abs().max() / ref.abs().max().clamp_min(1e-6))
        torch.cuda.synchronize()
        _lib.check_status(dev)
        CP.release_peer_buffers()
        q_out.put((rank, errs))
    except Exception:  # noqa: BLE001
        import traceback

        q_out.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,layout,impl", [(2, "zigzag", "gather"), (2, "contiguous", "peer"),
                                               (4, "zigzag", "gather"), (8, "zigzag", "gather")])
def test_ring_attention_model_matches_unsharded(world, layout, impl):
    for rank, errs in _spawn(_model_worker, world, layout, impl):
        assert isinstance(errs, dict), errs
        assert errs.pop("loss") < 5e-3, (rank, errs)
        for k, v in errs.items():
            assert v < 6e-2, (rank, k, v)
