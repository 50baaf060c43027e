"""Multi-process (gloo, CPU ranks) tests of the mesh and the sharded optimizer step."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world, *args, timeout: float = 240.0):
    """Spawns ``world`` gloo ranks; a rank that never finishes fails the test instead of hanging it."""
    port = _free_port()
    ctx = mp.spawn(_entry, args=(fn, world, port, args), nprocs=world, join=False)
    import time

    deadline = time.time() + timeout
    while not ctx.join(timeout=1.0):
        if time.time() > deadline:
            for p in ctx.processes:
                if p.is_alive():
                    p.terminate()
            raise TimeoutError(f"distributed test did not finish within {timeout}s")


def _entry(rank, fn, world, port, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        fn(rank, world, *args)
        dist.barrier()      # nobody tears its sockets down while a peer still has transfers in flight
    finally:
        dist.destroy_process_group()


def _tiny(seed):
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32)
    torch.manual_seed(seed)
    return LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)


def _sharded_step_worker(rank, world):
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig

    model = _tiny(seed=rank)  # different init per rank: the broadcast must make them equal
    tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.01,
                                    clip_grad=1.0)
    state = EasyDeLState.create(model=model, tx=tx, init_opt_state=True)
    assert state._dist is not None and state.flat.world_size == world
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 128, (2 * world, 16), generator=g)
    mine = data[2 * rank:2 * rank + 2]
    for _ in range(2):
        _, met = model.compute_loss(input_ids=mine, labels=mine)
        met.loss.backward()
        norm = state.apply_gradients()
    flat_w = state.flat.work.clone()
    gathered = [torch.empty_like(flat_w) for _ in range(world)]
    dist.all_gather(gathered, flat_w)
    for t in gathered:
        assert torch.equal(t, gathered[0]), "ranks diverged"
    if rank == 0:
        # single-process reference on the full batch (mean over ranks == mean over the global batch here)
        from easydel_b200.parallel.mesh import DeviceMesh

        ref = _tiny(seed=0)
        ref.config.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), ref.config.sharding_axis_names, rank=0, world_size=1))
        tx2, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.01,
                                         clip_grad=1.0)
        st2 = EasyDeLState.create(model=ref, tx=tx2, init_opt_state=True)
        assert st2._dist is None
        for _ in range(2):
            for r in range(world):
                mb = data[2 * r:2 * r + 2]
                _, met = ref.compute_loss(input_ids=mb, labels=mb, loss_scale=1.0 / world)
                met.loss.backward()
            n2 = st2.apply_gradients()
        a = dict(ref.named_parameters())
        for n_, p in model.named_parameters():
            assert torch.allclose(p, a[n_], atol=2e-5), n_
        assert abs(float(norm) - float(n2)) < 1e-4


def _mesh_worker(rank, world):
    from easydel_b200.parallel.mesh import DeviceMesh

    mesh = DeviceMesh.create((1, -1, 1, 2, 1), ("dp", "fsdp", "ep", "tp", "sp"))
    assert mesh.shape == {"dp": 1, "fsdp": world // 2, "ep": 1, "tp": 2, "sp": 1}
    tpg = mesh.get_group("tp")
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=tpg)
    base = rank - rank % 2
    assert t.item() == base + base + 1
    assert mesh.axis_index("tp") == rank % 2 and mesh.axis_index("fsdp") == rank // 2
    fg = mesh.get_group("fsdp")
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=fg)
    assert t.item() == sum(r for r in range(world) if r % 2 == rank % 2)


def test_mesh_groups_4_ranks():
    _run(_mesh_worker, 4)


def test_sharded_optimizer_matches_single_process():
    _run(_sharded_step_worker, 2)


def _ep_worker(rank, world, mode="alltoall"):
    """Expert-parallel MoE block (2 local experts per rank) equals the single-rank block on each rank's tokens,
    in outputs and in gradients of inputs, router weights and expert weights, for both token-exchange forms."""
    import os

    from easydel_b200.layers.moe import MoEBlock

    os.environ["EP_DISPATCH"] = mode
    torch.manual_seed(0)
    H, F, E, k, T = 16, 32, 2 * world, 2, 6
    full = MoEBlock(H, F, E, k, dtype=torch.float32)
    ep = MoEBlock(H, F, E, k, dtype=torch.float32, ep_size=world, ep_rank=rank, ep_group=dist.group.WORLD)
    El = E // world
    with torch.no_grad():
        ep.gate.weight.copy_(full.gate.weight)
        ep.gate_up_proj.weight.copy_(full.gate_up_proj.weight[rank * El:(rank + 1) * El])
        ep.down_proj.weight.copy_(full.down_proj.weight[rank * El:(rank + 1) * El])
    xs = torch.randn(world, 1, T, H)
    x_full = xs.reshape(1, world * T, H).clone().requires_grad_(True)
    y_full, _ = full(x_full)
    y_full.square().sum().backward()
    x = xs[rank].clone().requires_grad_(True)
    y, _ = ep(x)
    y.square().sum().backward()
    assert torch.allclose(y, y_full[:, rank * T:(rank + 1) * T], atol=1e-5)
    assert torch.allclose(x.grad, x_full.grad[:, rank * T:(rank + 1) * T], atol=1e-5)
    assert torch.allclose(ep.gate_up_proj.weight.grad, full.gate_up_proj.weight.grad[rank * El:(rank + 1) * El],
                          atol=1e-5)
    g = ep.gate.weight.grad.clone()
    dist.all_reduce(g)     # the router is replicated: its gradient is the sum over ranks
    assert torch.allclose(g, full.gate.weight.grad, atol=1e-5)


@pytest.mark.parametrize("mode,world", [("alltoall", 2), ("allgather", 2), ("alltoall", 4)])
def test_expert_parallel_block_matches_single_rank(mode, world):
    _run(_ep_worker, world, mode)


def _ep_step_worker(rank, world):
    """One optimizer step of an expert-parallel model equals the single-rank step on the union of the data."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.modules.families import Qwen3MoeConfig, Qwen3MoeForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
    from easydel_b200.parallel.mesh import DeviceMesh

    kw = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=8, moe_intermediate_size=16, num_experts=4, num_experts_per_tok=2,
              norm_topk_prob=True, router_aux_loss_coef=0.0, max_position_embeddings=32)
    full_cfg = Qwen3MoeConfig(**kw)
    full_cfg.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), full_cfg.sharding_axis_names, 0, 1))
    torch.manual_seed(0)
    full = Qwen3MoeForCausalLM(full_cfg, dtype=torch.float32, param_dtype=torch.float32)
    cfg = Qwen3MoeConfig(sharding_axis_dims=(1, 1, world, 1, 1), **kw)
    model = Qwen3MoeForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    El = 4 // world
    sd = {}
    for k, v in full.state_dict().items():
        sd[k] = v[rank * El:(rank + 1) * El].clone() if (v.dim() == 3 and v.shape[0] == 4) else v.clone()
    model.load_state_dict(sd)
    ids = torch.randint(0, 64, (world, 2, 16), generator=torch.Generator().manual_seed(5))

    def step(m, batch):
        tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.0,
                                        clip_grad=0.5)
        st = EasyDeLState.create(model=m, tx=tx, init_opt_state=True)
        _, met = m.compute_loss(input_ids=batch, labels=batch)
        met.loss.backward()
        return st.apply_gradients()

    n_full = step(full, ids.reshape(world * 2, 16))
    n_ep = step(model, ids[rank])
    assert abs(float(n_full) - float(n_ep)) < 1e-4 * max(1.0, float(n_full)), (float(n_full), float(n_ep))
    ref = full.state_dict()
    for k, v in model.state_dict().items():
        want = ref[k][rank * El:(rank + 1) * El] if (ref[k].dim() == 3 and ref[k].shape[0] == 4) else ref[k]
        assert torch.allclose(v, want, atol=2e-5), k


def test_expert_parallel_training_step_matches_single_rank():
    _run(_ep_step_worker, 2)


def _tp_checkpoint_worker(rank, world, tmp):
    """A tensor-parallel model (and its optimizer state) saves full tensors; a tp = 1 model loads them and gives
    the same logits as the tp = 2 forward; loading the same files back at tp = 2 restores every shard."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
    from easydel_b200.parallel.mesh import DeviceMesh

    kw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=32)
    torch.manual_seed(3)
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    model.shard_model()
    tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.0)
    state = EasyDeLState.create(model=model, tx=tx, init_opt_state=True)
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(1))
    _, met = model.compute_loss(input_ids=ids, labels=ids)
    met.loss.backward()
    state.apply_gradients()
    with torch.no_grad():
        logits_tp = model(input_ids=ids).logits
    state.save_state(tmp)
    dist.barrier()
    local_before = {k: v.clone() for k, v in model.state_dict().items()}
    m_before = {k: v.clone() for k, v in state.flat.opt_state.items()}
    # tp = 2 round trip of weights and optimizer state
    for p in model.parameters():
        p.data.zero_()
    for v in state.flat.opt_state.values():
        v.zero_()
    from easydel_b200.io import checkpoint as CK

    CK.load_state_into(state, tmp)
    for k, v in model.state_dict().items():
        assert torch.equal(v, local_before[k]), k
    for k, v in state.flat.opt_state.items():
        assert torch.equal(v, m_before[k]), k
    if rank == 0:
        import json

        with open(os.path.join(tmp, "tensorstore_index.json")) as f:
            idx = json.load(f)
        shapes = {e["path"]: e["shape"] for e in idx["prefixes"]["model"]}
        qk = [v for k, v in shapes.items() if k.endswith("self_attn/q_proj/kernel")][0]
        assert qk == [32, 32], qk      # full (in, out), not the tp-local half
        one = LlamaConfig(**kw)
        one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
        ref = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32)
        CK.load_weights_into(ref, tmp)
        with torch.no_grad():
            logits_one = ref(input_ids=ids).logits
        assert torch.allclose(logits_one, logits_tp, atol=1e-5), (logits_one - logits_tp).abs().max()
    dist.barrier()


def test_tensor_parallel_checkpoint_roundtrip(tmp_path):
    _run(_tp_checkpoint_worker, 2, str(tmp_path))


def _tp_clip_worker(rank, world):
    """A clipped optimizer step at tp = 2 uses one global gradient norm on both ranks (sharded parameters count
    every rank's piece, replicated ones once) and matches the single-process step."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
    from easydel_b200.parallel.mesh import DeviceMesh
    from easydel_b200.utils.parameters_transformation import shard_internal_state_for_tp

    kw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=32)
    one = LlamaConfig(**kw)
    one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
    torch.manual_seed(11)
    full = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32)
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    model.load_state_dict(shard_internal_state_for_tp(model, full.state_dict()))
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(2))

    def step(m):
        tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.0,
                                        clip_grad=0.05)
        st = EasyDeLState.create(model=m, tx=tx, init_opt_state=True)
        _, met = m.compute_loss(input_ids=ids, labels=ids)
        met.loss.backward()
        return st.apply_gradients()

    n_full, n_tp = step(full), step(model)
    assert model.model.sp.active and model.model.sp.rows_local == 16, "the tp model ran sequence-parallel"
    assert float(n_full) > 0.05, "the step must actually clip"
    assert abs(float(n_full) - float(n_tp)) < 1e-4 * max(1.0, float(n_full)), (float(n_full), float(n_tp))
    norms = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(norms, n_tp.detach().reshape(1).float())
    assert all(torch.equal(n, norms[0]) for n in norms)
    want = shard_internal_state_for_tp(model, full.state_dict())
    for k, v in model.state_dict().items():
        assert torch.allclose(v, want[k], atol=2e-5), k
    emb = model.state_dict()["model.embed_tokens.weight"].clone()
    parts = [torch.empty_like(emb) for _ in range(world)]
    dist.all_gather(parts, emb)
    assert torch.equal(parts[0], parts[1]), "replicated weights diverged across the tensor-parallel ranks"


def test_tensor_parallel_clip_uses_global_norm():
    _run(_tp_clip_worker, 2)


def _tp_logprob_worker(rank, world):
    """Sequence log-probabilities (the DPO / GRPO building block) of a tensor-parallel model running on
    sequence-sharded activations equal the single-process ones, in value and in gradients."""
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.parallel.mesh import DeviceMesh
    from easydel_b200.trainers._logprob_utils import sequence_logprobs
    from easydel_b200.utils.parameters_transformation import shard_internal_state_for_tp

    kw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=32)
    one = LlamaConfig(**kw)
    one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
    torch.manual_seed(5)
    full = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32)
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    model.load_state_dict(shard_internal_state_for_tp(model, full.state_dict()))
    ids = torch.randint(0, 128, (3, 12), generator=torch.Generator().manual_seed(4))
    mask = torch.ones_like(ids)
    mask[1, 9:] = 0
    wts = torch.tensor([1.0, -2.0, 0.5])

    def run(m):
        s, n, _ = sequence_logprobs(m, ids, attention_mask=mask, loss_mask=mask)
        (s * wts).sum().backward()
        return s.detach(), n

    s_full, n_full = run(full)
    s_tp, n_tp = run(model)
    assert model.model.sp.active and getattr(model, "sp_partial_grads", False)
    assert torch.allclose(s_tp, s_full, atol=1e-5) and torch.equal(n_tp, n_full)
    want = shard_internal_state_for_tp(model, {k: p.grad for k, p in full.named_parameters()})
    mods = dict(model.named_modules())
    for k, p in model.named_parameters():
        g = p.grad.clone()
        mod = mods[k.rpartition(".")[0]]
        sharded = getattr(mod, "tp_size", 1) > 1 and getattr(mod, "parallel_style", "") in ("column", "row") \
            and not (mod.parallel_style == "row" and k.endswith("bias"))
        if not sharded:
            dist.all_reduce(g)     # partial sums over the token shards
        assert torch.allclose(g, want[k], atol=1e-5), k


def test_tensor_parallel_sequence_logprobs_match():
    _run(_tp_logprob_worker, 2)


def _fsdp_sharded_worker(rank, world, tmp):
    """Parameter-sharded layers (every rank keeps 1/N of each decoder layer, layers gathered one at a time,
    gradients reduced per layer) take the same optimizer steps as a single process on the whole batch, over two
    accumulation micro-batches, and save / reload a checkpoint that a plain model reads."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.io import checkpoint as CK
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
    from easydel_b200.parallel.mesh import DeviceMesh

    kw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=32, gradient_checkpointing="nothing_saveable")

    def tx():
        return OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.01,
                                       clip_grad=0.1)[0]

    torch.manual_seed(rank)      # different initial weights per rank: rank 0's must win
    model = LlamaForCausalLM(LlamaConfig(fsdp_parameter_sharding="sharded", **kw), dtype=torch.float32,
                             param_dtype=torch.float32).train()
    state = EasyDeLState.create(model=model, tx=tx(), init_opt_state=True)
    rt = state._fsdp
    assert rt is not None and model.model.fsdp_layers is rt and rt.world == world
    assert model.model.layers[0].mlp.down_proj.weight.numel() == 0     # no full copy outside a layer's turn
    data = torch.randint(0, 128, (2, 2 * world, 16), generator=torch.Generator().manual_seed(7))
    for _ in range(2):
        for mb in range(2):
            mine = data[mb, 2 * rank:2 * rank + 2]
            _, met = model.compute_loss(input_ids=mine, labels=mine, loss_scale=0.5)
            met.loss.backward()
        norm = state.apply_gradients()
    # single-process reference
    one = LlamaConfig(**kw)
    one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
    torch.manual_seed(0)
    ref = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32).train()
    st2 = EasyDeLState.create(model=ref, tx=tx(), init_opt_state=True)
    for _ in range(2):
        for mb in range(2):
            for r in range(world):
                b = data[mb, 2 * r:2 * r + 2]
                _, met = ref.compute_loss(input_ids=b, labels=b, loss_scale=0.5 / world)
                met.loss.backward()
        n2 = st2.apply_gradients()
    assert abs(float(norm) - float(n2)) < 1e-4 * max(1.0, float(n2)), (float(norm), float(n2))
    rt.materialize()
    want = dict(ref.named_parameters())
    for n_, p in model.named_parameters():
        assert torch.allclose(p, want[n_], atol=3e-5), n_
    rt.dematerialize()
    # evaluation forward on the sharded model
    with torch.no_grad():
        ids = data[0, :2]
        a = model(input_ids=ids).logits
        b = ref(input_ids=ids).logits
    assert torch.allclose(a, b, atol=1e-4)
    # checkpoint: full tensors on disk, readable by a plain model; optimizer moments come back into the shards
    state.save_state(tmp)
    dist.barrier()
    mu_before = rt.opt_state["mu"].clone()
    rt.opt_state["mu"].zero_()
    rt.wshard.zero_()
    CK.load_state_into(state, tmp)
    assert torch.equal(rt.opt_state["mu"], mu_before)
    with torch.no_grad():
        assert torch.allclose(model(input_ids=ids).logits, b, atol=1e-4)
    if rank == 0:
        plain = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32)
        CK.load_weights_into(plain, tmp)
        with torch.no_grad():
            assert torch.allclose(plain(input_ids=ids).logits, b, atol=1e-4)
    dist.barrier()


def test_fsdp_parameter_sharded_layers_match_single_process(tmp_path):
    _run(_fsdp_sharded_worker, 2, str(tmp_path))


def _ring_worker(rank, world, layout):
    """Sequence sharded over the sp axis (attn_mechanism="ring"): loss, gradient norm and the updated weights of a
    clipped optimizer step equal the single-process step on the whole sequences; every rank ends with the same
    weights. Also the sharding helpers' bookkeeping."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
    from easydel_b200.parallel import context_parallel as CP
    from easydel_b200.parallel.mesh import DeviceMesh

    pos = torch.cat([CP.shard_positions(32, r, world, layout) for r in range(world)])
    assert sorted(pos.tolist()) == list(range(32))
    if layout == "zigzag":
        assert CP.shard_positions(32, 0, 2, "zigzag").tolist() == list(range(0, 8)) + list(range(24, 32))
    kw = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=64)
    one = LlamaConfig(**kw)
    one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
    torch.manual_seed(5)
    full = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32)
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, 1, world), attn_mechanism="ring", ring_attention_layout=layout, **kw)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    model.load_state_dict(full.state_dict())
    assert model.model.cp_group is not None and model.model.layers[0].self_attn.cp_layout == layout
    ids = torch.randint(0, 128, (2, 32), generator=torch.Generator().manual_seed(2))
    labels = ids.clone()
    labels[0, :5] = -100

    def step(m):
        tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-2), weight_decay=0.0,
                                        clip_grad=0.05)
        st = EasyDeLState.create(model=m, tx=tx, init_opt_state=True)
        _, met = m.compute_loss(input_ids=ids, labels=labels)
        met.loss.backward()
        return met.loss.detach(), st.apply_gradients()

    (l_full, n_full), (l_cp, n_cp) = step(full), step(model)
    assert abs(float(l_full) - float(l_cp)) < 1e-5 * max(1.0, float(l_full)), (float(l_full), float(l_cp))
    assert abs(float(n_full) - float(n_cp)) < 1e-4 * max(1.0, float(n_full)), (float(n_full), float(n_cp))
    for k, v in model.state_dict().items():
        assert torch.allclose(v, full.state_dict()[k], atol=2e-5), k
    w = model.state_dict()["model.layers.1.mlp.down_proj.weight"].clone()
    parts = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(parts, w)
    assert all(torch.equal(p, parts[0]) for p in parts)


@pytest.mark.parametrize("layout,world", [("zigzag", 2), ("contiguous", 2), ("zigzag", 4)])
def test_ring_attention_sequence_sharded_step_matches_single_process(layout, world):
    _run(_ring_worker, world, layout)


def _tp_esurge_worker(rank, world):
    """An eSurge engine over a tensor-parallel model (every rank runs the same scheduler on the same requests; the
    LM head is evaluated vocabulary-parallel) produces the tokens of the unsharded model's greedy generation."""
    from easydel_b200.inference import SamplingParams
    from easydel_b200.inference.esurge import eSurge
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.parallel.mesh import DeviceMesh
    from easydel_b200.utils.parameters_transformation import shard_internal_state_for_tp

    kw = dict(vocab_size=256, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512, eos_token_id=255)
    one = LlamaConfig(**kw)
    one.set_model_mesh(DeviceMesh((1, 1, 1, 1, 1), one.sharding_axis_names, 0, 1))
    torch.manual_seed(4)
    full = LlamaForCausalLM(one, dtype=torch.float32, param_dtype=torch.float32).eval()
    cfg = LlamaConfig(sharding_axis_dims=(1, 1, 1, world, 1), **kw)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    model.load_state_dict(shard_internal_state_for_tp(model, full.state_dict()))
    eng = eSurge(model, max_model_len=512, max_num_seqs=4, max_num_batched_tokens=64, num_pages=12)
    assert eng.runner.tp_group is not None
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 250, (n,), generator=g).tolist() for n in (150, 9)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ref = full.generate(torch.tensor([p]), max_new_tokens=10, eos_token_id=-1).sequences[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref, (rank, o.outputs[0].token_ids, ref)
    eng.close()


def test_esurge_tensor_parallel_matches_unsharded_generate():
    _run(_tp_esurge_worker, 2)


def _expert_tensor_worker(rank, world):
    """Expert tensor mode: experts spread over the tensor-parallel group, identical tokens on every rank, partial
    outputs summed. Output, input gradient, router gradient and the local experts' gradients equal the unsharded
    block's."""
    from easydel_b200.layers.moe import MoEBlock

    torch.manual_seed(0)
    H, F, E, k, T = 16, 32, 2 * world, 2, 10
    full = MoEBlock(H, F, E, k, dtype=torch.float32)
    etm = MoEBlock(H, F, E, k, dtype=torch.float32, tp_size=world, tp_rank=rank, tp_group=dist.group.WORLD,
                   expert_tensor_mode=True)
    assert etm.expert_tensor_mode and etm.num_local_experts == 2 and etm.gate_up_proj.weight._ep_over_tp
    El = E // world
    with torch.no_grad():
        etm.gate.weight.copy_(full.gate.weight)
        etm.gate_up_proj.weight.copy_(full.gate_up_proj.weight[rank * El:(rank + 1) * El])
        etm.down_proj.weight.copy_(full.down_proj.weight[rank * El:(rank + 1) * El])
    x0 = torch.randn(1, T, H)
    xa = x0.clone().requires_grad_(True)
    ya, _ = full(xa)
    ya.square().sum().backward()
    xb = x0.clone().requires_grad_(True)
    yb, _ = etm(xb)
    yb.square().sum().backward()
    assert torch.allclose(yb, ya, atol=1e-5)
    assert torch.allclose(xb.grad, xa.grad, atol=1e-5)
    assert torch.allclose(etm.gate.weight.grad, full.gate.weight.grad, atol=1e-5)
    assert torch.allclose(etm.down_proj.weight.grad, full.down_proj.weight.grad[rank * El:(rank + 1) * El], atol=1e-5)


def test_expert_tensor_mode_matches_unsharded_block():
    _run(_expert_tensor_worker, 2)
