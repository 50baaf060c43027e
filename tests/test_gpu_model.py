"""End-to-end model numerics on the GPU kernels versus the fp32 CPU reference path."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    from easydel_b200.modules.llama import LlamaConfig

    base = dict(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                max_position_embeddings=1024)
    base.update(kw)
    return LlamaConfig(**base)


def _pair(cfg):
    from easydel_b200.modules.llama import LlamaForCausalLM

    torch.manual_seed(0)
    ref = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)
    gpu = LlamaForCausalLM(copy.deepcopy(cfg), dtype=torch.bfloat16, param_dtype=torch.bfloat16)
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.cuda()
    # the reference sees the same bf16-rounded weights
    ref.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    return ref, gpu


def test_forward_logits_match_cpu_reference():
    ref, gpu = _pair(_cfg())
    ids = torch.randint(0, 2048, (2, 384))
    with torch.no_grad():
        lr = ref(input_ids=ids).logits
        lg = gpu(input_ids=ids.cuda()).logits.float().cpu()
    # reference tolerance for model parity: atol 0.125 on logits
    assert (lr - lg).abs().max().item() < 0.125
    assert torch.nn.functional.cosine_similarity(lr.flatten(), lg.flatten(), dim=0).item() > 0.999


@pytest.mark.parametrize("ckpt", ["", "nothing_saveable"])
def test_loss_and_grads_match_cpu_reference(ckpt):
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig

    ref, gpu = _pair(_cfg(gradient_checkpointing=ckpt))
    gpu.train()
    tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-3), weight_decay=0.0)
    state = EasyDeLState.create(model=gpu, tx=tx, init_opt_state=True)
    ids = torch.randint(0, 2048, (2, 256))
    _, mr = ref.compute_loss(input_ids=ids, labels=ids)
    mr.loss.backward()
    _, mg = gpu.compute_loss(input_ids=ids.cuda(), labels=ids.cuda())
    mg.loss.backward()
    state.flat.fold_param_grads()
    assert abs(mr.loss.item() - mg.loss.item()) < 2e-2
    ref_grads = dict((n, p.grad) for n, p in ref.named_parameters())
    worst = 0.0
    for n, view in state.flat.named_views(state.flat.grad):
        g = view.float().cpu()
        r = ref_grads[n]
        rel = (g - r).norm() / (r.norm() + 1e-8)
        worst = max(worst, rel.item())
        assert rel.item() < 0.08, f"{n}: relative grad error {rel.item():.4f}"
    norm = state.apply_gradients()
    ref_norm = torch.sqrt(sum(p.grad.float().pow(2).sum() for p in ref.parameters()))
    assert abs(norm.item() - ref_norm.item()) / ref_norm.item() < 0.03


def test_packed_segments_isolate_documents():
    ref, gpu = _pair(_cfg())
    ids = torch.randint(0, 2048, (1, 512))
    seg = torch.ones(1, 512, dtype=torch.int32)
    seg[0, 200:] = 2
    with torch.no_grad():
        lr = ref(input_ids=ids, segment_ids=seg).logits
        lg = gpu(input_ids=ids.cuda(), segment_ids=seg.cuda()).logits.float().cpu()
        alone = gpu(input_ids=ids[:, 200:].cuda()).logits.float().cpu()
    assert (lr - lg).abs().max().item() < 0.125
    assert (lg[:, 200:] - alone).abs().max().item() < 0.06


def test_micro_batch_accumulation_matches_full_batch():
    """Gradients accumulated over two half-batches scaled by 1/2 equal the full-batch gradients (LM head included)."""
    from easydel_b200.infra.base_state import EasyDeLState
    from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig

    def grads(split):
        _, gpu = _pair(_cfg())
        gpu.train()
        tx, _ = OptimizerFactory.create("adamw", SchedulerConfig(None, learning_rate=1e-3), weight_decay=0.0)
        st = EasyDeLState.create(model=gpu, tx=tx, init_opt_state=True)
        ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(5)).cuda()
        if split:
            for i in range(2):
                _, m = gpu.compute_loss(input_ids=ids[2 * i:2 * i + 2], labels=ids[2 * i:2 * i + 2], loss_scale=0.5)
                m.loss.backward()
        else:
            _, m = gpu.compute_loss(input_ids=ids, labels=ids)
            m.loss.backward()
        st.flat.fold_param_grads()
        return {n: v.clone() for n, v in st.flat.named_views(st.flat.grad)}

    a, b = grads(False), grads(True)
    for n in a:
        rel = ((a[n] - b[n]).norm() / (a[n].norm() + 1e-8)).item()
        assert rel < 0.03, f"{n}: {rel}"


@pytest.mark.parametrize("policy,targets", [("dots_saveable", None), ("save_only_these_names", ["attn_core", "mlp_gate"]),
                                            ("mlp_notsaveable", None), ("nothing_saveable", None)])
def test_activation_save_policies_match_no_checkpointing(policy, targets):
    """Every save policy gives the gradients of the un-checkpointed model; policies that keep op outputs launch
    fewer kernels in the recompute than full recomputation does."""
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
    from easydel_b200.ops import _lib

    def run(pol, tg):
        cfg = LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=64, max_position_embeddings=512,
                          gradient_checkpointing=pol, gradient_checkpointing_targets=tg)
        torch.manual_seed(0)
        m = LlamaForCausalLM(cfg, dtype=torch.bfloat16, param_dtype=torch.bfloat16).cuda().train()
        ids = torch.randint(0, 2048, (2, 256), generator=torch.Generator().manual_seed(1)).cuda()
        n0 = _lib.launch_count
        _, met = m.compute_loss(input_ids=ids, labels=ids)
        met.loss.backward()
        torch.cuda.synchronize()
        return float(met.loss), {k: p.grad.float().clone() for k, p in m.named_parameters()}, _lib.launch_count - n0

    loss0, g0, _ = run("everything_saveable", None)
    loss1, g1, n1 = run(policy, targets)
    assert abs(loss0 - loss1) < 1e-3
    for k in g0:
        assert torch.allclose(g0[k], g1[k], atol=2e-3, rtol=2e-2), k
    if policy != "nothing_saveable":
        _, _, n_full = run("nothing_saveable", None)
        assert n1 < n_full, (n1, n_full)
