"""Expert FFN kernels (routing tables, grouped GEMMs, combine) against the dense per-expert oracle."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(T, H, Fd, E, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * Fd, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, Fd, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    w, idx = torch.softmax(logits, -1).topk(k, -1)
    w = w / w.sum(-1, keepdim=True)
    return x, wgu, wd, w, idx


@pytest.mark.parametrize("T,H,Fd,E,k", [(300, 256, 384, 8, 2), (1000, 512, 768, 16, 4), (64, 128, 256, 32, 8)])
def test_moe_ffn_forward_backward(T, H, Fd, E, k):
    from easydel_b200.ops import moe_kernels as MK, reference as R

    x, wgu, wd, w, idx = _setup(T, H, Fd, E, k)
    xr, wgur, wdr, wr = (t.detach().float().requires_grad_(True) for t in (x, wgu, wd, w))
    ref = R.moe_experts(xr, wgur, wdr, wr, idx)
    dy = torch.randn_like(ref)
    ref.backward(dy)
    xg, wgug, wdg, wg = (t.detach().clone().requires_grad_(True) for t in (x, wgu, wd, w))
    y = MK.moe_ffn(xg, wgug, wdg, wg, idx)
    assert torch.allclose(y.float(), ref.detach(), atol=3e-2, rtol=3e-2), (y.float() - ref).abs().max()
    y.backward(dy.to(y.dtype))

    def close(a, b, name):
        rel = ((a.float() - b).norm() / (b.norm() + 1e-8)).item()
        assert rel < 0.05, f"{name}: {rel}"

    close(xg.grad, xr.grad, "dx")
    close(wgug.grad, wgur.grad, "dW_gate_up")
    close(wdg.grad, wdr.grad, "dW_down")
    close(wg.grad, wr.grad, "d routing weights")


def test_moe_main_grad_accumulation_and_empty_experts():
    from easydel_b200.ops import moe_kernels as MK, reference as R

    T, H, Fd, E, k = 200, 128, 256, 8, 2
    x, wgu, wd, w, idx = _setup(T, H, Fd, E, k, seed=3)
    idx = idx % 3  # experts 3..7 receive nothing
    wgu = wgu.clone().requires_grad_(True)
    wd = wd.clone().requires_grad_(True)
    wgu.main_grad = torch.zeros(wgu.shape, dtype=torch.float32, device="cuda")
    wd.main_grad = torch.zeros(wd.shape, dtype=torch.float32, device="cuda")
    for _ in range(2):
        y = MK.moe_ffn(x, wgu, wd, w, idx)
        y.float().sum().backward()
    xr, wgur, wdr = x.float(), wgu.detach().float().requires_grad_(True), wd.detach().float().requires_grad_(True)
    R.moe_experts(xr, wgur, wdr, w, idx).sum().backward()
    assert wgu.grad is None and wd.grad is None
    rel = ((wd.main_grad - 2 * wdr.grad).norm() / (2 * wdr.grad).norm()).item()
    assert rel < 0.05, rel
    assert wgu.main_grad[3:].abs().max().item() == 0


def test_moe_ffn_with_expert_biases_and_gptoss_gate():
    """Composed path: grouped GEMMs on the tensor cores + per-expert biases + the clamped GPT-OSS gate, against the
    CPU composition of the same op in fp32."""
    from easydel_b200.ops import grouped

    T, H, Fd, E, k = 300, 256, 384, 8, 2
    x, wgu, wd, w, idx = _setup(T, H, Fd, E, k, seed=5)
    g = torch.Generator(device="cuda").manual_seed(9)
    bgu = (torch.randn(E, 2 * Fd, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bd = (torch.randn(E, H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    cpu = [t.detach().float().cpu().requires_grad_(True) for t in (x, wgu, wd, w, bgu, bd)]
    ref = grouped.moe_ffn(cpu[0], cpu[1], cpu[2], cpu[3], idx.cpu(), "gptoss_swiglu", b_gate_up=cpu[4], b_down=cpu[5])
    dy = torch.randn_like(ref)
    ref.backward(dy)
    dev = [t.detach().clone().requires_grad_(True) for t in (x, wgu, wd, w, bgu, bd)]
    y = grouped.moe_ffn(dev[0], dev[1], dev[2], dev[3], idx, "gptoss_swiglu", b_gate_up=dev[4], b_down=dev[5])
    assert torch.allclose(y.float().cpu(), ref.detach(), atol=4e-2, rtol=4e-2), (y.float().cpu() - ref).abs().max()
    y.backward(dy.cuda().to(y.dtype))
    for a, b, name in zip(dev, cpu, ("dx", "dW_gate_up", "dW_down", "dw", "db_gate_up", "db_down")):
        rel = ((a.grad.float().cpu() - b.grad).norm() / (b.grad.norm() + 1e-8)).item()
        assert rel < 0.05, f"{name}: {rel}"
