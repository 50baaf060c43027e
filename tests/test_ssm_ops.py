"""Recurrent ops: the CUDA scans agree with the step-by-step PyTorch recurrences, including carried state."""

import pytest
import torch

from easydel_b200.ops import ssm


def _close(a, b, tol=3e-2):
    return (a.float() - b.float()).abs().max() <= tol * b.float().abs().max().clamp_min(1.0)


def test_references_carry_state_across_calls():
    torch.manual_seed(0)
    T, D, N = 12, 6, 4
    u, delta = torch.randn(T, D), torch.randn(T, D)
    A = -torch.rand(D, N)
    B, C = torch.randn(T, N), torch.randn(T, N)
    full = ssm.selective_scan_reference(u, delta, A, B, C)
    st = torch.zeros(1, D, N)
    a = ssm.selective_scan_reference(u[:7], delta[:7], A, B[:7], C[:7], state=st)
    b = ssm.selective_scan_reference(u[7:], delta[7:], A, B[7:], C[7:], state=st)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-5)
    q, k, v = torch.randn(T, 2, 8), torch.randn(T, 2, 8), torch.randn(T, 2, 5)
    g, beta = -torch.rand(T, 2), torch.rand(T, 2)
    full = ssm.delta_rule_reference(q, k, v, g, beta)
    st = torch.zeros(1, 2, 8, 5)
    parts = torch.cat([ssm.delta_rule_reference(q[:5], k[:5], v[:5], g[:5], beta[:5], state=st),
                       ssm.delta_rule_reference(q[5:], k[5:], v[5:], g[5:], beta[5:], state=st)])
    assert torch.allclose(parts, full, atol=1e-5)


@pytest.mark.gpu
def test_selective_scan_cuda():
    torch.manual_seed(1)
    dev, T, D, N = "cuda", 70, 192, 16
    cu = torch.tensor([0, 30, 70], dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)  # noqa: E731
    u, delta, z, B, C = bf(T, D), bf(T, D), bf(T, D), bf(T, N), bf(T, N)
    A, Dv, bias = -torch.rand(D, N, device=dev), torch.randn(D, device=dev), torch.randn(D, device=dev)
    s1, s2 = torch.zeros(2, D, N, device=dev), torch.zeros(2, D, N, device=dev)
    with torch.no_grad():
        got = ssm.selective_scan(u, delta, A, B, C, Dv, z, bias, True, cu, s1)
        ref = ssm.selective_scan_reference(u, delta, A, B, C, Dv, z, bias, True, cu, s2)
    assert _close(got, ref) and _close(s1, s2)


@pytest.mark.gpu
def test_ssd_scan_cuda():
    torch.manual_seed(2)
    dev, T, H, P, G, N = "cuda", 40, 4, 64, 2, 128
    cu = torch.tensor([0, 17, 40], dtype=torch.int32, device=dev)
    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)  # noqa: E731
    x, dt, B, C = bf(T, H, P), bf(T, H), bf(T, G, N) * 0.3, bf(T, G, N) * 0.3
    A, Dv = -torch.rand(H, device=dev), torch.randn(H, device=dev)
    s1, s2 = torch.zeros(2, H, P, N, device=dev), torch.zeros(2, H, P, N, device=dev)
    with torch.no_grad():
        got = ssm.ssd_scan(x, dt, A, B, C, Dv, None, True, cu, s1)
        ref = ssm.ssd_scan_reference(x, dt, A, B, C, Dv, None, True, cu, s2)
    assert _close(got, ref) and _close(s1, s2)


@pytest.mark.gpu
@pytest.mark.parametrize("DK,DV,kda", [(128, 128, False), (64, 96, False), (128, 128, True), (128, 256, False)])
def test_delta_rule_cuda(DK, DV, kda):
    torch.manual_seed(3)
    dev, T, H = "cuda", 33, 3
    cu = torch.tensor([0, 13, 33], dtype=torch.int32, device=dev)
    q = torch.nn.functional.normalize(torch.randn(T, H, DK, device=dev), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(T, H, DK, device=dev), dim=-1).to(torch.bfloat16)
    v = torch.randn(T, H, DV, device=dev).to(torch.bfloat16)
    g = -torch.rand(T, H, DK, device=dev) if kda else -torch.rand(T, H, device=dev)
    beta = torch.rand(T, H, device=dev).to(torch.bfloat16)
    s1, s2 = torch.zeros(2, H, DK, DV, device=dev), torch.zeros(2, H, DK, DV, device=dev)
    with torch.no_grad():
        got = ssm.gated_delta_rule(q, k, v, g, beta, None, cu, s1)
        ref = ssm.delta_rule_reference(q, k, v, g, beta, None, cu, s2)
    assert _close(got, ref) and _close(s1, s2)


@pytest.mark.gpu
def test_ragged_conv1d_cuda():
    torch.manual_seed(4)
    dev, T, Cn, W = "cuda", 50, 96, 4
    cu = torch.tensor([0, 3, 20, 50], dtype=torch.int32, device=dev)
    x = torch.randn(T, Cn, device=dev).to(torch.bfloat16)
    w = torch.randn(Cn, W, device=dev).to(torch.bfloat16)
    b = torch.randn(Cn, device=dev).to(torch.bfloat16)
    c1 = torch.randn(3, W - 1, Cn, device=dev).to(torch.bfloat16)
    c2 = c1.clone()
    with torch.no_grad():
        got = ssm.ragged_conv1d(x, w, b, cu, "silu", c1)
        ref = ssm.ragged_conv1d_reference(x, w, b, cu, "silu", c2)
    assert _close(got, ref) and torch.equal(c1, c2)


@pytest.mark.gpu
def test_wkv4_kernel_matches_reference_with_state():
    from easydel_b200.ops import ssm

    torch.manual_seed(0)
    C = 200
    cu = torch.tensor([0, 37, 100], dtype=torch.int32, device="cuda")
    k = torch.randn(100, C, device="cuda").to(torch.bfloat16)
    v = torch.randn(100, C, device="cuda").to(torch.bfloat16)
    decay, first = torch.randn(C, device="cuda") * 0.5 - 1.0, torch.randn(C, device="cuda") * 0.5
    st = torch.zeros(2, 3, C, device="cuda")
    st[:, 2] = -1e38
    st_ref = st.clone()
    out = ssm.wkv4(decay, first, k, v, cu, st)
    ref = ssm.wkv4_reference(decay, first, k.float(), v.float(), cu, st_ref)
    assert (out.float() - ref).abs().max() < 2e-2
    assert (st[:, :2] - st_ref[:, :2]).abs().max() < 1e-3 * max(1.0, float(st_ref[:, :2].abs().max()))
    # a second call continues from the state
    out2 = ssm.wkv4(decay, first, k, v, cu, st)
    ref2 = ssm.wkv4_reference(decay, first, k.float(), v.float(), cu, st_ref)
    assert (out2.float() - ref2).abs().max() < 2e-2


def test_chunked_selective_scan_and_ssd_match_the_sequential_references_with_gradients():
    """The forms training runs (parallel scan per chunk / chunked matrix form) against the one-token-at-a-time
    references: outputs, final states and every input gradient, on two packed sequences with initial states."""
    import torch

    from easydel_b200.ops import ssm

    torch.manual_seed(0)

    def mk(*s):
        return (torch.randn(*s) * 0.5).requires_grad_(True)

    cu = torch.tensor([0, 70, 150], dtype=torch.int32)
    T, Dm, N = 150, 12, 8
    u, delta, B, C, z = mk(T, Dm), mk(T, Dm), mk(T, N), mk(T, N), mk(T, Dm)
    A = (-torch.rand(Dm, N) - 0.1).requires_grad_(True)
    D, dtb = mk(Dm), mk(Dm)
    ins = [u, delta, A, B, C, D, z, dtb]
    s1 = torch.randn(2, Dm, N)
    s2 = s1.clone()
    y1 = ssm.selective_scan_reference(u, delta, A, B, C, D, z, dtb, True, cu, s1)
    y2 = ssm.selective_scan_chunked(u, delta, A, B, C, D, z, dtb, True, cu, s2, chunk=32)
    g1 = torch.autograd.grad(y1.square().sum(), ins)
    g2 = torch.autograd.grad(y2.square().sum(), ins)
    assert torch.allclose(y1, y2, atol=1e-5) and torch.allclose(s1, s2, atol=1e-5)
    assert all(torch.allclose(a, b, atol=2e-4, rtol=1e-4) for a, b in zip(g1, g2))

    T, H, P, G, N = 150, 4, 6, 2, 8
    x, dt, B, C = mk(T, H, P), mk(T, H), mk(T, G, N), mk(T, G, N)
    A = (-torch.rand(H) - 0.1).requires_grad_(True)
    D, dtb = mk(H), mk(H)
    ins = [x, dt, A, B, C, D, dtb]
    s1 = torch.randn(2, H, P, N)
    s2 = s1.clone()
    y1 = ssm.ssd_scan_reference(x, dt, A, B, C, D, dtb, True, cu, s1)
    y2 = ssm.ssd_scan_chunked(x, dt, A, B, C, D, dtb, True, cu, s2, chunk=32)
    g1 = torch.autograd.grad(y1.square().sum(), ins)
    g2 = torch.autograd.grad(y2.square().sum(), ins)
    assert torch.allclose(y1, y2, atol=2e-5) and torch.allclose(s1, s2, atol=2e-5)
    assert all(torch.allclose(a, b, atol=5e-4, rtol=1e-3) for a, b in zip(g1, g2))


@pytest.mark.gpu
def test_chunked_scans_on_the_gpu_match_the_recurrent_kernels():
    """Training's chunked forms (autograd on, CUDA tensors) against the inference kernels on the same inputs."""
    import torch

    from easydel_b200.ops import ssm

    torch.manual_seed(0)
    dev = "cuda"
    T, Dm, N = 700, 256, 16
    bf = lambda *s: (torch.randn(*s, device=dev) * 0.5).to(torch.bfloat16)   # noqa: E731
    u, delta, B, C, z = bf(T, Dm), bf(T, Dm), bf(T, N), bf(T, N), bf(T, Dm)
    A = -torch.rand(Dm, N, device=dev) - 0.1
    D, dtb = torch.randn(Dm, device=dev), torch.randn(Dm, device=dev) * 0.1
    cu = torch.tensor([0, 300, 700], dtype=torch.int32, device=dev)
    with torch.no_grad():
        want = ssm.selective_scan(u, delta, A, B, C, D, z, dtb, True, cu)
    ug = u.clone().requires_grad_(True)
    got = ssm.selective_scan(ug, delta, A, B, C, D, z, dtb, True, cu)          # gradients wanted: chunked form
    got.float().square().sum().backward()
    assert ug.grad is not None and torch.isfinite(ug.grad).all()
    assert (got.float() - want.float()).abs().max() < 0.06 * want.float().abs().max() + 0.02

    H, P, G, N = 8, 64, 2, 32
    x, dt, Bm, Cm = bf(T, H, P), bf(T, H), bf(T, G, N), bf(T, G, N)
    A2 = -torch.rand(H, device=dev) - 0.1
    D2, dtb2 = torch.randn(H, device=dev), torch.randn(H, device=dev) * 0.1
    with torch.no_grad():
        want = ssm.ssd_scan(x, dt, A2, Bm, Cm, D2, dtb2, True, cu)
    xg = x.clone().requires_grad_(True)
    got = ssm.ssd_scan(xg, dt, A2, Bm, Cm, D2, dtb2, True, cu)
    got.float().square().sum().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad).all()
    assert (got.float() - want.float()).abs().max() < 0.06 * want.float().abs().max() + 0.02

    Cn = 256
    k, v = bf(T, Cn), bf(T, Cn)
    decay, first = torch.randn(Cn, device=dev) * 0.5 - 1.0, torch.randn(Cn, device=dev) * 0.5
    with torch.no_grad():
        want = ssm.wkv4(decay, first, k, v, cu)                                  # the recurrent kernel
    kg = k.clone().requires_grad_(True)
    got = ssm.wkv4(decay, first, kg, v, cu)                                      # gradients wanted: chunked form
    got.float().square().sum().backward()
    assert kg.grad is not None and torch.isfinite(kg.grad).all()
    assert (got.float() - want.float()).abs().max() < 0.03


def test_chunked_wkv4_matches_the_sequential_reference_with_gradients():
    """RWKV-4's chunked matrix form against the per-token recurrence: outputs, the carried (num, den, max) triple
    and the gradients of decay, bonus, keys and values, on two packed sequences that start from a state."""
    import torch

    from easydel_b200.ops import ssm

    torch.manual_seed(0)
    T, C = 150, 24
    cu = torch.tensor([0, 70, 150], dtype=torch.int32)
    k = (torch.randn(T, C) * 2.0).requires_grad_(True)              # wide keys exercise the running maximum
    v = torch.randn(T, C).requires_grad_(True)
    decay = (torch.randn(C) * 0.5 - 1.0).requires_grad_(True)
    first = (torch.randn(C) * 0.5).requires_grad_(True)
    ins = [decay, first, k, v]
    s1 = torch.zeros(2, 3, C)
    s1[:, 2] = -1e38
    with torch.no_grad():                                           # a state that has already seen tokens
        ssm.wkv4_reference(decay, first, torch.randn(40, C), torch.randn(40, C), torch.tensor([0, 15, 40]), s1)
    s2 = s1.clone()
    y1 = ssm.wkv4_reference(decay, first, k, v, cu, s1)
    y2 = ssm.wkv4_chunked(decay, first, k, v, cu, s2, chunk=32)
    g1 = torch.autograd.grad(y1.square().sum(), ins)
    g2 = torch.autograd.grad(y2.square().sum(), ins)
    assert torch.allclose(y1, y2, atol=1e-5)
    assert torch.allclose(s1[:, 2], s2[:, 2], atol=1e-5)                                   # same maximum
    assert torch.allclose(s1[:, :2], s2[:, :2], atol=1e-5, rtol=1e-5)
    assert all(torch.allclose(a, b, atol=2e-4, rtol=1e-4) for a, b in zip(g1, g2))
    # the dispatcher agrees with the reference, and a fresh state and a ragged last chunk work too
    with torch.no_grad():
        assert torch.allclose(ssm.wkv4(decay, first, k, v, cu), ssm.wkv4_reference(decay, first, k, v, cu), atol=1e-5)
        assert torch.allclose(ssm.wkv4_chunked(decay, first, k[:7], v[:7], chunk=4),
                              ssm.wkv4_reference(decay, first, k[:7], v[:7]), atol=1e-5)
