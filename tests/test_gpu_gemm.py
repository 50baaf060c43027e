"""tcgen05 GEMM against an fp32 PyTorch matmul for every operand layout, tile width and epilogue."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


def _mk(M, N, K, a_mn, b_mn, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).to(torch.bfloat16)
    return a, b


def _close(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    # bf16 output rounding (2^-8 relative) plus accumulation noise
    assert err <= 1e-2 * scale + 1e-3 * (K ** 0.5), f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(a_mn, b_mn, bn):
    from easydel_b200.ops import kernels as K_

    M, N, K = 384, 512, 320
    a, b = _mk(M, N, K, a_mn, b_mn)
    out = K_.gemm(a, b, a_mn=a_mn, b_mn=b_mn, force_bn=bn)
    _close(out, _ref(a, b, a_mn, b_mn), K)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(384, 512, 320), (256, 256, 64), (1000, 1000, 1000), (2048, 4096, 1024)])
def test_gemm_cta_pair(a_mn, b_mn, M, N, K):
    """The 256 x 256 cta_group::2 kernel (two CTAs per tile) on every operand layout, ragged edges included."""
    from easydel_b200.ops import kernels as K_

    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned leading dimension")
    a, b = _mk(M, N, K, a_mn, b_mn, seed=M + K)
    out = K_.gemm(a, b, a_mn=a_mn, b_mn=b_mn, force_bn=512)
    _close(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_cta_pair_fp32_accumulate_bias():
    from easydel_b200.ops import kernels as K_

    M, N, K = 512, 768, 512
    a, b = _mk(M, N, K, True, True, seed=5)
    ref = _ref(a, b, True, True)
    acc = torch.ones((M, N), device="cuda", dtype=torch.float32)
    K_.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, force_bn=512)
    K_.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, force_bn=512)
    assert torch.allclose(acc, 1 + 2 * ref, atol=2e-2, rtol=1e-3)
    a, b = _mk(M, N, K, False, False, seed=6)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = K_.gemm(a, b, bias=bias, force_bn=512)
    _close(out, _ref(a, b, False, False) + bias.float(), K)


def test_gemm_benchmarked_shape_against_oracle():
    """The largest benchmarked forward shape (gate_up of Llama-3-8B at 8192 tokens) against fp32 matmul."""
    from easydel_b200.ops import kernels as K_

    M, N, K = 8192, 28672, 4096
    a, b = _mk(M, N, K, False, False, seed=11)
    for bn in (0, 512):
        out = K_.gemm(a, b, force_bn=bn)
        for r0 in (0, 4096, 8192 - 256):  # compare row bands (the fp32 reference of the whole product is 940 MB)
            ref = a[r0:r0 + 256].float() @ b.float().t()
            _close(out[r0:r0 + 256], ref, K)
        del out


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 264, 72), (1, 8, 8), (1000, 1000, 1000), (4096, 4096, 4096),
                                   (130, 40, 4104)])
def test_gemm_shapes(M, N, K):
    from easydel_b200.ops import kernels as K_

    a, b = _mk(M, N, K, False, False, seed=M + N + K)
    out = K_.gemm(a, b)
    _close(out, _ref(a, b, False, False), K)


def test_gemm_fp32_accumulate_and_bias():
    from easydel_b200.ops import kernels as K_

    M, N, K = 304, 520, 256
    a, b = _mk(M, N, K, True, True, seed=3)
    ref = _ref(a, b, True, True)
    acc = torch.ones((M, N), device="cuda", dtype=torch.float32)
    K_.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True)
    K_.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True)
    assert torch.allclose(acc, 1 + 2 * ref, atol=2e-2, rtol=1e-3)
    a, b = _mk(M, N, K, False, False, seed=4)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = K_.gemm(a, b, bias=bias)
    _close(out, _ref(a, b, False, False) + bias.float(), K)


def test_gemm_strided_views():
    from easydel_b200.ops import kernels as K_

    big_a = torch.randn(256, 1024, device="cuda").to(torch.bfloat16)
    big_b = torch.randn(512, 1024, device="cuda").to(torch.bfloat16)
    a = big_a[:, 128:640]
    b = big_b[:, 128:640]
    out_big = torch.zeros(256, 1024, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, 256:768]
    K_.gemm(a, b, out=out)
    _close(out, a.float() @ b.float().t(), 512)
    assert out_big[:, :256].abs().max().item() == 0 and out_big[:, 768:].abs().max().item() == 0


def test_gemm_deterministic():
    from easydel_b200.ops import kernels as K_

    a, b = _mk(1024, 2048, 512, False, False, seed=9)
    o1 = K_.gemm(a, b)
    o2 = K_.gemm(a, b)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 6144, 4096), (64, 1280, 8192), (256, 4096, 14336),
                                   (48, 8192, 1024)])
def test_gemm_skinny_uses_split_k(M, N, K):
    """Decode-shaped products take the split-K path and agree with the fp32 reference (with and without bias)."""
    from easydel_b200.ops import kernels as K_

    assert K_._splitk_plan(M, N, K, torch.device("cuda", 0)) > 1
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    for b in (None, bias):
        out = K_.gemm(a, w, bias=b)
        ref = a.float() @ w.float().t() + (b.float() if b is not None else 0)
        err = (out.float() - ref).abs().max() / ref.abs().max()
        assert err < 1e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,splits", [(256, 1280, 8192, 4), (200, 7168, 4096, 2), (64, 520, 1024, 3),
                                          (256, 8192, 1024, 1), (384, 768, 2048, 5)])
def test_pair_splitk_matches_fp32(M, N, K, splits):
    """Split-K on the CTA-pair kernel (decode-sized products), with bias, against an fp32 product; with at most two
    slices repeated calls give bit-identical results; the accumulators and strip counters are left at zero."""
    from easydel_b200.ops import kernels as K_

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    ref = a.float() @ w.float().t() + bias.float()
    out = K_.gemm(a, w, bias=bias, pair_splits=splits)
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    again = K_.gemm(a, w, bias=bias, pair_splits=splits)
    if splits <= 2:
        assert torch.equal(out, again)
    else:
        assert (out.float() - again.float()).abs().max() <= 1e-2 * ref.abs().max()
    for ws, counters in K_._PAIR_WS.values():
        assert int(counters.abs().sum()) == 0 and float(ws.abs().max()) == 0.0


@pytest.mark.parametrize("M,N,K", [(256, 7168, 2048), (200, 520, 1024), (384, 1000, 512)])
def test_pair_kernel_128_wide_tiles(M, N, K):
    """The CTA-pair kernel with 256 x 128 tiles (skinny products), ragged M and N, with bias, against fp32."""
    from easydel_b200.ops import kernels as K_

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    ref = a.float() @ w.float().t() + bias.float()
    out = K_.gemm(a, w, bias=bias, force_bn=384)
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
