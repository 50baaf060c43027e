"""Weight-only quantisation: every format round-trips within its expected error, the CUDA dequant / GEMV kernels
agree with the PyTorch reference, and a quantised model still generates the same greedy tokens as its dequantised
twin."""

import pytest
import torch

from easydel_b200.layers.quantization import (FORMATS, EasyDeLQuantizationConfig, EasyQuantizer, QuantizedLinear,
                                              dequantize_reference, quantize, quantized_matmul)

TOL = {"int8": 0.02, "a8bit": 0.02, "a4bit": 0.2, "affine": 0.2, "nf4": 0.2, "mxfp4": 0.3, "nvfp4": 0.25,
       "mxfp8": 0.08, "nvfp8": 0.08}


@pytest.mark.parametrize("fmt", sorted(FORMATS))
def test_roundtrip_error(fmt):
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.05
    q = quantize(w, fmt)
    back = dequantize_reference(q)
    rel = (back - w).norm() / w.norm()
    assert rel < TOL[fmt], (fmt, float(rel))
    assert q.nbytes() < w.numel() * 2
    x = torch.randn(3, 256)
    y = quantized_matmul(x, q)
    assert torch.allclose(y, x @ back.t(), atol=1e-4)


def test_quantizer_replaces_linears_and_keeps_outputs_close():
    from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        ref = model(input_ids=ids).logits
    model.quantize(EasyDeLQuantizationConfig("int8", block_size=64))
    n = sum(isinstance(m, QuantizedLinear) for m in model.modules())
    assert n == 2 * 4 and not isinstance(model.lm_head, QuantizedLinear)
    with torch.no_grad():
        got = model(input_ids=ids).logits
    assert (got - ref).abs().max() < 0.05 * ref.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["int8", "a4bit", "nf4", "mxfp4", "nvfp4", "mxfp8", "nvfp8"])
@pytest.mark.parametrize("M", [1, 5, 8, 64])
def test_cuda_kernels_match_reference(fmt, M):
    torch.manual_seed(1)
    N, K = 1000 if fmt != "nvfp8" else 512, 1024
    w = (torch.randn(N, K) * 0.05).cuda()
    q = quantize(w, fmt)
    ref_w = dequantize_reference(q)
    got_w = q.dequantize(torch.bfloat16)
    assert torch.allclose(got_w.float(), ref_w.to(torch.bfloat16).float(), atol=1e-6)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    y = quantized_matmul(x, q, bias)
    ref = x.float() @ ref_w.t() + bias.float()
    assert (y.float() - ref).abs().max() < 2e-2 * ref.abs().max().clamp_min(1.0)


def test_straight_through_and_qat_linear():
    """Fake quantisation for training: forward value = quantise -> dequantise, gradient = identity; a wrapped model
    trains its full-precision weights and converts to quantised linears whose output it already produced."""
    import torch
    from torch import nn

    from easydel_b200.layers import quantization as Q

    torch.manual_seed(0)
    w = torch.randn(8, 256, requires_grad=True)
    wq = Q.straight_through(w, "nf4")
    ref = Q.dequantize_reference(Q.quantize(w.detach(), "nf4"))
    assert torch.allclose(wq, ref) and not torch.equal(wq, w)
    (wq * torch.arange(256.0)).sum().backward()
    assert torch.allclose(w.grad, torch.arange(256.0).expand(8, 256))
    for fn in (Q.straight_through_8bit, Q.straight_through_mxfp4, Q.straight_through_mxfp8, Q.straight_through_nvfp8):
        assert fn(w).shape == w.shape
    b = Q.straight_through_1bit(w)
    assert torch.allclose(b.abs(), w.detach().abs().mean(-1, keepdim=True).expand_as(w))

    model = nn.Sequential(nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 8))
    quantizer = Q.EasyQuantizer("nf4", pattern=r".*")
    quantizer.apply_qat(model)
    assert model.qat_summary["modules"] == 2 and isinstance(model[0], Q.QATLinear)
    x = torch.randn(16, 256)
    before = model[0].inner.weight.detach().clone()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    loss = model(x).pow(2).mean()
    loss.backward()
    opt.step()
    assert not torch.equal(model[0].inner.weight, before)          # the full-precision weight moved
    y_qat = model(x)
    quantizer.finalize_qat(model)
    assert isinstance(model[0], Q.QuantizedLinear)
    assert torch.allclose(model(x), y_qat, atol=1e-4)
