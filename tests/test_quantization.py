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
