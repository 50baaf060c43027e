"""Weight-only quantisation: formats, tensors, the quantised linear and the model-wide quantiser.

Formats follow the reference's registry (easydel/layers/quantization/_configs.py:221-278 and
layers/linears/_linear_quantized.py): ``int8`` (symmetric), ``affine`` 4 / 8 bit (scale + zero), ``nf4``
(normal-float code book, absmax per block), ``mxfp4`` / ``mxfp8`` (e2m1 / e4m3 values with a power-of-two scale per
32), ``nvfp4`` (e2m1 with an e4m3 scale per 16) and ``nvfp8`` (e4m3 with one scale per row). All of them are stored
as ``codes`` + per-group ``scales`` (+ ``zeros``) + a code book, which is what ``csrc/quant.cu`` consumes:
decode steps (up to 8 rows) run the fused dequant-GEMV, larger batches dequantise into bf16 and use the tcgen05 GEMM.
"""

from __future__ import annotations

import enum

import ctypes as C
import re
import typing as tp
from dataclasses import dataclass

import torch
from torch import nn

from ..ops import _lib

_lib.register("edl_dequant_bf16", _lib.i32, [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                             _lib.vp, _lib.i64, _lib.vp])
_lib.register("edl_qgemv", _lib.i32, [_lib.vp, _lib.i64, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                      _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.i64, _lib.vp, _lib.vp, _lib.vp])

_NF4 = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
        -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
        0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0]
_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def _e4m3_table() -> torch.Tensor:
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    return torch.nan_to_num(t, nan=0.0)


FORMATS: dict[str, dict] = {
    "int8": dict(bits=8, group=128, kind="sym"),
    "a8bit": dict(bits=8, group=128, kind="affine"),
    "a4bit": dict(bits=4, group=64, kind="affine"),
    "affine": dict(bits=4, group=64, kind="affine"),
    "nf4": dict(bits=4, group=64, kind="lut", lut=_NF4),
    "mxfp4": dict(bits=4, group=32, kind="lut", lut=_E2M1, scale="e8m0"),
    "nvfp4": dict(bits=4, group=16, kind="lut", lut=_E2M1, scale="e4m3"),
    "mxfp8": dict(bits=8, group=32, kind="lut", lut="e4m3", scale="e8m0"),
    "nvfp8": dict(bits=8, group=-1, kind="lut", lut="e4m3"),
}


@dataclass
class EasyDeLQuantizationConfig:
    dtype: str = "nf4"
    block_size: int | None = None
    pattern: str | None = None            # regex on module names; default: every linear except heads / routers
    quantize_tensors: bool = True
    bits: int | None = None

    def spec(self) -> dict:
        if self.dtype not in FORMATS:
            raise ValueError(f"unknown quantisation dtype {self.dtype!r}; known: {sorted(FORMATS)}")
        s = dict(FORMATS[self.dtype])
        if self.bits in (4, 8) and s["kind"] == "affine":
            s["bits"] = self.bits
        if self.block_size and s["group"] > 0 and "scale" not in s:
            s["group"] = self.block_size
        return s


QuantizationConfig = EasyDeLQuantizationConfig


class QuantizationType(str, enum.Enum):
    """The weight formats of :data:`FORMATS` under the reference's enum name."""

    INT8 = "int8"
    A8BIT = "a8bit"
    A4BIT = "a4bit"
    AFFINE = "affine"
    NF4 = "nf4"
    MXFP4 = "mxfp4"
    NVFP4 = "nvfp4"
    MXFP8 = "mxfp8"
    NVFP8 = "nvfp8"


def _lut_tensor(spec: dict, device) -> torch.Tensor:
    lut = spec.get("lut")
    if spec["kind"] == "sym":
        t = torch.arange(256, dtype=torch.float32)
        t = torch.where(t >= 128, t - 256, t)
    elif spec["kind"] == "affine":
        t = torch.arange(1 << spec["bits"], dtype=torch.float32)
    elif isinstance(lut, str):
        t = _e4m3_table()
    else:
        t = torch.tensor(lut, dtype=torch.float32)
    return t.to(device)


def _round_scale(s: torch.Tensor, how: str | None) -> torch.Tensor:
    if how == "e8m0":      # power of two, rounded up so that the block maximum stays representable
        return torch.exp2(torch.ceil(torch.log2(s.clamp_min(2.0 ** -126))))
    if how == "e4m3":
        return s.clamp(max=448.0).to(torch.float8_e4m3fn).float().clamp_min(2.0 ** -9)
    return s


class QuantizedTensor:
    """``w[n, k] = lut[codes[n, k]] * scales[n, k // group] (+ zeros)``; 4-bit codes are packed two per byte."""

    def __init__(self, codes, scales, zeros, lut, bits: int, group: int, shape, fmt: str):
        self.codes, self.scales, self.zeros, self.lut = codes, scales, zeros, lut
        self.bits, self.group, self.shape, self.fmt = bits, group, tuple(shape), fmt

    @property
    def device(self):
        return self.codes.device

    def nbytes(self) -> int:
        n = self.codes.numel() + self.scales.numel() * 2
        return n + (self.zeros.numel() * 2 if self.zeros is not None else 0)

    def to(self, device) -> "QuantizedTensor":
        z = self.zeros.to(device) if self.zeros is not None else None
        return QuantizedTensor(self.codes.to(device), self.scales.to(device), z, self.lut.to(device), self.bits,
                               self.group, self.shape, self.fmt)

    def dequantize(self, dtype=torch.bfloat16) -> torch.Tensor:
        N, K = self.shape
        if self.codes.is_cuda and _lib.available() and dtype == torch.bfloat16:
            out = torch.empty(N, K, dtype=torch.bfloat16, device=self.device)
            _lib.call("edl_dequant_bf16", self.codes.data_ptr(), self.scales.data_ptr(), _lib.ptr(self.zeros),
                      self.lut.data_ptr(), self.bits, N, K, self.group, out.data_ptr(), K, _lib.stream_ptr())
            return out
        return dequantize_reference(self).to(dtype)


def dequantize_reference(q: QuantizedTensor) -> torch.Tensor:
    N, K = q.shape
    codes = q.codes.long()
    if q.bits == 4:
        codes = torch.stack([codes & 0xF, codes >> 4], -1).reshape(N, K)
    vals = q.lut.float()[codes]
    sc = q.scales.float().repeat_interleave(q.group, 1)
    w = vals * sc
    if q.zeros is not None:
        w = w + q.zeros.float().repeat_interleave(q.group, 1)
    return w


def quantize(w: torch.Tensor, config: EasyDeLQuantizationConfig | str = "nf4") -> QuantizedTensor:
    """Quantises a ``[N, K]`` weight along K (host-side math in PyTorch; this is a load-time operation)."""
    cfg = EasyDeLQuantizationConfig(config) if isinstance(config, str) else config
    spec = cfg.spec()
    N, K = w.shape
    bits = spec["bits"]
    group = K if spec["group"] <= 0 else spec["group"]
    per16 = 32 if bits == 4 else 16
    if K % group or K % per16:
        raise ValueError(f"in_features {K} must be a multiple of the group size {group} and of {per16}")
    wf = w.detach().float().reshape(N, K // group, group)
    lut = _lut_tensor(spec, w.device)
    zeros = None
    if spec["kind"] == "sym":
        scale = (wf.abs().amax(-1) / 127.0).clamp_min(1e-8)
        scale = scale.to(torch.bfloat16).float()
        q = torch.round(wf / scale[..., None]).clamp(-127, 127)
        codes = torch.where(q < 0, q + 256, q).to(torch.uint8)
    elif spec["kind"] == "affine":
        lo, hi = wf.amin(-1), wf.amax(-1)
        levels = (1 << bits) - 1
        scale = ((hi - lo) / levels).clamp_min(1e-8).to(torch.bfloat16).float()
        zeros = lo.to(torch.bfloat16)
        codes = torch.round((wf - zeros.float()[..., None]) / scale[..., None]).clamp(0, levels).to(torch.uint8)
    else:
        top = lut.abs().max()
        scale = _round_scale((wf.abs().amax(-1) / top).clamp_min(1e-12), spec.get("scale"))
        scale = scale.to(torch.bfloat16).float()
        target = wf / scale[..., None]
        if lut.numel() == 16:
            codes = (target[..., None] - lut.view(1, 1, 1, -1)).abs().argmin(-1).to(torch.uint8)
        else:  # e4m3: round through the hardware cast, then read the byte pattern
            codes = target.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    codes = codes.reshape(N, K)
    if bits == 4:
        codes = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return QuantizedTensor(codes.contiguous(), scale.to(torch.bfloat16).contiguous(),
                           zeros.contiguous() if zeros is not None else None, lut, bits, group, (N, K), cfg.dtype)


def quantized_matmul(x: torch.Tensor, q: QuantizedTensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ W^T`` for a quantised ``W``; picks the fused GEMV for decode-sized inputs."""
    N, K = q.shape
    x2 = x.reshape(-1, K)
    M = x2.shape[0]
    per16 = 32 if q.bits == 4 else 16
    if x2.is_cuda and _lib.available() and x2.dtype == torch.bfloat16:
        if M <= 8 and q.group % per16 == 0:
            x32 = x2.float().contiguous()     # the kernel reads fp32 activations (a few rows: converted once)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
            _lib.call("edl_qgemv", x32.data_ptr(), K, q.codes.data_ptr(),
                      q.scales.data_ptr(), _lib.ptr(q.zeros), q.lut.data_ptr(), q.bits, M, N, K, q.group,
                      out.data_ptr(), N, _lib.ptr(bias), _lib.status_word(x.device).data_ptr(), _lib.stream_ptr())
            return out.view(*x.shape[:-1], N)
        from ..ops import functional as F

        return F.linear(x, q.dequantize(torch.bfloat16), bias)
    y = x2.float() @ dequantize_reference(q).t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype).view(*x.shape[:-1], N)


class QuantizedLinear(nn.Module):
    """Drop-in for the parallel linears after quantisation (inference only; weights are buffers)."""

    def __init__(self, q: QuantizedTensor, bias: torch.Tensor | None = None, source: nn.Module | None = None):
        super().__init__()
        self.fmt, self.bits, self.group = q.fmt, q.bits, q.group
        self.out_features, self.in_features = q.shape
        self.register_buffer("codes", q.codes)
        self.register_buffer("scales", q.scales)
        self.register_buffer("zeros", q.zeros)
        self.register_buffer("lut", q.lut)
        self.register_buffer("bias", bias.detach().clone() if bias is not None else None)
        for attr in ("out_splits", "parallel_style", "tp_size", "tp_rank", "tp_group"):
            if source is not None and hasattr(source, attr):
                setattr(self, attr, getattr(source, attr))
        self._source_forward = None
        if source is not None and getattr(source, "tp_size", 1) > 1:
            self._source_forward = type(source).__name__

    def local_out_splits(self):
        return getattr(self, "out_splits", (self.out_features,))

    def tensor(self) -> QuantizedTensor:
        return QuantizedTensor(self.codes, self.scales, self.zeros, self.lut, self.bits, self.group,
                               (self.out_features, self.in_features), self.fmt)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp_group = getattr(self, "tp_group", None)
        if tp_group is not None and getattr(self, "parallel_style", None) == "row":
            from ..parallel import tp

            y = quantized_matmul(x, self.tensor(), None)
            y = tp.all_reduce(y, tp_group)
            return y if self.bias is None else y + self.bias
        return quantized_matmul(x, self.tensor(), self.bias)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, fmt={self.fmt}, bits={self.bits}, group={self.group}"


_DEFAULT_SKIP = re.compile(r"(lm_head|embed|score|router|\.gate$|value_head|norm)")


class EasyQuantizer:
    def __init__(self, quantization_config: EasyDeLQuantizationConfig | str | None = None, **kw):
        if isinstance(quantization_config, str):
            quantization_config = EasyDeLQuantizationConfig(quantization_config, **kw)
        self.config = quantization_config or EasyDeLQuantizationConfig(**kw)

    def _wanted(self, name: str, mod: nn.Module) -> bool:
        w = getattr(mod, "weight", None)
        if not isinstance(w, torch.Tensor) or w.dim() != 2 or isinstance(mod, (nn.Embedding, QuantizedLinear)):
            return False
        if not hasattr(mod, "forward") or type(mod).__name__ in ("Embed",):
            return False
        if self.config.pattern:
            return re.search(self.config.pattern, name) is not None
        return _DEFAULT_SKIP.search(name) is None

    def quantize_linear(self, mod: nn.Module) -> QuantizedLinear:
        return QuantizedLinear(quantize(mod.weight, self.config), getattr(mod, "bias", None), mod)

    def apply_quantization(self, model: nn.Module, verbose: bool = False) -> nn.Module:
        spec = self.config.spec()
        per16 = 32 if spec["bits"] == 4 else 16
        n_done, saved = 0, 0
        for name, mod in list(model.named_modules()):
            if not self._wanted(name, mod):
                continue
            K = mod.weight.shape[1]
            group = K if spec["group"] <= 0 else spec["group"]
            if K % group or K % per16:
                continue
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            q = self.quantize_linear(mod)
            saved += mod.weight.numel() * mod.weight.element_size() - q.tensor().nbytes()
            setattr(parent, leaf, q)
            n_done += 1
        if verbose:
            print(f"[quantize] {n_done} linears -> {self.config.dtype}, {saved / 2**20:.1f} MiB saved")
        model.quantization_summary = {"modules": n_done, "bytes_saved": saved, "format": self.config.dtype}
        return model


# ------------------------------------------------------------------------------------------------- KV cache
def quantize_kv_int8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-(token, head) symmetric int8 for cached keys / values: returns (codes int8, scales bf16)."""
    scale = (x.float().abs().amax(-1, keepdim=True) / 127.0).clamp_min(1e-8)
    return torch.round(x.float() / scale).clamp(-127, 127).to(torch.int8), scale.to(torch.bfloat16)


def dequantize_kv_int8(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return (codes.float() * scales.float()).to(dtype)


# ------------------------------------------------------------------------------------------------- QAT
class _StraightThrough(torch.autograd.Function):
    """Forward: the weight as it comes back from quantise -> dequantise; backward: identity."""

    @staticmethod
    def forward(ctx, w, cfg):
        w2 = w.reshape(-1, w.shape[-1])
        return dequantize_reference(quantize(w2.detach(), cfg)).to(w.dtype).view(w.shape)

    @staticmethod
    def backward(ctx, g):
        return g, None


def straight_through(w: torch.Tensor, dtype: str | QuantizationType | EasyDeLQuantizationConfig = "nf4",
                     block_size: int | None = None) -> torch.Tensor:
    """Fake-quantised weight for quantisation-aware training: the value the quantised format would hold, with the
    gradient passed through unchanged (the reference's ``straight_through``,
    easydel/layers/quantization/_straight_through.py)."""
    if isinstance(dtype, EasyDeLQuantizationConfig):
        cfg = dtype
    else:
        cfg = EasyDeLQuantizationConfig(getattr(dtype, "value", dtype), block_size=block_size)
    return _StraightThrough.apply(w, cfg)


def straight_through_nf4(w, block_size: int | None = None):
    return straight_through(w, "nf4", block_size)


def straight_through_8bit(w, block_size: int | None = None):
    return straight_through(w, "int8", block_size)


def straight_through_mxfp4(w):
    return straight_through(w, "mxfp4")


def straight_through_mxfp8(w):
    return straight_through(w, "mxfp8")


def straight_through_nvfp8(w):
    return straight_through(w, "nvfp8")


def straight_through_1bit(w: torch.Tensor) -> torch.Tensor:
    """sign(w) scaled by the mean magnitude of each row, gradient passed through."""
    q = torch.sign(w) * w.abs().mean(-1, keepdim=True)
    return w + (q - w).detach()


class QATLinear(nn.Module):
    """Wraps a linear layer for quantisation-aware training: the forward product uses the fake-quantised weight, the
    optimizer keeps updating the full-precision one. ``EasyQuantizer.apply_qat`` installs it; ``convert`` turns the
    trained layer into a :class:`QuantizedLinear`."""

    def __init__(self, inner: nn.Module, config: EasyDeLQuantizationConfig):
        super().__init__()
        self.inner, self.config = inner, config

    @property
    def weight(self):
        return self.inner.weight

    @property
    def bias(self):
        return getattr(self.inner, "bias", None)

    def forward(self, x, *args, **kw):
        from ..ops import functional as F

        w = straight_through(self.inner.weight, self.config)
        y = F.linear(x, w, getattr(self.inner, "bias", None))
        return y

    def convert(self) -> QuantizedLinear:
        return QuantizedLinear(quantize(self.inner.weight.detach(), self.config), getattr(self.inner, "bias", None),
                               self.inner)


def _apply_qat(self, model: nn.Module) -> nn.Module:
    """Replaces every linear the quantiser would quantise by a :class:`QATLinear` around it (plain, non-parallel
    linears: a tensor-parallel layer keeps its own forward)."""
    n = 0
    for name, mod in list(model.named_modules()):
        if not self._wanted(name, mod) or isinstance(mod, QATLinear) or getattr(mod, "tp_size", 1) > 1:
            continue
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        if isinstance(parent, QATLinear):
            continue
        setattr(parent, leaf, QATLinear(mod, self.config))
        n += 1
    model.qat_summary = {"modules": n, "format": self.config.dtype}
    return model


def _finalize_qat(self, model: nn.Module) -> nn.Module:
    """Turns the :class:`QATLinear` wrappers of a trained model into quantised linears."""
    for name, mod in list(model.named_modules()):
        if isinstance(mod, QATLinear):
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, mod.convert())
    return model


EasyQuantizer.apply_qat = _apply_qat
EasyQuantizer.finalize_qat = _finalize_qat
