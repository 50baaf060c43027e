"""TurboQuant KV-cache compression (easydel/layers/quantization/_turboquant.py:48-140; the kernels it calls live in
ejkernel.quantization.turboquant).

Two stages per head vector of dimension ``d``:

1. *Rotate and scalar-quantise.* ``x = ||x|| * u``; a fixed random orthogonal matrix makes every coordinate of
   ``Pi u`` follow the same known law (density proportional to ``(1 - t^2)^((d-3)/2)`` on ``[-1, 1]``), so one
   Lloyd-Max codebook, solved once per ``(bits, d)``, is optimal for all coordinates. Values use all ``b`` bits.
2. *Sign sketch of the residual (keys only).* Keys spend ``b - 1`` bits on the codebook and one bit per sketch row on
   ``sign(S r)`` of the residual ``r = u - u_hat`` with a Gaussian ``S``; ``<q, r>`` is then estimated without bias by
   ``||r|| * sqrt(pi / 2) / m * <S q, sign(S r)>``, which removes the bias scalar quantisation puts on attention scores.

Everything here is plain tensor code (the compression runs once per appended token; scoring is two small GEMMs).
"""

from __future__ import annotations

import dataclasses
import functools
import math

import torch


@dataclasses.dataclass(frozen=True)
class TurboQuantConfig:
    bits: int = 4                  # total bits per coordinate: keys use bits-1 + the sign sketch, values use bits
    qjl_dim: int | None = None     # sketch rows for keys; default head_dim
    seed: int = 42

    def __post_init__(self):
        if self.bits < 2 or self.bits > 8:
            raise ValueError(f"bits must be in [2, 8], got {self.bits}")

    @property
    def key_codebook_bits(self) -> int:
        return self.bits - 1

    @property
    def value_codebook_bits(self) -> int:
        return self.bits

    @property
    def key_codebook_size(self) -> int:
        return 1 << self.key_codebook_bits

    @property
    def value_codebook_size(self) -> int:
        return 1 << self.value_codebook_bits


@functools.lru_cache(maxsize=32)
def solve_lloyd_max(bits: int, dim: int, grid: int = 20001, iters: int = 200) -> torch.Tensor:
    """Centroids of the MSE-optimal ``2^bits``-level quantiser of one coordinate of a uniform unit vector in R^dim."""
    t = torch.linspace(-1.0, 1.0, grid, dtype=torch.float64)
    w = (1.0 - t * t).clamp_min(0.0) ** ((dim - 3) / 2.0)
    w = w / w.sum()
    n = 1 << bits
    cdf = torch.cumsum(w, 0)
    c = torch.stack([t[torch.searchsorted(cdf, torch.tensor((i + 0.5) / n, dtype=torch.float64)).clamp(max=grid - 1)]
                     for i in range(n)])
    for _ in range(iters):
        edges = torch.cat([t[:1] - 1, (c[1:] + c[:-1]) / 2, t[-1:] + 1])
        idx = torch.bucketize(t, edges[1:-1])
        num = torch.zeros(n, dtype=torch.float64).index_add_(0, idx, w * t)
        den = torch.zeros(n, dtype=torch.float64).index_add_(0, idx, w)
        new = torch.where(den > 0, num / den.clamp_min(1e-300), c)
        if (new - c).abs().max() < 1e-10:
            c = new
            break
        c = new
    return ((c - c.flip(0)) / 2).float()      # the law is symmetric: remove the grid's rounding asymmetry


@dataclasses.dataclass(frozen=True)
class TurboQuantConstants:
    key_codebook: torch.Tensor       # [2^(bits-1)]
    value_codebook: torch.Tensor     # [2^bits]
    rotation_matrix: torch.Tensor    # [d, d] orthogonal
    qjl_projection: torch.Tensor     # [m, d] Gaussian
    qjl_dim: int
    bits: int

    @classmethod
    def create(cls, config: TurboQuantConfig, head_dim: int, layer_index: int = 0, device=None):
        g = torch.Generator().manual_seed(config.seed + layer_index)
        q, r = torch.linalg.qr(torch.randn(head_dim, head_dim, generator=g, dtype=torch.float64))
        q = q * torch.sign(torch.diagonal(r))[None, :]          # a Haar-distributed rotation
        m = config.qjl_dim or head_dim
        s = torch.randn(m, head_dim, generator=g, dtype=torch.float32)
        return cls(solve_lloyd_max(config.key_codebook_bits, head_dim).to(device),
                   solve_lloyd_max(config.value_codebook_bits, head_dim).to(device),
                   q.float().to(device), s.to(device), m, config.bits)

    def to(self, device):
        return dataclasses.replace(self, key_codebook=self.key_codebook.to(device),
                                   value_codebook=self.value_codebook.to(device),
                                   rotation_matrix=self.rotation_matrix.to(device),
                                   qjl_projection=self.qjl_projection.to(device))


def _nearest(x: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    edges = (codebook[1:] + codebook[:-1]) / 2
    return torch.bucketize(x, edges)


def quantize_values(v: torch.Tensor, k: TurboQuantConstants):
    """v ``[..., d]`` -> (codes uint8 ``[..., d]``, norms fp32 ``[...]``)."""
    vf = v.float()
    norm = vf.norm(dim=-1)
    u = (vf / norm.clamp_min(1e-20)[..., None]) @ k.rotation_matrix.t()
    return _nearest(u, k.value_codebook).to(torch.uint8), norm


def dequantize_values(codes: torch.Tensor, norms: torch.Tensor, k: TurboQuantConstants, dtype=torch.float32):
    u = k.value_codebook[codes.long()]
    return ((u @ k.rotation_matrix) * norms[..., None]).to(dtype)


def quantize_keys(x: torch.Tensor, k: TurboQuantConstants):
    """x ``[..., d]`` -> (codes uint8, norms fp32, sign bits bool ``[..., m]``, residual norms fp32)."""
    xf = x.float()
    norm = xf.norm(dim=-1)
    u = (xf / norm.clamp_min(1e-20)[..., None]) @ k.rotation_matrix.t()
    codes = _nearest(u, k.key_codebook)
    r = (u - k.key_codebook[codes]) @ k.rotation_matrix           # residual back in the original basis
    return codes.to(torch.uint8), norm, (r @ k.qjl_projection.t()) >= 0, r.norm(dim=-1)


def key_scores(q: torch.Tensor, codes, norms, signs, rnorms, k: TurboQuantConstants) -> torch.Tensor:
    """Unbiased estimate of ``q @ K^T``: q ``[..., Tq, d]``, compressed keys of ``Tk`` tokens -> ``[..., Tq, Tk]``."""
    qf = q.float()
    main = (qf @ k.rotation_matrix.t()) @ k.key_codebook[codes.long()].transpose(-1, -2)
    sketch = (qf @ k.qjl_projection.t()) @ (signs.float() * 2 - 1).transpose(-1, -2)
    corr = sketch * (math.sqrt(math.pi / 2) / k.qjl_dim) * rnorms[..., None, :]
    return (main + corr) * norms[..., None, :]


def attention(q, kq: tuple, vq: tuple, k: TurboQuantConstants, scale: float | None = None, causal: bool = True):
    """Softmax attention over a compressed cache. q ``[B, H, Tq, d]``; ``kq`` / ``vq`` as returned by the quantisers
    for ``[B, H, Tk, d]`` keys / values (the query rows are the last ``Tq`` positions)."""
    d = q.shape[-1]
    s = key_scores(q, *kq, k) * (scale if scale is not None else d ** -0.5)
    Tq, Tk = s.shape[-2:]
    if causal:
        qpos = torch.arange(Tk - Tq, Tk, device=s.device)[:, None]
        s = s.masked_fill(torch.arange(Tk, device=s.device)[None, :] > qpos, float("-inf"))
    return torch.softmax(s, -1) @ dequantize_values(*vq, k)


def compression_ratio(config: TurboQuantConfig, head_dim: int) -> float:
    """bf16 bytes over compressed bytes for one (key, value) pair of a head."""
    m = config.qjl_dim or head_dim
    key_bits = head_dim * config.key_codebook_bits + m + 2 * 32
    val_bits = head_dim * config.value_codebook_bits + 32
    return (2 * head_dim * 16) / (key_bits + val_bits)
