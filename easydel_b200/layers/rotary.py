"""Rotary position embeddings: frequency variants and the module that owns the cos/sin tables.

Covers the ``rope_type`` family of the reference (easydel/layers/rotary/_compute_fns.py,
_modules.py:131-1198, _utils.py:165-244): default, linear, dynamic-NTK, YaRN, llama3,
phi-3 long-rope, deepseek-YaRN and multimodal (section-wise) mRoPE. The tables are
fp32 ``[max_position, rot_dim/2]``; the rotation itself runs in the fused
RoPE kernel (or the reference math on CPU) through :func:`easydel_b200.ops.functional.rope_packed`.
"""

from __future__ import annotations

import math
import typing as tp
from dataclasses import dataclass, field

import torch


def _base_inv_freq(base: float, rotary_dim: int) -> torch.Tensor:
    return 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def _yarn_find_correction_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_find_correction_range(low_rot: float, high_rot: float, dim: int, base: float, max_pos: int,
                                truncate: bool = True):
    low = _yarn_find_correction_dim(low_rot, dim, base, max_pos)
    high = _yarn_find_correction_dim(high_rot, dim, base, max_pos)
    if truncate:
        low, high = math.floor(low), math.ceil(high)
    return max(low, 0), min(high, dim - 1)


def _yarn_linear_ramp(low: float, high: float, n: int) -> torch.Tensor:
    if low == high:
        high += 0.001
    return ((torch.arange(n, dtype=torch.float32) - low) / (high - low)).clamp_(0, 1)


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


@dataclass
class RopeConfig:
    """Normalised view of HF's ``rope_scaling`` / ``rope_parameters`` dict."""

    rope_type: str = "default"
    factor: float | None = None
    original_max_position_embeddings: int | None = None
    low_freq_factor: float | None = None
    high_freq_factor: float | None = None
    beta_fast: float | None = None
    beta_slow: float | None = None
    mscale: float | None = None
    mscale_all_dim: float | None = None
    attention_factor: float | None = None
    short_factor: list[float] | None = None
    long_factor: list[float] | None = None
    mrope_section: list[int] | None = None
    mrope_interleaved: bool = False
    truncate: bool = True
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict | None) -> "RopeConfig":
        if not d:
            return cls()
        d = dict(d)
        rt = d.pop("rope_type", None) or d.pop("type", None) or "default"
        if rt == "su":
            rt = "longrope"
        known = {k: d.pop(k) for k in list(d) if k in cls.__dataclass_fields__ and k not in ("rope_type", "extra")}
        return cls(rope_type=rt, extra=d, **known)

    def to_dict(self) -> dict:
        out = {"rope_type": self.rope_type}
        for k in self.__dataclass_fields__:
            if k in ("rope_type", "extra"):
                continue
            v = getattr(self, k)
            if v is not None and v is not False and not (k == "truncate" and v is True):
                out[k] = v
        out.update(self.extra)
        return out


def get_inv_frequencies(rope: RopeConfig, base: float, rotary_dim: int, max_position: int,
                        seq_len: int | None = None) -> tuple[torch.Tensor, float]:
    """Returns (inv_freq [rot/2], attention_scaling) for the configured variant."""
    t = rope.rope_type
    inv = _base_inv_freq(base, rotary_dim)
    scaling = 1.0
    if t in ("default", "mrope", None):
        pass
    elif t == "linear":
        inv = inv / float(rope.factor or 1.0)
    elif t == "dynamic":
        factor = float(rope.factor or 1.0)
        orig = rope.original_max_position_embeddings or max_position
        sl = max(seq_len or max_position, orig)
        nb = base * ((factor * sl / orig) - (factor - 1)) ** (rotary_dim / (rotary_dim - 2))
        inv = _base_inv_freq(nb, rotary_dim)
    elif t == "llama3":
        factor = float(rope.factor or 8.0)
        lo = float(rope.low_freq_factor or 1.0)
        hi = float(rope.high_freq_factor or 4.0)
        old = float(rope.original_max_position_embeddings or 8192)
        low_wl, high_wl = old / lo, old / hi
        wl = 2 * math.pi / inv
        scaled = torch.where(wl > low_wl, inv / factor, inv)
        smooth = (old / wl - lo) / (hi - lo)
        smoothed = (1 - smooth) * inv / factor + smooth * inv
        mid = (wl >= high_wl) & (wl <= low_wl)
        inv = torch.where(mid, smoothed, scaled)
    elif t in ("yarn", "deepseek_yarn"):
        factor = float(rope.factor or 1.0)
        orig = rope.original_max_position_embeddings or max_position
        bf = float(rope.beta_fast or 32.0)
        bs = float(rope.beta_slow or 1.0)
        low, high = _yarn_find_correction_range(bf, bs, rotary_dim, base, orig, rope.truncate)
        extrap = inv
        interp = inv / factor
        mask = 1.0 - _yarn_linear_ramp(low, high, rotary_dim // 2)
        inv = interp * (1 - mask) + extrap * mask
        if rope.attention_factor is not None:
            scaling = float(rope.attention_factor)
        elif rope.mscale is not None and rope.mscale_all_dim is not None:
            scaling = yarn_get_mscale(factor, float(rope.mscale)) / yarn_get_mscale(factor, float(rope.mscale_all_dim))
        else:
            scaling = yarn_get_mscale(factor, float(rope.mscale or 1.0)) if t == "deepseek_yarn" else (
                0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0)
    elif t == "longrope":
        orig = rope.original_max_position_embeddings or max_position
        sl = seq_len or max_position
        ext = torch.tensor(rope.long_factor if sl > orig else rope.short_factor, dtype=torch.float32)
        inv = 1.0 / (ext * base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
        factor = rope.factor or (max_position / orig)
        if rope.attention_factor is not None:
            scaling = float(rope.attention_factor)
        else:
            scaling = 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(orig))
    else:
        raise ValueError(f"unknown rope_type {t!r}")
    return inv, scaling


def get_frequencies(rope: RopeConfig, base: float, rotary_dim: int, max_position: int) -> tuple[torch.Tensor,
                                                                                                 torch.Tensor]:
    """cos / sin tables ``[max_position, rot/2]`` in fp32, attention scaling folded in."""
    inv, scaling = get_inv_frequencies(rope, base, rotary_dim, max_position, seq_len=max_position)
    pos = torch.arange(max_position, dtype=torch.float32)
    ang = torch.outer(pos, inv)
    return (ang.cos() * scaling).contiguous(), (ang.sin() * scaling).contiguous()


class RotaryEmbedding(torch.nn.Module):
    """Owns the tables and applies the rotation to packed projections.

    ``is_neox_style=True`` rotates halves (Llama, Qwen, Mistral...), False rotates interleaved
    pairs (GPT-J style). ``rotary_dim < head_size`` gives partial rotary (Phi, GPT-NeoX, GLM).
    """

    def __init__(self, head_size: int, rotary_dim: int, max_position: int, base: float, is_neox_style: bool = True,
                 rope_scaling: dict | RopeConfig | None = None, dtype=None):
        super().__init__()
        self.head_size = head_size
        self.rotary_dim = rotary_dim
        self.max_position = max_position
        self.base = base
        self.is_neox_style = is_neox_style
        self.rope = rope_scaling if isinstance(rope_scaling, RopeConfig) else RopeConfig.from_dict(rope_scaling)
        cos, sin = get_frequencies(self.rope, base, rotary_dim, max_position)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def extra_repr(self) -> str:
        return (f"head_size={self.head_size}, rotary_dim={self.rotary_dim}, max_position={self.max_position}, "
                f"base={self.base}, type={self.rope.rope_type}")

    def tables(self, device) -> tuple[torch.Tensor, torch.Tensor]:
        if self.cos.device != device:
            self.cos = self.cos.to(device)
            self.sin = self.sin.to(device)
        return self.cos, self.sin

    def rotate_packed(self, qkv: torch.Tensor, positions: torch.Tensor, n_heads: int, col0: int = 0,
                      inplace: bool = False) -> torch.Tensor:
        """Rotates ``n_heads`` consecutive heads of a packed projection ``[..., width]`` starting at ``col0``
        (``inplace``: in the projection's own memory when no gradient is needed)."""
        from ..ops import functional as F

        cos, sin = self.tables(qkv.device)
        shape = qkv.shape
        out = F.rope_packed(qkv.reshape(-1, shape[-1]), positions.reshape(-1), cos, sin, n_heads, self.head_size,
                            col0=col0, rot_dim=self.rotary_dim, interleaved=not self.is_neox_style, inplace=inplace)
        return out.view(shape)

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor):
        """q ``[..., Hq, D]``, k ``[..., Hk, D]`` -> rotated copies (reference-style call signature)."""
        from ..ops import reference as R

        cos, sin = self.tables(q.device)
        pos = positions.reshape(-1)
        q2 = R.apply_rope(q.reshape(-1, q.shape[-2], q.shape[-1]), pos, cos, sin, self.rotary_dim,
                          not self.is_neox_style).view(q.shape)
        k2 = R.apply_rope(k.reshape(-1, k.shape[-2], k.shape[-1]), pos, cos, sin, self.rotary_dim,
                          not self.is_neox_style).view(k.shape)
        return q2, k2


class MultiModalRotaryEmbedding(RotaryEmbedding):
    """mRoPE (Qwen2-VL family): three position streams (temporal, height, width) own sections of the
    frequency axis (easydel/layers/rotary/_modules.py, ``mrope_section``)."""

    def cos_sin_for(self, positions3: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """positions3 ``[3, T]`` -> per-token cos/sin ``[T, rot/2]`` assembled section-wise."""
        cos, sin = self.tables(positions3.device)
        sec = self.rope.mrope_section or [self.rotary_dim // 2]
        if self.rope.mrope_interleaved and positions3.shape[0] == 3:
            # frequencies cycle through the streams (T H W T H W ... T T): H owns 1, 4, 7, ... below 3 * sec[1],
            # W owns 2, 5, 8, ... below 3 * sec[2], the temporal stream keeps the rest
            c, s = cos[positions3[0]].clone(), sin[positions3[0]].clone()
            for dim, off in ((1, 1), (2, 2)):
                idx = slice(off, sec[dim] * 3, 3)
                c[:, idx], s[:, idx] = cos[positions3[dim]][:, idx], sin[positions3[dim]][:, idx]
            return c, s
        outs_c, outs_s, start = [], [], 0
        for i, n in enumerate(sec):
            p = positions3[i % positions3.shape[0]]
            outs_c.append(cos[p][:, start:start + n])
            outs_s.append(sin[p][:, start:start + n])
            start += n
        return torch.cat(outs_c, -1), torch.cat(outs_s, -1)

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor):
        from ..ops import reference as R

        if positions.dim() == 1 or positions.shape[0] != 3:
            return super().forward(positions, q, k)
        c, s = self.cos_sin_for(positions.reshape(3, -1))

        def rot(x):
            x3 = x.reshape(-1, x.shape[-2], x.shape[-1])
            xr = R.rotate(x3[..., : self.rotary_dim].float(), c[:, None], s[:, None], not self.is_neox_style)
            if self.rotary_dim < x.shape[-1]:
                xr = torch.cat([xr, x3[..., self.rotary_dim:].float()], -1)
            return xr.to(x.dtype).view(x.shape)

        return rot(q), rot(k)


_ROPE_CACHE: dict[tuple, RotaryEmbedding] = {}


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float, is_neox_style: bool = True,
             rope_scaling: dict | None = None, dtype=None, partial_rotary_factor: float = 1.0) -> RotaryEmbedding:
    """Factory with a cache keyed on the full parameter set (as easydel/layers/rotary get_rope does)."""
    if partial_rotary_factor < 1.0:
        rotary_dim = int(rotary_dim * partial_rotary_factor)
        rotary_dim -= rotary_dim % 2
    key = (head_size, rotary_dim, max_position, float(base), is_neox_style,
           None if not rope_scaling else tuple(sorted((k, str(v)) for k, v in dict(rope_scaling).items())))
    if key not in _ROPE_CACHE:
        cfg = RopeConfig.from_dict(rope_scaling)
        cls = MultiModalRotaryEmbedding if cfg.mrope_section else RotaryEmbedding
        _ROPE_CACHE[key] = cls(head_size, rotary_dim, max_position, base, is_neox_style, cfg)
    return _ROPE_CACHE[key]
