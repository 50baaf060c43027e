"""Plain PyTorch implementations of every op in this package.

They serve two purposes: they are the oracle the CUDA kernels are tested
against (run them in fp32), and they are the execution path for CPU tensors
(config-1 style plumbing runs, unit tests, multi-rank gloo tests). They are
written for clarity, not speed, and are differentiable through autograd.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

ACT2FN = {
    "silu": F.silu,
    "swish": F.silu,
    "gelu": F.gelu,
    "gelu_new": lambda x: F.gelu(x, approximate="tanh"),
    "gelu_tanh": lambda x: F.gelu(x, approximate="tanh"),
    "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh"),
    "relu": F.relu,
    "relu2": lambda x: F.relu(x).square(),
    "tanh": torch.tanh,
    "sigmoid": torch.sigmoid,
    "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x),
    "linear": lambda x: x,
}


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


def rms_norm(x, w, eps, w_offset: float = 0.0):
    dt = x.dtype
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * (w.float() + w_offset)).to(dt)


def layer_norm(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), None if w is None else w.float(), None if b is None else b.float(),
                        eps).to(x.dtype)


def _gptoss_swiglu(g, u, alpha: float = 1.702, limit: float = 7.0):
    """GPT-OSS expert activation: clamped gate through x*sigmoid(alpha x), clamped linear branch offset by one."""
    g = g.clamp(max=limit)
    u = u.clamp(min=-limit, max=limit)
    return (u + 1) * (g * torch.sigmoid(g * alpha))


# gated activations that are not of the form act(gate) * up
GATED_FNS = {"gptoss_swiglu": _gptoss_swiglu}


def gated_act(gu, act: str = "silu"):
    g, u = gu.chunk(2, dim=-1)
    if act in GATED_FNS:
        return GATED_FNS[act](g, u)
    return ACT2FN[act](g) * u


def rotate(x, cos, sin, interleaved: bool = False):
    """x: [..., rot]; cos/sin broadcastable [..., rot/2]."""
    if interleaved:
        x1, x2 = x[..., 0::2], x[..., 1::2]
        return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def apply_rope(x, pos, cos_table, sin_table, rot_dim=None, interleaved: bool = False):
    """x: [T, H, D]; pos: [T]; tables [maxpos, rot/2] fp32. Returns the same dtype as x."""
    D = x.shape[-1]
    rot = rot_dim or D
    c = cos_table[pos][:, None, :]
    s = sin_table[pos][:, None, :]
    xr = rotate(x[..., :rot].float(), c, s, interleaved)
    if rot < D:
        xr = torch.cat([xr, x[..., rot:].float()], dim=-1)
    return xr.to(x.dtype)


def attention(q, k, v, *, causal: bool = True, scale: float | None = None, segment_ids=None, q_offset=None,
              sliding_window: int | None = None, softcap: float = 0.0, sinks=None, bias=None, kv_segment_ids=None,
              return_lse: bool = False):
    """Dense softmax attention, the oracle for the flash kernels.

    q: [B, Tq, Hq, D]; k, v: [B, Tk, Hkv, D]. GQA by repeating KV heads.
    ``segment_ids`` [B, Tq] (0 = padding): tokens attend only inside their segment.
    ``q_offset`` [B] or int: absolute position of q row 0 relative to k row 0
    (default Tk - Tq, i.e. the queries are the last Tq positions).
    ``sinks`` [Hq]: per-head extra logit that joins the softmax but carries no value.
    """
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    if bias is not None:
        s = s + bias.float()
    if q_offset is None:
        q_offset = Tk - Tq
    qpos = torch.arange(Tq, device=q.device)[None, :] + (
        q_offset[:, None] if isinstance(q_offset, torch.Tensor) else q_offset)
    kpos = torch.arange(Tk, device=q.device)[None, :]
    mask = torch.ones(B, Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= kpos[:, None, :] <= qpos[:, :, None]
    if sliding_window is not None and sliding_window > 0:
        mask &= kpos[:, None, :] > (qpos[:, :, None] - sliding_window)
    if segment_ids is not None:
        ks = kv_segment_ids if kv_segment_ids is not None else segment_ids
        mask &= (segment_ids[:, :, None] == ks[:, None, :]) & (ks[:, None, :] != 0)
    s = s.masked_fill(~mask[:, None], float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(1, Hq, 1, 1).expand(B, Hq, Tq, 1)
        s_all = torch.cat([s, sk], dim=-1)
        lse = torch.logsumexp(s_all, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    lse_safe = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    p = torch.exp(s - lse_safe[..., None])
    p = torch.where(mask[:, None], p, torch.zeros_like(p))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return o, lse
    return o


def cross_entropy(logits, labels, *, ignore_index: int = -100, label_smoothing: float = 0.0, z_loss: float = 0.0,
                  softcap: float = 0.0):
    """Per-token loss [rows] in fp32 (0 where ignored), plus lse."""
    z = logits.float()
    if softcap and softcap > 0:
        z = softcap * torch.tanh(z / softcap)
    lse = torch.logsumexp(z, dim=-1)
    valid = labels != ignore_index
    safe = labels.clamp(min=0)
    zl = z.gather(-1, safe[..., None]).squeeze(-1)
    loss = (1 - label_smoothing) * (lse - zl) + label_smoothing * (lse - z.mean(-1)) + z_loss * lse.pow(2)
    return torch.where(valid, loss, torch.zeros_like(loss)), lse


def token_logprob(logits, labels, *, ignore_index: int = -100, temperature: float = 1.0):
    z = logits.float() / temperature
    lp = torch.log_softmax(z, dim=-1)
    safe = labels.clamp(min=0)
    out = lp.gather(-1, safe[..., None]).squeeze(-1)
    return torch.where(labels != ignore_index, out, torch.zeros_like(out))


def adamw_step(p, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step):
    """In-place AdamW on fp32 tensors with decoupled weight decay (torch.optim.AdamW semantics)."""
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    p.mul_(1 - lr * weight_decay)
    p.addcdiv_(m / bc1, denom, value=-lr)
    return p


def moe_router(logits, top_k: int, norm_topk: bool = True, scoring: str = "softmax"):
    """fp32 routing: probabilities over all experts, top-k, optional renormalisation."""
    lf = logits.float()
    probs = torch.softmax(lf, dim=-1) if scoring == "softmax" else torch.sigmoid(lf)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w, idx, probs


def moe_experts(x, w_gate_up, w_down, topk_w, topk_idx, act: str = "silu"):
    """Dense per-expert loop. w_gate_up [E, 2F, H], w_down [E, H, F] (torch Linear layout per expert)."""
    T, H = x.shape
    E = w_gate_up.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = (topk_idx == e)
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = gated_act(F.linear(x[tok], w_gate_up[e]), act)
        y = F.linear(h, w_down[e]).float()
        out.index_add_(0, tok, y * topk_w[tok, slot].float()[:, None])
    return out.to(x.dtype)
