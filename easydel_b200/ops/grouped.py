"""Expert (grouped) GEMMs and the token permutation around them.

``moe_ffn`` is the dropless expert FFN: tokens are repeated ``k`` times, sorted by expert into
segments padded to a multiple of 128 rows, pushed through two grouped GEMMs with the gated
activation in between, and combined back per token in fp32 with the routing weights
(easydel/layers/moe/_communication_utils.py:764-963, ``grouped_matmul`` at
easydel/layers/moe/_moe_module.py:1110-1124). CUDA tensors use the kernels in
``csrc/moe.cu`` / ``csrc/gemm_grouped.cu``; CPU tensors use the dense per-expert oracle.
"""

from __future__ import annotations

import torch

from . import _lib, functional as F, reference as R


def _sort_by_expert(topk_idx: torch.Tensor, num_experts: int):
    """Stable sort of the flattened (token, slot) pairs by expert id."""
    flat = topk_idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    group_sizes = torch.bincount(flat, minlength=num_experts)
    return order, group_sizes


def grouped_linear(x_sorted: torch.Tensor, w: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """``y[rows of group e] = x[rows of group e] @ w[e].T`` with ``w`` ``[E, out, in]``.

    Rows of ``x_sorted`` are grouped by expert in order; ``group_sizes`` ``[E]`` gives the counts.
    """
    if _lib.use_kernels(x_sorted):
        from . import moe_kernels as MK

        return MK.grouped_linear(x_sorted, w, group_sizes)
    outs = []
    start = 0
    for e, n in enumerate(group_sizes.tolist()):
        outs.append(R.linear(x_sorted[start:start + n], w[e]))
        start += n
    return torch.cat(outs, dim=0) if outs else x_sorted.new_zeros(0, w.shape[1])


def moe_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, topk_w: torch.Tensor,
            topk_idx: torch.Tensor, act: str = "silu", expert_offset: int = 0, b_gate_up: torch.Tensor | None = None,
            b_down: torch.Tensor | None = None) -> torch.Tensor:
    """Dropless routed-expert FFN on one device. x ``[T,H]``, topk_* ``[T,k]`` -> ``[T,H]``.

    ``b_gate_up`` ``[E, 2F]`` / ``b_down`` ``[E, H]`` are per-expert biases (GPT-OSS); with them, or with a gated
    activation outside the fused kernels' set, the GPU path composes the grouped GEMMs with elementwise torch ops.
    """
    if _lib.use_kernels(x):
        from . import moe_kernels as MK

        if b_gate_up is None and b_down is None and act in MK.K.ACT_IDS:
            return MK.moe_ffn(x, w_gate_up, w_down, topk_w, topk_idx, act, expert_offset)
        return MK.moe_ffn_composed(x, w_gate_up, w_down, topk_w, topk_idx, act, b_gate_up, b_down, expert_offset)
    T, H = x.shape
    k = topk_idx.shape[1]
    E = w_gate_up.shape[0]
    if expert_offset:
        raise ValueError("the CPU path takes local expert indices")
    order, group_sizes = _sort_by_expert(topk_idx, E)
    tok = order // k
    xs = x[tok]
    row_e = topk_idx.reshape(-1)[order]
    h = grouped_linear(xs, w_gate_up, group_sizes)
    if b_gate_up is not None:
        h = h + b_gate_up[row_e]
    a = F.gated_act(h, act)
    ys = grouped_linear(a, w_down, group_sizes)
    if b_down is not None:
        ys = ys + b_down[row_e]
    wflat = topk_w.reshape(-1)[order].to(torch.float32)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out = out.index_add(0, tok, ys.float() * wflat[:, None])
    return out.to(x.dtype)
