"""Mixture-of-experts block: router, token permutation, expert FFNs, weighted combine, aux losses.

Behavioural counterpart of ``BaseMoeModule`` (easydel/layers/moe/_moe_module.py:108-1791) and the
permutation helpers in ``_communication_utils.py:764-963``:

* router logits -> fp32 softmax (or sigmoid) over all experts -> top-k -> optional renormalisation
  (``TOP_K`` vs ``TOP_K_NDIV``), DeepSeek group-limited selection and score-correction bias;
* tokens are repeated ``k`` times and sorted by expert (dropless, no capacity), the experts run as
  one grouped GEMM over the ragged groups, outputs are un-sorted and combined in fp32;
* load-balancing auxiliary loss and router z-loss are returned for the model to add to the loss.

Expert weights are stacked ``[E, out, in]`` (torch layout per expert); the checkpoint writer
stores them as the reference's ``(E, in, out)`` kernels. Under expert parallelism each rank
owns ``E / ep`` experts and ``parallel.ep`` moves tokens between ranks around the grouped GEMM.
"""

from __future__ import annotations

import typing as tp

import torch
from torch import nn

from ..ops import functional as F
from ..ops import grouped as G
from .linears import ColumnParallelLinear
from .mlp import GatedMLP


class MoELinear(nn.Module):
    """Stacked expert weights ``[E_local, out, in]`` (ParallelMoELinear, _linear_moe.py:90-542)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, dtype=torch.float32,
                 init_std: float = 0.01, parallel_style: str = "column", device=None, bias: bool = False):
        super().__init__()
        self.num_experts, self.in_features, self.out_features = num_experts, in_features, out_features
        self.parallel_style = parallel_style
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features, dtype=dtype, device=device))
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, 0.0, init_std)
        self.bias = nn.Parameter(torch.zeros(num_experts, out_features, dtype=dtype, device=device)) if bias else None

    def forward(self, x_sorted: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
        return G.grouped_linear(x_sorted, self.weight, group_sizes)


def load_balancing_loss(router_probs: torch.Tensor, topk_idx: torch.Tensor, num_experts: int,
                        attention_mask: torch.Tensor | None = None) -> torch.Tensor:
    """Switch-style auxiliary loss ``E * sum_e f_e * P_e`` (easydel/infra/loss_utils.py:1760-1892).

    ``router_probs`` ``[T, E]`` fp32 probabilities, ``topk_idx`` ``[T, k]``.
    """
    T, k = topk_idx.shape
    onehot = torch.zeros(T, num_experts, dtype=torch.float32, device=router_probs.device)
    onehot.scatter_add_(1, topk_idx, torch.ones_like(topk_idx, dtype=torch.float32))
    if attention_mask is not None:
        m = attention_mask.reshape(-1, 1).to(torch.float32)
        denom = m.sum().clamp_min(1.0)
        tokens_per_expert = (onehot * m).sum(0) / denom
        prob_per_expert = (router_probs * m).sum(0) / denom
    else:
        tokens_per_expert = onehot.mean(0)
        prob_per_expert = router_probs.mean(0)
    return num_experts * (tokens_per_expert * prob_per_expert).sum()


def router_z_loss(router_logits: torch.Tensor) -> torch.Tensor:
    return torch.logsumexp(router_logits.float(), dim=-1).pow(2).mean()


class MoeRoutingStrategy:
    """Routing strategies of the reference (easydel/layers/moe/_communication_utils.py:1024-1078)."""

    TOP_K = "top_k"                 # top-k experts per token, weights renormalised to sum to one
    TOP_K_NDIV = "top_k_ndiv"       # top-k experts per token, raw probabilities as weights
    SWITCH = "switch"               # one expert per token, weight exactly one
    EMPTY_CHOICE = "expert_choice"  # every expert picks its own tokens (capacity = tokens * k / experts)
    HASH = "hash"                   # token -> experts by token position, uniform weights (debugging / baselines)


class MoeLoadBalancingStrategy:
    """Auxiliary load-balancing losses (easydel/layers/moe/_moe_module.py:440-510)."""

    STANDARD = "standard"
    SWITCH_TRANSFORMER = "switch_transformer"
    EMPTY_CHOICE = "expert_choice"
    NONE = "none"


def load_balancing_loss_by_strategy(router_probs: torch.Tensor, expert_loads: torch.Tensor, num_experts: int, top_k: int,
                                    strategy: str = MoeLoadBalancingStrategy.STANDARD,
                                    coef: float | None = 1.0) -> torch.Tensor | None:
    """``router_probs`` ``[T, E]`` fp32, ``expert_loads`` ``[E]`` token counts per expert."""
    if strategy == MoeLoadBalancingStrategy.NONE or coef is None:
        return None
    loads = expert_loads.to(torch.float32)
    if strategy == MoeLoadBalancingStrategy.STANDARD:
        return coef * ((loads * num_experts / top_k) * router_probs.mean(0)).sum()
    if strategy == MoeLoadBalancingStrategy.SWITCH_TRANSFORMER:
        return coef * num_experts * ((loads / router_probs.shape[0]) * router_probs.mean(0)).sum()
    if strategy == MoeLoadBalancingStrategy.EMPTY_CHOICE:
        return coef * loads.var(unbiased=False)
    raise ValueError(f"Unknown load balancing strategy: {strategy}")


def apply_capacity(idx: torch.Tensor, weights: torch.Tensor, num_experts: int, capacity: int):
    """Token-choice routing with a per-expert capacity: of the tokens that chose an expert, the first ``capacity``
    (in token order, first choices before second choices) keep it; the others lose that choice (weight zero).
    Returns ``(weights with dropped choices zeroed, keep mask [T, k])``."""
    T, k = idx.shape
    flat = idx.t().reshape(-1)                       # choice-major: every token's first choice comes first
    onehot = torch.nn.functional.one_hot(flat, num_experts)
    rank_in_expert = (onehot.cumsum(0) - 1).gather(1, flat[:, None])[:, 0]
    keep = (rank_in_expert < capacity).view(k, T).t()
    return weights * keep.to(weights.dtype), keep


class MoEBlock(nn.Module):
    """Router + routed experts (+ optional shared experts)."""

    def __init__(self, hidden_size: int, moe_intermediate_size: int, num_experts: int, top_k: int, *,
                 act: str = "silu", norm_topk_prob: bool = True, scoring: str = "softmax",
                 routed_scaling_factor: float = 1.0, n_group: int = 1, topk_group: int = 1,
                 use_score_bias: bool = False, router_bias: bool = False, shared_intermediate_size: int = 0,
                 shared_gate: bool = False, dtype=torch.float32, init_std: float = 0.02, expert_init_std: float = 0.01,
                 ep_size: int = 1, ep_rank: int = 0, ep_group=None, tp_size: int = 1, tp_rank: int = 0,
                 tp_group=None, router_dtype=None, expert_bias: bool = False, scale_input: bool = False,
                 router_jitter_eps: float = 0.01, routing_strategy: str | None = None,
                 capacity_factor: float | None = None,
                 load_balancing_strategy: str = MoeLoadBalancingStrategy.STANDARD, lbl_coef: float | None = None,
                 rzl_coef: float | None = None, expert_tensor_mode: bool = False):
        super().__init__()
        # Expert tensor mode (the reference's ``use_expert_tensor_mode``, easydel/layers/linears/_linear_moe.py:113,
        # :330): the experts are spread over the TENSOR-parallel group instead of an expert-parallel one. Every rank
        # of that group sees the same tokens, so nothing is exchanged: a rank runs its own experts on all tokens and
        # the partial outputs are summed over the group.
        self.expert_tensor_mode = bool(expert_tensor_mode and tp_size > 1 and ep_size == 1)
        if self.expert_tensor_mode:
            ep_size, ep_rank, ep_group = tp_size, tp_rank, tp_group
        # None = top-k with (TOP_K) or without (TOP_K_NDIV) renormalisation, as ``norm_topk_prob`` says
        self.routing_strategy = getattr(routing_strategy, "value", routing_strategy)
        self.capacity_factor = capacity_factor     # None = dropless
        self.load_balancing_strategy = getattr(load_balancing_strategy, "value", load_balancing_strategy)
        self.lbl_coef, self.rzl_coef = lbl_coef, rzl_coef
        self.last_aux_losses: dict[str, torch.Tensor] = {}
        self.router_jitter_eps = router_jitter_eps
        # Llama-4: the routing score multiplies the expert's input instead of its output
        self.scale_input = scale_input
        if num_experts % ep_size:
            raise ValueError(f"{num_experts} experts not divisible by ep={ep_size}")
        self.hidden_size, self.num_experts, self.top_k = hidden_size, num_experts, top_k
        self.act, self.norm_topk_prob, self.scoring = act, norm_topk_prob, scoring
        self.routed_scaling_factor = routed_scaling_factor
        self.n_group, self.topk_group = n_group, topk_group
        self.ep_size, self.ep_rank, self.ep_group = ep_size, ep_rank, ep_group
        self.num_local_experts = num_experts // ep_size
        self.gate = ColumnParallelLinear(hidden_size, num_experts, bias=router_bias, dtype=router_dtype or dtype,
                                         init_std=init_std)
        self.e_score_correction_bias = nn.Parameter(torch.zeros(num_experts, dtype=torch.float32)) \
            if use_score_bias else None
        self.gate_up_proj = MoELinear(self.num_local_experts, hidden_size, 2 * moe_intermediate_size, dtype,
                                      expert_init_std, "column", bias=expert_bias)
        self.down_proj = MoELinear(self.num_local_experts, moe_intermediate_size, hidden_size, dtype,
                                   expert_init_std, "row", bias=expert_bias)
        if ep_size > 1:   # these weights differ per rank: their gradients are not summed over the group
            for lin in (self.gate_up_proj, self.down_proj):
                for p in (lin.weight, lin.bias):
                    if p is not None:
                        p._ep_local = True
                        p._ep_over_tp = self.expert_tensor_mode   # the group they differ over is the tp group
        self.shared_experts = None
        self.shared_expert_gate = None
        if shared_intermediate_size > 0:
            self.shared_experts = GatedMLP(hidden_size, shared_intermediate_size, act, False, dtype, init_std,
                                           tp_size, tp_rank, tp_group)
            if shared_gate:
                self.shared_expert_gate = ColumnParallelLinear(hidden_size, 1, bias=False, dtype=dtype,
                                                               init_std=init_std)

    # ------------------------------------------------------------------ routing
    def _route_sparsemixer(self, lf: torch.Tensor):
        """Phi-3.5-MoE routing (deterministic form): experts are picked one after the other by arg-max; the weight
        of each pick is its softmax probability among the experts whose logit lies within a relative margin
        ``2 * jitter_eps`` of that pick's logit (earlier picks excluded)."""
        eps = self.router_jitter_eps
        scores = lf
        ws, ids = [], []
        for _ in range(self.top_k):
            top, ind = scores.max(dim=-1, keepdim=True)
            factor = lf.abs().clamp(min=top)
            drop = ((top - lf) / factor) > (2 * eps)
            gates = torch.softmax(scores.masked_fill(drop, float("-inf")), dim=-1)
            ws.append(gates.gather(-1, ind))
            ids.append(ind)
            scores = scores.scatter(-1, ind, float("-inf"))
        return torch.cat(ws, -1), torch.cat(ids, -1), torch.softmax(lf, dim=-1)

    def _route_by_strategy(self, lf: torch.Tensor):
        """SWITCH / EXPERT_CHOICE / HASH routing; returns None for the top-k strategies handled by :meth:`route`."""
        st = self.routing_strategy
        T, E = lf.shape
        k = self.top_k
        if st == MoeRoutingStrategy.SWITCH:
            probs = torch.softmax(lf, dim=-1)
            idx = probs.argmax(-1, keepdim=True)
            w = torch.ones(T, 1, dtype=torch.float32, device=lf.device)
            if k > 1:   # the kernels take k choices per token: the others are expert 0 with weight zero
                idx = torch.cat([idx, idx.new_zeros(T, k - 1)], 1)
                w = torch.cat([w, w.new_zeros(T, k - 1)], 1)
            return w, idx, probs
        if st == MoeRoutingStrategy.HASH:
            probs = torch.softmax(lf, dim=-1)
            base = torch.arange(T, device=lf.device)[:, None] * k + torch.arange(k, device=lf.device)[None]
            idx = base % E
            return torch.full((T, k), 1.0 / k, dtype=torch.float32, device=lf.device), idx, probs
        if st == MoeRoutingStrategy.EMPTY_CHOICE:
            # every expert takes its `cap` highest-scoring tokens; a token may be taken by 0..E experts. In the
            # token-major form the kernels use, each token lists up to k of the experts that took it (the ones
            # with its highest scores); choices beyond the experts that took it get weight zero.
            probs = torch.softmax(lf, dim=-1)
            cap = max(1, min(T, int(round(T * k / E * (self.capacity_factor or 1.0)))))
            taken = torch.zeros(T, E, dtype=torch.bool, device=lf.device)
            top_tok = probs.topk(cap, dim=0).indices                    # [cap, E]
            taken.scatter_(0, top_tok, True)
            score = torch.where(taken, probs, probs.new_full((), -1.0))
            val, idx = score.topk(k, dim=-1)
            w = torch.where(val >= 0, torch.full_like(val, 1.0 / k), torch.zeros_like(val))
            return w, idx, probs
        return None

    def aux_losses(self, logits: torch.Tensor, probs: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor) -> dict:
        """Load-balancing loss and router z-loss of this call, when their coefficients are set (the reference's
        ``lbl_coef`` / ``rzl_coef``, easydel/layers/moe/_moe_module.py:440-560)."""
        out = {}
        if self.lbl_coef is not None and self.load_balancing_strategy != MoeLoadBalancingStrategy.NONE:
            used = idx[weights > 0] if weights is not None else idx.reshape(-1)
            loads = torch.bincount(used.reshape(-1), minlength=self.num_experts)
            out["load_balancing_loss"] = load_balancing_loss_by_strategy(
                probs, loads, self.num_experts, self.top_k, self.load_balancing_strategy, self.lbl_coef)
        if self.rzl_coef is not None:
            out["router_z_loss"] = self.rzl_coef * router_z_loss(logits)
        return out

    def route(self, logits: torch.Tensor):
        """Returns (weights [T,k] fp32, idx [T,k] int64, probs [T,E] fp32)."""
        lf = logits.float()
        if self.routing_strategy in (MoeRoutingStrategy.SWITCH, MoeRoutingStrategy.HASH,
                                     MoeRoutingStrategy.EMPTY_CHOICE):
            return self._route_by_strategy(lf)
        if self.scoring == "sparsemixer":
            return self._route_sparsemixer(lf)
        probs = torch.softmax(lf, dim=-1) if self.scoring == "softmax" else torch.sigmoid(lf)
        scores = probs
        if self.e_score_correction_bias is not None:
            scores = probs + self.e_score_correction_bias
        if self.n_group > 1:
            T, E = scores.shape
            g = scores.view(T, self.n_group, E // self.n_group)
            if self.e_score_correction_bias is not None:
                gscore = g.topk(2, dim=-1).values.sum(-1)
            else:
                gscore = g.max(-1).values
            gidx = gscore.topk(self.topk_group, dim=-1).indices
            gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
            # experts of the groups that lost are out of the race: -inf for softmax scores, 0 for the
            # bias-corrected sigmoid scores (DeepSeek-V3 convention)
            fill = float("-inf") if self.e_score_correction_bias is None else 0.0
            scores = torch.where(gmask[..., None] > 0, g, torch.full_like(g, fill)).view(T, E)
        idx = scores.topk(self.top_k, dim=-1).indices
        w = probs.gather(-1, idx)
        renorm = self.norm_topk_prob if self.routing_strategy is None else \
            self.routing_strategy == MoeRoutingStrategy.TOP_K
        if renorm:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        w = w * self.routed_scaling_factor
        if self.capacity_factor is not None:       # capacity path: choices beyond an expert's capacity are dropped
            T = idx.shape[0]
            cap = max(1, int(self.capacity_factor * T * self.top_k / self.num_experts + 0.999))
            w, _ = apply_capacity(idx, w, self.num_experts, cap)
        return w, idx, probs

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor):
        """x ``[B,T,H]`` -> (y ``[B,T,H]``, router_logits ``[B*T,E]``)."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        logits = self.gate(x2)
        w, idx, probs = self.route(logits)
        if self.lbl_coef is not None or self.rzl_coef is not None:
            self.last_aux_losses = self.aux_losses(logits, probs, idx, w)
        if self.scale_input:
            T, k = idx.shape
            x_in = (x2[:, None, :] * w[..., None].to(x2.dtype)).reshape(T * k, -1)
            one = torch.ones(T * k, 1, dtype=w.dtype, device=w.device)
            if self.ep_size > 1:
                from ..parallel import ep as epar

                y = epar.expert_parallel_ffn(self, x_in, one, idx.reshape(T * k, 1))
            else:
                y = G.moe_ffn(x_in, self.gate_up_proj.weight, self.down_proj.weight, one, idx.reshape(T * k, 1),
                              self.act, b_gate_up=self.gate_up_proj.bias, b_down=self.down_proj.bias)
            y = y.view(T, k, -1).sum(1)
        elif self.expert_tensor_mode:
            from ..parallel import tp as tpar

            # same tokens on every rank: local experts on all of them, partial outputs summed over the group; the
            # input and routing-weight gradients are the sums of the ranks' contributions
            xin, win = tpar.copy_to_tp(x2, self.ep_group), tpar.copy_to_tp(w, self.ep_group)
            off = self.ep_rank * self.num_local_experts
            if x2.is_cuda:
                part = G.moe_ffn(xin, self.gate_up_proj.weight, self.down_proj.weight, win, idx, self.act,
                                 b_gate_up=self.gate_up_proj.bias, b_down=self.down_proj.bias, expert_offset=off)
            else:   # reference path: local indices, pairs owned by other ranks get weight zero
                local = idx - off
                mine = (local >= 0) & (local < self.num_local_experts)
                part = G.moe_ffn(xin, self.gate_up_proj.weight, self.down_proj.weight, win * mine.to(win.dtype),
                                 local.clamp(0, self.num_local_experts - 1), self.act,
                                 b_gate_up=self.gate_up_proj.bias, b_down=self.down_proj.bias)
            y = tpar._ReduceFromTP.apply(part, self.ep_group) if torch.is_grad_enabled() else \
                tpar.all_reduce(part, self.ep_group)
        elif self.ep_size > 1:
            from ..parallel import ep as epar

            y = epar.expert_parallel_ffn(self, x2, w, idx)
        else:
            y = G.moe_ffn(x2, self.gate_up_proj.weight, self.down_proj.weight, w, idx, self.act,
                          b_gate_up=self.gate_up_proj.bias, b_down=self.down_proj.bias)
        if self.shared_experts is not None:
            s = self.shared_experts(x2)
            if self.shared_expert_gate is not None:
                s = s * torch.sigmoid(self.shared_expert_gate(x2).float()).to(s.dtype)
            y = y + s
        return y.view(shape), logits
