"""Library + NCCL comparator for the headline benchmark (``bench.py --impl library``).

The same Llama-3-8B SFT step as ``bench.py`` measures, written the way a PyTorch user would
write it with stock parts only: ``nn.Linear`` (cuBLAS), ``scaled_dot_product_attention`` (the
library flash kernel), ``F.rms_norm``, ``F.cross_entropy`` over materialised logits,
``torch.utils.checkpoint`` around every decoder layer, FSDP2 (``fully_shard``: NCCL all-gather of
bf16 parameters, fp32 reduce-scatter of gradients) and the unfused ``torch.optim.AdamW`` over
fp32 master weights. Nothing from ``easydel_b200`` is imported here; the numbers this arm prints
say what the libraries alone get out of the same GPUs on the same config.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


class _Block(nn.Module):
    def __init__(self, hidden: int, ffn: int, heads: int, kv_heads: int, head_dim: int, eps: float):
        super().__init__()
        self.heads, self.kv_heads, self.head_dim, self.eps = heads, kv_heads, head_dim, eps
        self.input_norm = nn.Parameter(torch.ones(hidden))
        self.post_norm = nn.Parameter(torch.ones(hidden))
        self.qkv = nn.Linear(hidden, (heads + 2 * kv_heads) * head_dim, bias=False)
        self.o = nn.Linear(heads * head_dim, hidden, bias=False)
        self.gate_up = nn.Linear(hidden, 2 * ffn, bias=False)
        self.down = nn.Linear(ffn, hidden, bias=False)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        B, T, H = x.shape
        h = F.rms_norm(x, (H,), self.input_norm, self.eps)
        qkv = self.qkv(h)
        q, k, v = qkv.split([self.heads * self.head_dim, self.kv_heads * self.head_dim,
                             self.kv_heads * self.head_dim], dim=-1)
        q = q.view(B, T, self.heads, self.head_dim).transpose(1, 2)
        k = k.view(B, T, self.kv_heads, self.head_dim).transpose(1, 2)
        v = v.view(B, T, self.kv_heads, self.head_dim).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, T, -1))
        h = F.rms_norm(x, (H,), self.post_norm, self.eps)
        g, u = self.gate_up(h).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class LibraryLlama(nn.Module):
    def __init__(self, vocab: int, hidden: int, ffn: int, layers: int, heads: int, kv_heads: int, head_dim: int,
                 eps: float, theta: float, max_len: int):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.layers = nn.ModuleList([_Block(hidden, ffn, heads, kv_heads, head_dim, eps) for _ in range(layers)])
        self.final_norm = nn.Parameter(torch.ones(hidden))
        self.lm_head = nn.Linear(hidden, vocab, bias=False)
        self.eps = eps
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        ang = torch.arange(max_len, dtype=torch.float32)[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos()[None, None], persistent=False)
        self.register_buffer("sin", ang.sin()[None, None], persistent=False)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        T = ids.shape[1]
        cos, sin = self.cos[:, :, :T].to(torch.bfloat16), self.sin[:, :, :T].to(torch.bfloat16)
        x = self.embed(ids)
        for blk in self.layers:
            x = checkpoint(blk, x, cos, sin, use_reentrant=False)
        x = F.rms_norm(x, (x.shape[-1],), self.final_norm, self.eps)
        logits = self.lm_head(x)
        return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1))


def build(dev: torch.device, world: int, *, vocab: int, layers: int, seq: int):
    """Random-init Llama-3-8B geometry, FSDP2-wrapped per decoder layer, and its optimizer."""
    torch.manual_seed(1234)
    with torch.device("meta"):
        model = LibraryLlama(vocab, 4096, 14336, layers, 32, 8, 128, 1e-5, 500000.0, seq)
    how = "fsdp2 (fully_shard per layer, bf16 params / fp32 reduce, NCCL)"
    try:
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for blk in model.layers:
            fully_shard(blk, mp_policy=mp, reshard_after_forward=world > 1)
        fully_shard(model, mp_policy=mp, reshard_after_forward=world > 1)
        model.to_empty(device=dev)
        autocast = False
    except Exception as e:  # a torch build without FSDP2 for this world size: plain autocast over fp32 weights
        if world > 1:
            raise
        how = f"single GPU, torch.autocast(bf16) over fp32 weights (fully_shard unavailable: {type(e).__name__})"
        model.to_empty(device=dev)
        autocast = True
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm"):
                p.fill_(1.0)
            else:
                nn.init.normal_(p, std=0.02)
        inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32, device=dev) / 128))
        ang = torch.arange(seq, dtype=torch.float32, device=dev)[:, None] * inv[None, :]
        model.cos, model.sin = ang.cos()[None, None], ang.sin()[None, None]
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01,
                            foreach=True, fused=False)
    return model, opt, autocast, how


def train_step(model, opt, batch: dict, micro: int, autocast: bool, clip: float = 1.0) -> torch.Tensor:
    """One optimizer step over ``micro`` micro-batches of one sequence each; returns the mean loss (device)."""
    ids, labels = batch["input_ids"], batch["labels"]
    n = ids.shape[0] // micro
    total = torch.zeros((), device=ids.device)
    sync_ctl = hasattr(model, "set_requires_gradient_sync")
    for i in range(micro):
        if sync_ctl:
            model.set_requires_gradient_sync(i == micro - 1)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            loss = model(ids[i * n:(i + 1) * n], labels[i * n:(i + 1) * n]) / micro
        loss.backward()
        total += loss.detach()
    torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
    opt.step()
    opt.zero_grad(set_to_none=True)
    return total
