"""Token embedding (easydel/layers/embeddings/_embeddings.py:66-227)."""

from __future__ import annotations

import torch
from torch import nn

from ..ops import functional as F


class Embed(nn.Module):
    parallel_style = "column"  # same semantic spec as a column-parallel kernel in the reference

    def __init__(self, num_embeddings: int, features: int, dtype: torch.dtype = torch.float32, init_std: float = 0.02,
                 padding_idx: int | None = None, device=None):
        super().__init__()
        self.num_embeddings, self.features, self.padding_idx = num_embeddings, features, padding_idx
        self.weight = nn.Parameter(torch.empty(num_embeddings, features, dtype=dtype, device=device))
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, 0.0, init_std)
            if padding_idx is not None:
                with torch.no_grad():
                    self.weight[padding_idx].zero_()

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return F.embedding(self.weight, ids)

    def attend(self, h: torch.Tensor) -> torch.Tensor:
        """Tied LM head: ``h @ E^T``."""
        return F.linear(h, self.weight)
