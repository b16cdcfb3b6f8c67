"""RMSNorm / QKNorm modules (reference: triton_kernels/modules/normalization.py:8-26)."""
from __future__ import annotations

import torch
from torch import Tensor, nn

from triton_kernels_b200.kernels.normalization import rms_norm


class RMSNorm(nn.Module):
    """Learned-scale RMS normalisation over the last dim; parameter `scale`, initialised to 1."""

    def __init__(self, dim: int) -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        return rms_norm(x, self.scale)


class QKNorm(nn.Module):
    """Independent RMSNorm for queries and keys; results take v's dtype."""

    def __init__(self, dim: int) -> None:
        super().__init__()
        self.query_norm = RMSNorm(dim)
        self.key_norm = RMSNorm(dim)

    def forward(self, q: Tensor, k: Tensor, v: Tensor) -> tuple[Tensor, Tensor]:
        return self.query_norm(q).to(v), self.key_norm(k).to(v)
