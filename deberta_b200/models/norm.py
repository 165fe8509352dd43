"""RMSNorm module (fp32 reduction, ``norm.py:9-47`` of the reference)."""

from __future__ import annotations

import torch
from torch import nn

from deberta_b200.ops.norm import rms_norm


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x²) + eps) * weight``."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(int(hidden_size)))
        self.eps = float(eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.eps}"
