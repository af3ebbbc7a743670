"""Dense gated feed-forwards of the sequence-mixer model families.

``ClampedGatedFFN``: ``g = min(W_gate h + b, limit)``, ``u = clamp(W_up h + b, -limit, limit)``, ``y = g sigmoid(slope g) (u + 1)``,
output ``W_down y + b``.  The gate and up projections are one stacked product (bias in its epilogue); the activation is one kernel
(``csrc/seqmix/activations.cu``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import seqmix


class ClampedGatedFFN(nn.Module):
    def __init__(self, width: int, ff: int, limit: float, slope: float = 1.702, bias: bool = True, dtype: torch.dtype = torch.bfloat16,
                 device=None):
        super().__init__()
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.limit, self.slope = float(limit), float(slope)
        self.up = mk(2 * ff, width)                                                  # rows: gate | up
        self.down = mk(width, ff)
        self.up_bias, self.down_bias = (mk(2 * ff), mk(width)) if bias else (None, None)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """``h [N, width]`` → ``[N, width]``."""
        return F.linear(seqmix.clamped_glu(F.linear(h, self.up, self.up_bias), self.limit, self.slope), self.down, self.down_bias)
