"""Minimal gated recurrent unit as a sequence mixer (minGRU: Feng et al., "Were RNNs All We Needed?"): the gates read only the
current token, never the state, so a prompt is one matrix product followed by a scan over time.  Per channel of ``rwidth``:
``z = sigmoid(W_z h + b_z)``, ``u = W_x h + b_x``, candidate ``c = u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` below (a positive,
continuous activation), ``s_t = (1 - z) s_(t-1) + z c`` and the block returns ``W_o (s_t * silu(W_g h))``.  The gate, the
candidate and the state are float; the state starts at zero and is carried per sequence (``csrc/seqmix/linear_recurrence.cu``).

``z``, ``u`` and the output gate are ONE stacked projection of the input.  ``extra_rows`` more rows can ride on it for the
caller (a block that gates its residual from the same input): ``forward`` then returns ``(output, extra [B,S,extra_rows])``."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class MinGRU(nn.Module):
    def __init__(self, width: int, rwidth: int, dtype: torch.dtype = torch.bfloat16, device=None, extra_rows: int = 0):
        super().__init__()
        self.rwidth, self.extra_rows, self.dtype = rwidth, extra_rows, dtype
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.in_proj, self.in_bias = mk(3 * rwidth + extra_rows, width), mk(3 * rwidth + extra_rows)      # rows: z | u | gate | extra
        self.o = mk(width, rwidth)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"rec": ((self.rwidth,), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]):
        W = self.rwidth
        p = F.linear(h, self.in_proj, self.in_bias)
        mixed = seqmix.mingru_scan(p[..., :W], p[..., W:2 * W], p[..., 2 * W:3 * W], st["rec"], ctx.slots, ctx.lens, ctx.fresh)
        y = F.linear(mixed, self.o)
        return (y, p[..., 3 * W:]) if self.extra_rows else y
