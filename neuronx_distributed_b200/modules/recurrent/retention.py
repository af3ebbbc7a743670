"""Retention: linear attention with ONE fixed decay per head and no softmax or denominator (Sun et al., "Retentive Network: A
Successor to Transformer for Large Language Models").  Per head a float matrix state ``S [dim, vdim]``:
``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``.  Queries and keys are rotated by their position (rotate-half pairs on
the first ``rot_dims`` coordinates of each head) and the keys scaled by ``dim^-1/2``, both in float: everything that enters the
recurrence after the projections is float.  Each head's read-out is divided by its root mean square (no gain), multiplied by
``silu(W_g h)`` and projected out.  q, k, v and the gate are one stacked projection; state per sequence: the float matrix."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class Retention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], rot_base: float, rot_dims: int,
                 eps: float = 1e-6, dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        assert len(decay) == heads, "one decay per head"
        assert rot_dims % 2 == 0 and rot_dims <= dim, "the rotated coordinates are pairs inside a head"
        self.heads, self.dim, self.vdim, self.rot_dims, self.eps, self.dtype = heads, dim, vdim, rot_dims, eps, dtype
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.in_proj = mk(2 * heads * dim + 2 * heads * vdim, width)                 # rows: q | k | v | gate
        self.o = mk(width, heads * vdim)
        self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=torch.float32, device=device), persistent=False)
        self.register_buffer("unit", torch.ones(vdim, dtype=torch.float32, device=device), persistent=False)
        self.register_buffer("inv_freq", seqmix.rotary_inv_freq(rot_dims, rot_base, device), persistent=False)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"rec": ((self.heads, self.dim, self.vdim), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        N, H, D, V = B * S, self.heads, self.dim, self.vdim
        p = F.linear(h, self.in_proj)
        nq, nv = H * D, H * V
        f = seqmix.rotary_qkv_f32(p[..., :2 * nq + nv], H, H, D, self.rot_dims, self.inv_freq, ctx.pos0, 1.0, D ** -0.5)
        q, k, v = f[..., :nq].unflatten(-1, (H, D)), f[..., nq:2 * nq].unflatten(-1, (H, D)), f[..., 2 * nq:].unflatten(-1, (H, V))
        o = seqmix.retention_scan(q, k, v, self.decay, st["rec"], ctx.slots, ctx.lens, ctx.fresh)             # float [B,S,H,V]
        on = seqmix.group_rms_norm_gated(o.view(N, nv), p.view(N, -1)[:, 2 * nq + nv:], self.unit, H, self.eps, False, out_dtype=h.dtype)
        return F.linear(on, self.o).view(B, S, -1)
