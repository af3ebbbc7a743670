"""Gated delta rule: per head a matrix memory ``M [dim, vdim]`` that decays by one data-dependent factor per head and token, then
overwrites what it holds at the current key with the current value, ``M <- g M;  u = beta (v - M^T k);  M <- M + k u^T``, and is
read with the query AFTER the write, ``o = M^T q`` (Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta
Rule").  q and k (``kv_heads`` of them, shared by groups of value heads) and v pass short causal convolutions and silu, q and k
are made unit vectors in float; ``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` are float.  Each
head's read-out is RMS-normed over ``vdim`` (one weight vector shared by the heads) and gated by ``silu(W_g h)``.

q, k, v and the gate are one stacked projection (and ONE convolution over the q|k|v channels); the two per-head scalars come
from a second, float-accumulated product.  State per sequence: the convolution history and the float memory.

Options: ``channel_decay`` — one decay per head AND key channel, ``g [heads, dim]`` scaling the rows of M (``dt_bias`` then holds
``heads * dim`` numbers, ``a_log`` stays per head); ``decay_rank`` / ``gate_rank`` > 0 — the decay pre-activations / the gate logits
come through a low-rank pair ``W_2 (W_1 h)`` whose first factor rides in the stacked projection; ``gate_act`` — ``silu`` or
``sigmoid`` on the output gate."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from ..short_conv import ShortConv


class GatedDeltaRule(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float = 1e-6,
                 dtype: torch.dtype = torch.bfloat16, device=None, channel_decay: bool = False, decay_rank: int = 0, gate_rank: int = 0,
                 gate_act: str = "silu"):
        super().__init__()
        assert heads % kv_heads == 0, "value heads must divide into the query/key heads"
        assert gate_act in ("silu", "sigmoid") and (decay_rank == 0 or channel_decay), "a low-rank decay is a decay per channel"
        self.heads, self.kv_heads, self.dim, self.vdim, self.eps, self.dtype = heads, kv_heads, dim, vdim, eps, dtype
        self.channel_decay, self.decay_rank, self.gate_rank, self.gate_act = channel_decay, int(decay_rank), int(gate_rank), gate_act
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.zeros(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.n_qk, self.n_v = kv_heads * dim, heads * vdim
        n_decay = heads * dim if channel_decay else heads
        self.n_gate = self.gate_rank or self.n_v
        # rows: q | k | v | gate (or its low-rank factor) | the decay's low-rank factor
        self.in_proj = mk(2 * self.n_qk + self.n_v + self.n_gate + self.decay_rank, width)
        self.ba_proj = mk(heads + (0 if self.decay_rank else n_decay), width)        # rows: beta logits | decay pre-activations
        if self.gate_rank:
            self.gate_up = mk(self.n_v, self.gate_rank)
        if self.decay_rank:
            self.decay_up = mk(n_decay, self.decay_rank)
        self.conv = ShortConv(2 * self.n_qk + self.n_v, taps, bias=False, residual=False, device=device)
        self.a_log, self.dt_bias = f32(heads), f32(n_decay)
        self.norm = f32(vdim)
        self.o = mk(width, heads * vdim)

    @property
    def out_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"conv": self.conv.state_spec(self.dtype), "rec": ((self.heads, self.dim, self.vdim), torch.float32)}

    def mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        """``h [B,S,width]`` → the normed, gated heads times ``out_scale`` in ``out [B*S, heads*vdim]`` (any row stride)."""
        B, S, W = h.shape
        N, H, G, D, V = B * S, self.heads, self.kv_heads, self.dim, self.vdim
        p = F.linear(h, self.in_proj)
        nc = 2 * self.n_qk + self.n_v
        c = self.conv(p[..., :nc], st["conv"], ctx, h.dtype, silu=True)              # [B,S,q|k|v]
        q, k = c[..., :self.n_qk].unflatten(-1, (G, D)), c[..., self.n_qk:2 * self.n_qk].unflatten(-1, (G, D))
        v = c[..., 2 * self.n_qk:].unflatten(-1, (H, V))
        ba = seqmix.linear_f32(h.view(N, W), self.ba_proj).view(B, S, -1)
        p2 = p.view(N, -1)
        if self.decay_rank:
            r0 = nc + self.n_gate
            araw = seqmix.linear_f32(p2[:, r0:r0 + self.decay_rank], self.decay_up).view(B, S, -1)
        else:
            araw = ba[..., H:]
        if self.channel_decay:
            araw = araw.unflatten(-1, (H, D))
        o = seqmix.gated_delta_scan(q, k, v, ba[..., :H], araw, self.a_log, self.dt_bias, st["rec"], ctx.slots, ctx.lens, ctx.fresh)
        gate = F.linear(p2[:, nc:nc + self.gate_rank], self.gate_up) if self.gate_rank else p2[:, nc:nc + self.n_v]
        return seqmix.group_rms_norm_gated(o.view(N, H * V), gate, self.norm, H, self.eps, False, out, out_scale, gate_act=self.gate_act)

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        heads = torch.empty(B * S, self.out_features, dtype=h.dtype, device=h.device)
        return F.linear(self.mix(h, ctx, st, heads), self.o).view(B, S, -1)
