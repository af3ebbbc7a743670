"""Grouped-query softmax attention whose heads talk to each other before the softmax, over aligned chunks of positions and / or a
sliding window, with keys that double as values (``csrc/seqmix/headmix_attention.cu``, ``headmix_prefill.cu``).

Queries and keys are projections of the input followed by a short causal convolution per channel (its last ``taps - 1`` inputs are
state); the VALUES are the convolved keys before rotation, so there is no value projection and ``vdim = dim``.  Queries and keys
are rotated by position on their first ``rot_dims`` coordinates (rotate-half pairs, in float).  The score of head g for a (query,
key) pair is ``q_g . k * scale * temp[g]``; the heads' scores of the pair are then mixed, ``score_h = sum_g talk[h,g] score_g``
(Shazeer et al., "Talking-Heads Attention", the mixing before the softmax).  Position i sees ``j <= i`` with ``floor(i / chunk) =
floor(j / chunk)`` (chunks count from the sequence's first position) and / or ``i - j < window``.  The softmax's denominator also
holds ``exp(sink[h])``, a learned number per head with no key and no value.  The concatenated heads are multiplied coordinate by
coordinate with ``sigmoid(W_g h)`` and projected out.  ``temp``, ``talk`` and ``sink`` are optional.

State per sequence: the convolution history of q|k and a ring of ``min(chunk, window)`` rotated key rows and value rows (position
j sits in row ``j mod ring``; a chunk's first token overwrites the row of the previous chunk's first token, which it no longer sees).
q, k and the gate are one stacked projection and ONE convolution runs over the q|k channels.  The mixing is linear in the queries, so
the kernels move it onto them: head h's mixed query against key head c is ``Q'[h,c,:] = sum_{g in group c} talk[h,g] scale temp[g] q_g``
and its score is one dot product of ``Q'[h]`` with the position's keys of all key heads side by side; after that the attention is an
ordinary one with key size ``kv_heads * dim``.  ``mix`` writes the gated heads into
a caller's buffer; ``forward`` is the stand-alone layer."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from ..short_conv import ShortConv


class HeadMixAttention(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, taps: int, scale: float, rot_base: float, rot_dims: int,
                 chunk: int = 0, window: int = 0, talk: bool = True, temp: bool = True, sink: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device=None, max_seq_len: int = 1 << 30):
        super().__init__()
        assert heads % kv_heads == 0, "query heads must divide into the key/value heads"
        assert rot_dims % 2 == 0 and rot_dims <= dim, "the rotated coordinates are pairs inside a head"
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, dim
        self.chunk, self.window, self.scale, self.rot_dims, self.dtype = int(chunk), int(window), float(scale), rot_dims, dtype
        spans = [s for s in (self.chunk, self.window) if s > 0]
        self.ring = max(1, min(spans + [max_seq_len]))
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.n_q, self.n_k = heads * dim, kv_heads * dim
        self.in_proj = mk(self.n_q + self.n_k + heads * dim, width)                  # rows: q | k | gate
        self.conv = ShortConv(self.n_q + self.n_k, max(1, taps), bias=False, residual=False, device=device)
        self.temp = nn.Parameter(torch.ones(heads, dtype=torch.float32, device=device), requires_grad=False) if temp else None
        self.talk = nn.Parameter(torch.eye(heads, dtype=torch.float32, device=device), requires_grad=False) if talk else None
        self.sink = nn.Parameter(torch.zeros(heads, dtype=torch.float32, device=device), requires_grad=False) if sink else None
        self.o = mk(width, heads * dim)
        self.register_buffer("inv_freq", seqmix.rotary_inv_freq(rot_dims, rot_base, device), persistent=False)
        self.register_buffer("unit", torch.ones(heads, dtype=torch.float32, device=device), persistent=False)
        self._coef = None

    @property
    def out_features(self) -> int:
        return self.heads * self.dim

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {"conv": self.conv.state_spec(self.dtype), "k": ((self.ring, self.kv_heads, self.dim), self.dtype),
                "v": ((self.ring, self.kv_heads, self.dim), self.dtype)}

    def _mix_weights(self) -> torch.Tensor:
        """``talk[h,g] * scale * temp[g]`` (float ``[H,H]``), formed once per set of weights."""
        key = tuple((p.data_ptr(), p._version) for p in (self.temp, self.talk) if p is not None)
        if self._coef is None or self._coef[0] != key:
            coef = (self.unit if self.temp is None else self.temp.detach()) * self.scale
            talk = torch.eye(self.heads, dtype=torch.float32, device=coef.device) if self.talk is None else self.talk.detach()
            self._coef = (key, (talk * coef[None, :]).contiguous())
        return self._coef[1]

    def mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        """``h [B,S,width]`` → the gated heads in ``out [B*S, heads*dim]`` (a view with any row stride)."""
        B, S, _ = h.shape
        if not ctx.fresh and S != 1:
            raise ValueError("attention continues a sequence one token at a time")
        H, G, D = self.heads, self.kv_heads, self.dim
        p = F.linear(h, self.in_proj)
        nqk = self.n_q + self.n_k
        c = self.conv(p[..., :nqk], st["conv"], ctx, h.dtype)                        # [B,S,q|k]
        q = c[..., :self.n_q].unflatten(-1, (H, D))
        k = c[..., self.n_q:].unflatten(-1, (G, D))
        qmix, rows = seqmix.headmix_qk_prepare(q, k, self._mix_weights(), self.rot_dims, self.inv_freq, ctx.pos0, ctx.lens, ctx.slots,
                                               st["k"], st["v"], want_rows=ctx.fresh)
        gate = p[..., nqk:]
        if ctx.fresh:
            return seqmix.headmix_attention_prompt(qmix, rows, k, self.sink, gate, ctx.lens, self.chunk, self.window, out)
        return seqmix.headmix_attention_token(qmix, st["k"], st["v"], self.sink, gate, ctx.slots, ctx.pos0, ctx.lens, self.chunk,
                                              self.window, out)

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        heads = torch.empty(B * S, self.out_features, dtype=h.dtype, device=h.device)
        return F.linear(self.mix(h, ctx, st, heads), self.o).view(B, S, -1)
