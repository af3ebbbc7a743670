"""Grouped-query attention over a sliding window: biased or plain q/k/v projections, an RMS norm on queries and keys, scores
``q.k * scale`` optionally capped as ``softcap * tanh(score / softcap)``, and optionally one sigmoid output gate per head read from
the layer's input.  Position i sees ``i - window < j <= i``, so each sequence keeps a ring of ``window`` key and value rows
(``csrc/seqmix/window_attention.cu``).

Options.  ``qk_norm``: ``"head"`` — every head is normed by itself with one weight vector of ``dim`` numbers shared by the heads;
``"all"`` — one root mean square over the whole query (key) projection, weights of ``heads * dim`` (``kv_heads * dim``) numbers;
``None``.  ``rot_dims > 0``: after the norm the first ``rot_dims`` coordinates of every query and key head are rotated at the
token's position (pairs ``i, i + rot_dims/2``; a checkpoint that pairs neighbours is de-interleaved when it is loaded,
``utils.deinterleave_rows``), frequencies ``rot_base^(-2i/rot_dims)`` optionally rescaled for a longer context (``rot_scaling``).
``weights``: ``"softmax"`` over the visible keys, or ``"sigmoid"`` — every visible key weighs ``sigmoid(score + score_bias[h])`` by
itself, with one learned bias per query head and no normalisation over the keys.  ``kv_key`` with ``shares_kv``: the layer has no key
/ value projections and no cache of its own; it attends with its own queries, window and biases over the prepared keys and the
values another layer (same head counts and rotation) made in this step (``ctx.scratch[kv_key]``) and keeps in ITS ring (passed in
as ``st``); the owning layer is built with ``kv_key`` and ``ring_window`` = the widest window among its users.  ``extra_rows`` more
rows can ride on the stacked projection for the caller: ``forward`` then returns ``(output, extra [B,S,extra_rows])``.

q, k, v, the gate logits and the extra rows are one stacked projection of the input; the norm, the ring store and the attention
read their parts of it in place through strides.  ``mix`` writes the gated heads (times a caller's scale) into a caller's buffer
so that a layer that sums several mixers can run ONE output projection over all of them; ``forward`` is the stand-alone layer."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class GatedWindowAttention(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, window: int, scale: float, softcap: float = 0.0,
                 eps: float = 1e-6, qk_norm=True, head_gate: bool = True, dtype: torch.dtype = torch.bfloat16, device=None,
                 max_seq_len: int = 1 << 30, bias: bool = True, weights: str = "softmax", rot_dims: int = 0, rot_base: float = 10000.0,
                 rot_scaling: Optional[dict] = None, kv_key=None, shares_kv: bool = False, ring_window: int = 0, extra_rows: int = 0):
        super().__init__()
        assert heads % kv_heads == 0, "query heads must divide into the key/value heads"
        assert weights in ("softmax", "sigmoid"), weights
        assert not shares_kv or kv_key is not None, "a layer that borrows keys names their owner"
        qk_norm = {True: "head", False: None}.get(qk_norm, qk_norm)
        assert qk_norm in ("head", "all", None), qk_norm
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.window, self.scale, self.softcap, self.eps, self.dtype = int(window), float(scale), float(softcap), eps, dtype
        self.ring = max(1, min(max(self.window, int(ring_window)), max_seq_len))
        self.head_gate, self.qk_norm, self.rot_dims = head_gate, qk_norm, int(rot_dims)
        self.kv_key, self.shares_kv, self.extra_rows = kv_key, shares_kv, int(extra_rows)
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.ones(*s, dtype=torch.float32, device=device), requires_grad=False)
        self.n_q = heads * dim
        self.n_k, self.n_v = (0, 0) if shares_kv else (kv_heads * dim, kv_heads * vdim)
        rows = self.stacked_rows(heads, 0 if shares_kv else kv_heads, dim, vdim, head_gate, extra_rows)
        self.in_proj = mk(rows, width)                                               # rows: q | k | v | gate | extra | zero padding
        self.in_bias = mk(rows) if bias else None
        per = {"head": (dim, dim), "all": (heads * dim, kv_heads * dim), None: (0, 0)}[qk_norm]
        self.q_norm = f32(per[0]) if qk_norm else None
        self.k_norm = f32(per[1]) if qk_norm and not shares_kv else None
        self.score_bias = nn.Parameter(torch.zeros(heads, dtype=torch.float32, device=device), requires_grad=False) if weights == "sigmoid" else None
        if self.rot_dims:
            self.register_buffer("inv_freq", seqmix.rotary_inv_freq(self.rot_dims, rot_base, device, rot_scaling), persistent=False)
        else:
            self.inv_freq = None
        self.o = mk(width, heads * vdim)

    @staticmethod
    def stacked_rows(heads: int, kv_heads: int, dim: int, vdim: int, head_gate: bool = True, extra_rows: int = 0) -> int:
        """Rows of the stacked projection: q | k | v | gate | extra, padded to a whole 8 so that token rows stay 16-byte aligned in
        bfloat16 (the fused prompt kernel reads q, k and v in place)."""
        n = heads * dim + kv_heads * (dim + vdim) + (heads if head_gate else 0) + extra_rows
        return -(-n // 8) * 8

    @property
    def out_features(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        if self.shares_kv:
            return {}
        return {"k": ((self.ring, self.kv_heads, self.dim), self.dtype), "v": ((self.ring, self.kv_heads, self.vdim), self.dtype)}

    def _mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor, out_scale: float):
        B, S, _ = h.shape
        if not ctx.fresh and S != 1:
            raise ValueError("window attention continues a sequence one token at a time")
        H, G, D, V = self.heads, self.kv_heads, self.dim, self.vdim
        p = F.linear(h, self.in_proj, self.in_bias)
        a, b, c = self.n_q, self.n_q + self.n_k, self.n_q + self.n_k + self.n_v
        q = p[..., :a].unflatten(-1, (H, D))
        gate = p[..., c:c + H] if self.head_gate else None
        e0 = c + (H if self.head_gate else 0)
        extra = p[..., e0:e0 + self.extra_rows] if self.extra_rows else None
        rot = dict(norm_all=self.qk_norm == "all", inv_freq=self.inv_freq, rot_dims=self.rot_dims)
        if self.shares_kv:
            seqmix.window_qk_prepare(q, None, None, self.q_norm, None, self.eps, ctx.pos0, ctx.lens, ctx.slots, None, None, **rot)
            k, v = ctx.scratch[self.kv_key] if ctx.fresh else (None, None)
        else:
            k, v = p[..., a:b].unflatten(-1, (G, D)), p[..., b:c].unflatten(-1, (G, V))
            seqmix.window_qk_prepare(q, k, v, self.q_norm, self.k_norm, self.eps, ctx.pos0, ctx.lens, ctx.slots, st["k"], st["v"], **rot)
            if self.kv_key is not None and ctx.fresh:
                ctx.scratch[self.kv_key] = (k, v)
        if ctx.fresh:
            seqmix.window_attention_prompt(q, k, v, gate, ctx.lens, self.window, self.scale, self.softcap, out, out_scale, self.score_bias)
        else:
            seqmix.window_attention_token(q, st["k"], st["v"], gate, ctx.slots, ctx.pos0, ctx.lens, self.window, self.scale, self.softcap,
                                          out, out_scale, self.score_bias)
        return out, extra

    def mix(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor], out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
        """``h [B,S,width]`` → the gated heads times ``out_scale`` in ``out [B*S, heads*vdim]`` (a view with any row stride)."""
        return self._mix(h, ctx, st, out, out_scale)[0]

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]):
        B, S, _ = h.shape
        heads = torch.empty(B * S, self.out_features, dtype=h.dtype, device=h.device)
        heads, extra = self._mix(h, ctx, st, heads, 1.0)
        y = F.linear(heads, self.o).view(B, S, -1)
        return (y, extra) if self.extra_rows else y
