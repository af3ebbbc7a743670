"""Latent (compressed key/value) attention with rotary positions on a separate key part and a sliding window.

Per token the layer keeps only a normalised latent ``c`` (``kv_rank`` numbers) and ONE rotated key part shared by all heads
(``rot_dim`` numbers).  Queries go through their own latent.  A head's score against position j is
``(q_unrot . W_uk c_j + q_rot . k_rot_j) * scale``.  Position i sees ``i - window < j <= i``, so the cache is a ring of ``window``
rows per sequence (``csrc/seqmix/latent_attention.cu``).  A prompt that starts a sequence attends over its own prepared rows
and leaves its last ``window`` rows in the ring; later single tokens append to the ring and attend over it.

Two evaluation orders.  Single tokens are bound by reading the ring, so they use the absorbed form ``(W_uk^T q_unrot) . c_j``:
neither keys nor values are expanded, the weighted sum of latents comes back and ``W_uv`` is applied afterwards; one kernel
per ring chunk scores all heads against the chunk's rows and weights the same rows, a second merges the chunks' partial softmaxes
(``csrc/seqmix/latent_decode.cu``; rows wider than the kernel's limit go through matrix products over the gathered ring).  Prompts are
bound by arithmetic, so they expand every head's keys and values once and spend ``dim + rot_dim + vdim`` multiply-adds per
(query, key, head) instead of ``2 kv_rank + rot_dim``: in bfloat16 with sizes in whole 16s as ONE kernel that keeps scores and
weights on chip (``csrc/seqmix/latent_prefill.cu``), otherwise (float, odd sizes) as block matrix products around a float softmax
kernel.  With ``block_products=False`` both run the one-kernel absorbed form.

Options: ``q_rank = 0`` — queries are one direct projection of the input (no query latent); ``head_gate`` — head h's output is
multiplied by ``sigmoid(W_g h)_h``; ``kv_key`` with ``shares_kv`` — the layer has no key/value down-projection and no cache of its
own: it attends over the latents and rotated key parts another layer (same ``kv_rank``, ``rot_dim`` and rotation) prepared in this
step (``ctx.scratch[kv_key]``) and keeps in ITS ring (passed in as ``st``), with its own ``W_uk``, ``W_uv``, queries and window; the
owning layer is built with ``kv_key`` and ``ring_window`` = the widest window among its users.  Rotation pairs are rotate-half; a
checkpoint with interleaved pairs is de-interleaved when it is loaded (``utils.deinterleave_rows``)."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix


class LatentWindowAttention(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, window: int,
                 scale: float, rot_base: float, rot_dims: int, eps: float, dtype: torch.dtype = torch.bfloat16, device=None,
                 max_seq_len: int = 1 << 30, block_products: bool = True, query_block: int = 128, head_gate: bool = False,
                 kv_key=None, shares_kv: bool = False, ring_window: int = 0):
        super().__init__()
        assert not shares_kv or kv_key is not None, "a layer that borrows keys names their owner"
        self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank = heads, dim, rot_dim, vdim, kv_rank, q_rank
        self.window, self.scale, self.rot_dims, self.eps, self.dtype = window, scale, rot_dims, eps, dtype
        self.ring = max(1, min(max(window, ring_window), max_seq_len))
        self.kv_key, self.shares_kv = kv_key, shares_kv
        self.block_products, self.query_block = block_products, query_block
        self.fused_prompt = True          # bfloat16 prompts of fitting sizes in one kernel (csrc/seqmix/latent_prefill.cu)
        self.max_seq_len = max_seq_len
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        f32 = lambda *s: nn.Parameter(torch.ones(*s, dtype=torch.float32, device=device), requires_grad=False)
        if q_rank:
            self.dq, self.dq_norm, self.uq = mk(q_rank, width), f32(q_rank), mk(heads * (dim + rot_dim), q_rank)
        else:
            self.q_proj = mk(heads * (dim + rot_dim), width)
        if not shares_kv:
            self.dkv, self.dkv_norm = mk(kv_rank + rot_dim, width), f32(kv_rank)
        self.head_gate = mk(heads, width) if head_gate else None
        self.uk, self.uv = mk(heads, dim, kv_rank), mk(heads, vdim, kv_rank)          # per head [out, in]
        self.o = mk(width, heads * vdim)
        self.register_buffer("inv_freq", seqmix.rotary_inv_freq(rot_dims, rot_base, device), persistent=False)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        if self.shares_kv:
            return {}
        return {"kv": ((self.ring, self.kv_rank + self.rot_dim), self.dtype)}

    def _gated(self, heads: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """``heads [N, H*vdim]`` times the per-head sigmoid gates read from the layer's input (float logits)."""
        if self.head_gate is None:
            return heads
        return seqmix.sigmoid_gate_mul_(heads, seqmix.linear_f32(h.view(heads.shape[0], -1), self.head_gate))

    def forward(self, h: torch.Tensor, ctx, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        B, S, _ = h.shape
        N, H, D, R = B * S, self.heads, self.dim, self.rot_dim
        if self.q_rank:
            cq = seqmix.rms_norm(F.linear(h.view(N, -1), self.dq), self.dq_norm, self.eps)
            q = F.linear(cq, self.uq).view(B, S, H, D + R)
        else:
            q = F.linear(h, self.q_proj).view(B, S, H, D + R)
        if self.shares_kv:
            rows = ctx.scratch[self.kv_key] if ctx.fresh else None
        else:
            kv = F.linear(h, self.dkv)
            rows = seqmix.latent_kv_store(kv, self.dkv_norm, self.eps, self.inv_freq, self.rot_dims, ctx.pos0, ctx.lens, ctx.slots, st["kv"],
                                          want_rows=ctx.fresh)
            if self.kv_key is not None and ctx.fresh:
                ctx.scratch[self.kv_key] = rows
        seqmix.rope_q_(q, D, self.rot_dims, self.inv_freq, ctx.pos0)
        if ctx.fresh and self.block_products:
            if self.fused_prompt and seqmix.latent_prompt_fused_ok(q, D, R, self.kv_rank + R, self.vdim):
                c = rows[..., :self.kv_rank]
                kx, vx = F.linear(c, self.uk.view(H * D, -1)), F.linear(c, self.uv.view(H * self.vdim, -1))
                heads = seqmix.latent_prompt_attention(q, kx, rows, vx, ctx.lens, D, R, self.vdim, self.window, self.scale)
            else:
                heads = self._attend_prompt(q, rows, ctx)
            return F.linear(self._gated(heads, h), self.o).view(B, S, -1)
        qa = torch.bmm(q.view(N, H, D + R)[:, :, :D].transpose(0, 1), self.uk)                       # [H,N,D] @ [H,D,C]
        if S == 1 and not ctx.fresh and self.kv_rank + R <= seqmix.LATENT_ROW_MAX:
            o = seqmix.latent_window_attention(qa, q, D, st["kv"], ctx.slots, ctx.pos0, ctx.lens, self.window, self.scale)
        elif self.block_products and S == 1:
            o = self._attend_ring(qa, q, ctx, st)
        elif ctx.fresh:
            o = seqmix.latent_window_attention(qa, q, D, rows, None, ctx.pos0, ctx.lens, self.window, self.scale)
        else:
            o = seqmix.latent_window_attention(qa, q, D, st["kv"], ctx.slots, ctx.pos0, ctx.lens, self.window, self.scale)
        ov = torch.bmm(o, self.uv.transpose(1, 2))                                                     # [H,N,C] @ [H,C,V]
        return F.linear(self._gated(ov.transpose(0, 1).reshape(N, H * self.vdim), h), self.o).view(B, S, -1)

    def _attend_prompt(self, q: torch.Tensor, rows: torch.Tensor, ctx) -> torch.Tensor:
        """A prompt in the expanded form: every head's keys ``[W_uk c | rotated part]`` and values ``W_uv c`` are formed by two
        matrix products, which costs ``dim + rot_dim + vdim`` multiply-adds per (query, key, head) instead of the absorbed form's
        ``2 kv_rank + rot_dim``.  Queries, keys and values are laid out ``(sequence, head)``-major with the tokens padded to whole
        blocks of ``query_block``; block ``m`` of that layout multiplies the ``query_block + window - 1`` rows that end with its
        own (rounded up to whole 128-byte score rows), taken as an overlapping strided view, so one batched product covers all sequences, heads and blocks.  Rows of the view
        that belong to the neighbouring head (before a sequence's first token) are positions < 0, which the softmax masks.
        Returns the heads' outputs ``[B*S, H*vdim]``."""
        B, S, H, _ = q.shape
        C, R, D, V = self.kv_rank, self.rot_dim, self.dim, self.vdim
        Qb = min(self.query_block, S)
        nblk = -(-S // Qb)
        Sp, w = nblk * Qb, min(self.window, S)
        pad, M = w - 1, B * H * nblk
        span = -(-(Qb + w - 1) // 32) * 32            # whole 128-byte rows of scores; the extra columns are positions after the query
        tail = span - (Qb + w - 1)
        c = rows[..., :C]
        kbuf, vbuf = rows.new_zeros(pad + B * H * Sp + tail, D + R), rows.new_zeros(pad + B * H * Sp + tail, V)
        kv, vv = kbuf[pad:pad + B * H * Sp].view(B, H, Sp, D + R), vbuf[pad:pad + B * H * Sp].view(B, H, Sp, V)
        kv[:, :, :S, :D] = F.linear(c, self.uk.view(H * D, C)).view(B, S, H, D).permute(0, 2, 1, 3)
        kv[:, :, :S, D:] = rows[:, None, :, C:]
        vv[:, :, :S] = F.linear(c, self.uv.view(H * V, C)).view(B, S, H, V).permute(0, 2, 1, 3)
        qbuf = q.new_zeros(B, H, Sp, D + R) if Sp != S else q.new_empty(B, H, Sp, D + R)
        qbuf[:, :, :S] = q.permute(0, 2, 1, 3)
        qm = qbuf.view(M, Qb, D + R)
        kwin = kbuf.as_strided((M, span, D + R), (Qb * (D + R), D + R, 1))
        vwin = vbuf.as_strided((M, span, V), (Qb * V, V, 1))
        pos0, lens = ctx.pos0.repeat_interleave(H), ctx.lens.repeat_interleave(H)
        out = q.new_empty(M, Qb, V)
        group = max(1, (1 << 28) // (nblk * Qb * span))                      # (sequence, head) pairs per pass: scores stay <= 1 GiB
        for g0 in range(0, B * H, group):
            g1 = min(B * H, g0 + group)
            m0, m1 = g0 * nblk, g1 * nblk
            sc = seqmix.matmul_f32(qm[m0:m1], kwin[m0:m1].transpose(1, 2)).view(g1 - g0, nblk, Qb, span)
            p = seqmix.window_softmax(sc, self.scale, False, 1, Qb, nblk, w, self.window, pos0[g0:g1], lens[g0:g1], q.dtype)
            torch.bmm(p.view(m1 - m0, Qb, span), vwin[m0:m1], out=out[m0:m1])
        return out.view(B, H, Sp, V)[:, :, :S].permute(0, 2, 1, 3).reshape(B * S, H * V)

    def _attend_ring(self, qa: torch.Tensor, q: torch.Tensor, ctx, st) -> torch.Tensor:
        """Single tokens against their sequences' rings, in the absorbed form, as matrix products with the heads folded into the
        row dimension (all heads share the keys); the softmax over the visible ring rows runs in float in between.  ``[H, B, C]``."""
        B, S, H, _ = q.shape
        C, R, D = self.kv_rank, self.rot_dim, self.dim
        qcat = torch.cat([qa.view(H, B, S, C).permute(1, 2, 0, 3), q[..., D:]], -1)                   # [B,1,H,C+R]
        kc = st["kv"].index_select(0, ctx.slots.long())                                                # [B,ring,C+R]
        sc = seqmix.matmul_f32(qcat.view(B, H, C + R), kc.transpose(1, 2))                             # [B,H,ring]
        p = seqmix.window_softmax(sc, self.scale, True, H, 1, 1, 1, self.window, ctx.pos0, ctx.lens, q.dtype)
        return torch.bmm(p, kc[..., :C]).transpose(0, 1).contiguous()                                  # [H,B,C]
