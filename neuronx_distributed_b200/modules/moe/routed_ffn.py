"""Routed feed-forward with independent (non-renormalised) expert weights, for serving: scores ``s = act(W_router h)`` in float
(the framework's ``RouterTopK``; sigmoid or softmax), the ``top`` largest are chosen, the output is
``sum_e s_e * scale * expert_e(h)`` plus an always-on shared expert.  Experts have no biases and are kept as stacks: plain,
``W_down gelu(W_up h)`` with ``up [E, ff, width]``, or gated, ``W_down (silu(W_gate h) * (W_up h))`` with the gate rows stacked
over the up rows in ``up [E, 2 ff, width]``; ``down [E, width, ff]``.

``router_act="softmax_top"``: the ``top`` largest LOGITS are chosen and the weights are the softmax over the chosen logits only
(renormalised by construction).  ``router_bias``: the logits are ``W_router h + b``.  ``expert_act``: the plain experts' activation,
``"gelu"`` (erf form) or ``"relu_sq"`` (the square of relu).

Two more options of the router.  ``choice_bias``: a float vector added to the scores for the CHOICE only (the weights stay the plain
scores).  ``identity_experts``: the router's last outputs name experts without tensors whose output is the input itself; their
weights are summed per token and enter the combine as a weighted copy of the input.

Two execution shapes, both summing the chosen experts in float (``moe_combine``):
* few rows (token generation): the chosen experts' matrices are streamed once by ``indexed_gemv`` — no host synchronisation;
* many rows (prompts), bfloat16 with sizes the tensor-core kernel takes: the framework's blockwise layout (``blockwise.py``: rows
  grouped by expert into blocks of 128, one index-build launch) and its grouped tcgen05 GEMM, two launches for all experts;
* many rows otherwise (float, odd sizes, extension not built): rows are sorted by expert and every non-empty expert runs two
  dense matrix products."""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import seqmix
from .routing import RouterTopK


class RoutedFFN(nn.Module):
    small_batch_rows = 64          # up to this many (row, expert) pairs the streaming path is used

    def __init__(self, width: int, ff: int, experts: int, top: int, weight_scale: float = 1.0, shared_ff: int = 0,
                 router_act: str = "sigmoid", gated: bool = False, identity_experts: int = 0, choice_bias: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device=None, router_bias: bool = False, expert_act: str = "gelu"):
        super().__init__()
        assert expert_act in ("gelu", "relu_sq"), expert_act
        assert router_act != "softmax_top" or not (identity_experts or choice_bias), "softmax over the chosen logits: plain experts only"
        self.expert_act = expert_act
        self.width, self.ff, self.experts, self.top, self.weight_scale, self.shared_ff = width, ff, experts, top, weight_scale, shared_ff
        self.gated, self.identity_experts = gated, identity_experts
        self.router = RouterTopK(experts + identity_experts, top, width, dtype=torch.float32, device=device, bias=router_bias,
                                 act_fn="softmax" if router_act == "softmax_top" else router_act,
                                 apply_act_fn_over_topk=router_act == "softmax_top")
        self.router_act = router_act
        self.router.requires_grad_(False)
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=device), requires_grad=False)
        self.up, self.down = mk(experts, (2 if gated else 1) * ff, width), mk(experts, width, ff)
        self.correction = nn.Parameter(torch.zeros(experts + identity_experts, dtype=torch.float32, device=device),
                                       requires_grad=False) if choice_bias else None
        if shared_ff:
            self.shared_up, self.shared_down = mk(shared_ff, width), mk(width, shared_ff)
        self._router_lowp = None       # (version of the router matrix, its bfloat16 transpose or None when that would round)

    def _router_logits(self, h: torch.Tensor) -> torch.Tensor:
        """Float logits.  When the activations are bfloat16 and the (float) router matrix holds only numbers that bfloat16 represents
        exactly — a checkpoint stored in bfloat16 — the product runs on the bfloat16 operands with float accumulation: the same
        products and a float sum, on the tensor cores.  Otherwise the framework router's float product."""
        z = self._router_products(h)
        b = self.router.linear_router.bias
        return z if b is None else z + b

    def _router_products(self, h: torch.Tensor) -> torch.Tensor:
        w = self.router.linear_router.weight
        if h.is_cuda and h.shape[0] <= seqmix.SMALL_LINEAR_ROWS:
            return seqmix.linear_f32(h, w)                         # a warp per (row, expert): float products of the stored numbers
        if h.dtype != torch.bfloat16 or not h.is_cuda:
            return F.linear(h.float(), w)
        if self._router_lowp is None or self._router_lowp[0] != w._version:
            low = w.detach().to(torch.bfloat16)
            self._router_lowp = (w._version, low.t().contiguous() if bool((low.float() == w).all()) else None)
        if self._router_lowp[1] is None:
            return F.linear(h.float(), w)
        return seqmix.matmul_f32(h[None], self._router_lowp[1][None])[0]

    def route(self, h: torch.Tensor):
        """Float scores of all experts → (weights ``[N, top]`` float, expert ids ``[N, top]``, identity share ``[N]`` float or None):
        one kernel for scores, correction, top-k and the identity experts' share (``seqmix.route_topk``)."""
        w, idx, ident = seqmix.route_topk(self._router_logits(h), self.correction, self.top, self.experts, self.router_act,
                                          self.weight_scale)
        return w, idx, (ident if self.identity_experts else None)

    def _act(self, y: torch.Tensor) -> torch.Tensor:
        """The experts' activation on the up-projection's output: ``[M, ff]`` (plain) or ``[M, 2 ff]`` → ``[M, ff]`` (gated)."""
        if self.gated:
            return seqmix.silu_mul(y)
        return seqmix.relu_sq(y) if self.expert_act == "relu_sq" else seqmix.gelu_erf(y)

    block_rows = 128               # rows per block of the grouped GEMM

    def _grouped_kernels(self, h: torch.Tensor):
        """The main extension when its grouped GEMM can take this call (bfloat16 on the GPU, sizes in whole 64s), else None."""
        if not (h.is_cuda and h.dtype == torch.bfloat16 and self.width % 64 == 0 and self.ff % 64 == 0):
            return None
        from ...ops import _ext

        e = _ext.ext()
        return e if e is not None and hasattr(e, "grouped_gemm") else None

    def _experts_grouped(self, h: torch.Tensor, idx: torch.Tensor):
        """All chosen experts in two grouped GEMMs over the blockwise layout → (rows ``[blocks * 128, width]``, ``src [N, top]``
        naming the row that holds each (token, choice)).  Padding slots compute on token 0 and are never referenced."""
        from ...ops import _ext
        from .blockwise import build_block_metadata

        e, bs = _ext.ext(), self.block_rows
        ident = None
        if self.identity_experts:                      # identity choices form one more group; its blocks run some expert's matrices
            ident = idx >= self.experts                # (finite rows that the combine weighs with zero)
            idx = torch.where(ident, torch.full_like(idx, self.experts), idx)
        b2e, tp2id, _ = build_block_metadata(idx, self.experts + (1 if self.identity_experts else 0), bs)
        group = b2e.long()                                                         # the group of every block, the extra one included
        b2e = b2e.to(torch.int32).clamp(max=self.experts - 1).contiguous()
        tp = tp2id[: b2e.numel() * bs].long()
        x = h[tp.clamp(min=0)]
        _ext.count_launch(2)
        eo = e.grouped_gemm(self._act(e.grouped_gemm(x, self.up, b2e, bs, True)), self.down, b2e, bs, True)
        N, top = idx.shape                                                         # no host synchronisation: padding slots write
        tok, exp = tp.clamp(min=0), group.repeat_interleave(bs)                    # to a spare entry past the end
        choice = (idx[tok] == exp[:, None]).to(torch.int32).argmax(1)
        flat = torch.empty(N * top + 1, dtype=torch.int32, device=h.device)
        flat[torch.where(tp >= 0, tok * top + choice, N * top)] = torch.arange(tp.numel(), dtype=torch.int32, device=h.device)
        src = flat[: N * top].view(N, top)
        if ident is not None:
            src = torch.where(ident, torch.zeros_like(src), src)                   # any row: its weight is zero
        return eo, src

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """``h [N, width]`` → ``[N, width]``."""
        N = h.shape[0]
        w, idx, ident_w = self.route(h)                            # identity choices: weight 0, their scores summed in ident_w
        M = N * self.top
        if M <= self.small_batch_rows:
            sel = idx.reshape(-1).to(torch.int32)                  # the streaming kernels skip rows that name no matrix
            mid = seqmix.indexed_gemv(self.up, sel, h.repeat_interleave(self.top, 0), "silu_glu" if self.gated else self.expert_act)
            eo = seqmix.indexed_gemv(self.down, sel, mid, None)
            src = torch.arange(M, device=h.device, dtype=torch.int32).view(N, self.top)
        elif self._grouped_kernels(h) is not None:
            eo, src = self._experts_grouped(h, idx)
        else:
            flat = idx.reshape(-1)
            order = torch.argsort(flat, stable=True)
            counts = torch.bincount(flat, minlength=self.experts + self.identity_experts).tolist()[:self.experts]
            xs = h[order // self.top]
            eo = torch.zeros(M, self.width, dtype=h.dtype, device=h.device) if self.identity_experts else \
                torch.empty(M, self.width, dtype=h.dtype, device=h.device)
            off = 0
            for e, c in enumerate(counts):
                if c:
                    eo[off:off + c] = F.linear(self._act(F.linear(xs[off:off + c], self.up[e])), self.down[e])
                    off += c
            src = torch.empty(M, dtype=torch.int32, device=h.device)
            src[order] = torch.arange(M, device=h.device, dtype=torch.int32)
            src = src.view(N, self.top)
        if self.identity_experts:
            if self.shared_ff:
                raise NotImplementedError("identity experts together with a shared expert")
            return seqmix.moe_combine(eo, src, w.contiguous(), h, ident_w)
        base = F.linear(seqmix.gelu_erf(F.linear(h, self.shared_up)), self.shared_down) if self.shared_ff else None
        return seqmix.moe_combine(eo, src, w.contiguous(), base)
