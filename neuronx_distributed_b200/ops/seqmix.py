"""Sequence-mixer ops: short causal convolutions with carried history, scalar / vector RMS norms (optionally accumulated into a
float residual stream, or closing a block whose norm follows a gated residual sum), token embeddings with sinusoids or a hashed
pair table, latent / grouped-query / head-mixing sliding-window attention over ring caches (softmax or independent sigmoid weights),
gated linear recurrences (per-key-channel decay; real-gated LRU; minGRU), matrix-state recurrences, xIELU / erf-GELU / squared relu
and the small-batch pieces of a routed feed-forward.

CUDA tensors run the hand-written kernels of ``csrc/seqmix`` (one small extension per kernel group, built in-tree on first use so
that a fresh checkout compiles only the files of the mechanisms its model has); CPU tensors run the plain PyTorch statements below, which define the semantics.
Conventions: activations are ``[B, S, ...]`` right-padded batches with ``lens [B]`` (int32) real tokens per row; ``slots [B]``
(int32) names each row's block in a state tensor; ``fresh`` means the rows start a sequence in this call (history / state = 0).
Everything the kernels keep in float (statistics, scores, decays, states) is float here as well."""
from __future__ import annotations

import importlib.machinery
import importlib.util
import math
import os
import sys
from pathlib import Path
from typing import Optional

import torch
import torch.nn.functional as F

from . import _ext

SEQ_BUILD_DIR = _ext.BUILD_DIR / "seqmix"
CSRC = _ext.PKG_DIR.parent / "csrc" / "seqmix"

# Kernel groups, each its own extension ``nxd_b200_seq_<group>_C`` built in-tree on first use, so that a model compiles only the
# mechanisms it has: group → (sources, functions it exports).
GROUPS = {
    "core": (["short_conv.cu", "norms.cu", "activations.cu", "embed.cu", "rotary.cu", "bind_core.cpp"],
             ["short_conv", "rms_norm", "add_rms_norm_", "xielu", "gelu_erf", "silu_mul", "indexed_gemv", "moe_combine", "embed_sinusoid",
              "group_rms_norm_gated", "route_topk", "small_linear_f32", "clamped_glu", "sigmoid_gate_mul_", "rotary_qkv_f32", "relu_sq",
              "embed_bigram", "postnorm_gated_"]),
    "latent": (["latent_attention.cu", "latent_decode.cu", "latent_prefill.cu", "bind_latent.cpp"],
               ["latent_kv_store", "rope_q_", "latent_window_attention", "window_softmax", "latent_prompt_attention",
                "latent_prompt_attention_fits"]),
    "linrec": (["linear_recurrence.cu", "gla_chunked.cu", "bind_linrec.cpp"], ["gla_scan", "rglru_scan", "retention_scan", "mingru_scan"]),
    "headmix": (["headmix_attention.cu", "headmix_decode.cu", "headmix_prefill.cu", "bind_headmix.cpp"],
                ["headmix_qk_prepare", "headmix_attention_prompt", "headmix_attention_token"]),
    "window": (["window_attention.cu", "window_prefill.cu", "bind_window.cpp"], ["window_qk_prepare", "window_attention_prompt", "window_attention_token"]),
    "matrec": (["matrix_recurrence.cu", "bind_matrec.cpp"], ["gated_delta_scan", "ssd_scan"]),
}
_GROUP_OF = {fn: g for g, (_, fns) in GROUPS.items() for fn in fns}
_MODS = {}


def ext_name(group: str) -> str:
    return f"nxd_b200_seq_{group}_C"


def build_group(group: str, verbose: bool = False) -> Path:
    """Compile one kernel group for sm_100a into ``_build/seqmix/<group>`` (IEEE math: no fast-math, the float paths are
    exact-rounded)."""
    from torch.utils import cpp_extension

    out = SEQ_BUILD_DIR / group
    out.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    srcs = [str(CSRC / f) for f in GROUPS[group][0]]
    cpp_extension.load(name=ext_name(group), sources=srcs, extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                                          "--expt-relaxed-constexpr"],
                       extra_include_paths=[str(CSRC)], build_directory=str(out), verbose=verbose, is_python_module=True,
                       with_cuda=True)
    so = out / f"{ext_name(group)}.so"
    assert so.exists(), f"build did not produce {so}"
    return so


def build(verbose: bool = False):
    """Compile every kernel group; returns the built libraries."""
    return [build_group(g, verbose) for g in GROUPS]


def _group_module(group: str):
    """A group's extension module; built on first use when absent or older than its sources (needs nvcc, no GPU)."""
    if group not in _MODS:
        so = SEQ_BUILD_DIR / group / f"{ext_name(group)}.so"
        deps = [CSRC / f for f in GROUPS[group][0]] + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
        if not so.exists() or so.stat().st_mtime < max(p.stat().st_mtime for p in deps):
            build_group(group)
        loader = importlib.machinery.ExtensionFileLoader(ext_name(group), str(so))
        mod = importlib.util.module_from_spec(importlib.util.spec_from_loader(ext_name(group), loader))
        loader.exec_module(mod)
        sys.modules[ext_name(group)] = mod
        _MODS[group] = mod
    return _MODS[group]


class _Kernels:
    """``ext().name`` → the function ``name`` of whichever group exports it."""

    def __getattr__(self, name: str):
        if name not in _GROUP_OF:
            raise AttributeError(name)
        fn = getattr(_group_module(_GROUP_OF[name]), name)
        setattr(self, name, fn)
        return fn


_KERNELS = _Kernels()


def ext():
    return _KERNELS


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


# --------------------------------------------------------------------------------------------------------------- short convolution
def short_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, slots: torch.Tensor,
               lens: torch.Tensor, fresh: bool, residual: bool, out_dtype: torch.dtype, silu: bool = False) -> torch.Tensor:
    """``x [B,S,C]``, ``w [C,taps]`` float, ``state [slots, taps-1, C]`` of x's dtype (updated in place) → ``[B,S,C]``:
    ``out_t = act((x_t if residual) + bias + sum_j w[:, j] * in_(t-taps+1+j))`` with ``act`` the identity or ``silu``; rows past
    ``lens`` give zeros."""
    if _cuda(x):
        _ext.count_launch()
        return ext().short_conv(x, w, bias, state, _i32(slots), _i32(lens), fresh, residual, out_dtype == torch.bfloat16, silu)
    B, S, C = x.shape
    taps = w.shape[1]
    hist = torch.zeros(B, taps - 1, C, dtype=x.dtype) if fresh else state[slots.long()]
    full = torch.cat([hist, x], 1).float()                                            # [B, taps-1+S, C]
    out = sum(w[:, j] * full[:, j:j + S] for j in range(taps))
    if bias is not None:
        out = out + bias
    if residual:
        out = out + x.float()
    if silu:
        out = F.silu(out)
    keep = torch.arange(S)[None, :] < lens[:, None]
    out = torch.where(keep[..., None], out, torch.zeros_like(out))
    if taps > 1:
        idx = lens.long()[:, None] + torch.arange(taps - 1)[None, :]                   # last taps-1 inputs end at hist+len
        state[slots.long()] = torch.cat([hist, x], 1).gather(1, idx[..., None].expand(B, taps - 1, C))
    return out.to(out_dtype)


# --------------------------------------------------------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, gate: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None, center: bool = False) -> torch.Tensor:
    """Rows of ``x [rows, C]`` divided by their root mean square, times ``w`` (``[C]`` or one number), times ``silu(gate)``.
    ``center``: the row's mean is taken off first (a layer norm with a gain and no bias: the statistics are the mean and the mean
    squared deviation)."""
    out_dtype = out_dtype or x.dtype
    if _cuda(x):
        _ext.count_launch()
        return ext().rms_norm(x, w, eps, gate, out_dtype == torch.bfloat16, center)
    xf = x.float()
    if center:
        xf = xf - xf.mean(-1, keepdim=True)
    y = xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w
    if gate is not None:
        y = y * F.silu(gate.float())
    return y.to(out_dtype)


def add_rms_norm_(res: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, center: bool = False) -> torch.Tensor:
    """``res`` (float ``[rows, C]``) ``+= y / rms(y) * w`` in place (``center``: y's mean is taken off first)."""
    if _cuda(y):
        _ext.count_launch()
        ext().add_rms_norm_(res, y, w, eps, center)
        return res
    yf = y.float()
    if center:
        yf = yf - yf.mean(-1, keepdim=True)
    res += yf / torch.sqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * w
    return res


def postnorm_gated_(x: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], w: torch.Tensor, alpha: float, eps: float,
                    lowp: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The closing step of a block whose norm comes after the residual sum, on the float stream ``x [rows, C]`` in place:
    ``x <- rms_norm(alpha * x + sigmoid(gate) * y) * w`` (``gate`` None: ``alpha * x + y``).  ``y`` and ``gate`` are ``[rows, C]``
    views of one dtype (row strides free); ``lowp`` (``[rows, C]`` of that dtype) receives a copy of the result."""
    if _cuda(x):
        _ext.count_launch()
        ext().postnorm_gated_(x, y, gate, w, float(alpha), float(eps), lowp)
        return x
    v = alpha * x + (y.float() if gate is None else torch.sigmoid(gate.float()) * y.float())
    x.copy_(v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w)
    if lowp is not None:
        lowp.copy_(x.to(lowp.dtype))
    return x


# ---------------------------------------------------------------------------------------------------------------- latent attention
def rotary_inv_freq(dims: int, base: float, device=None, scaling: Optional[dict] = None) -> torch.Tensor:
    """``base^(-2i/dims)`` for i < dims/2, rounded once from float64.  ``scaling`` (``factor``, ``low``, ``high``, ``original``)
    rescales them for a longer context by wavelength ``l = 2 pi / f``: kept where ``l < original / high``, divided by ``factor`` where
    ``l > original / low``, and in between blended with ``s = (original / l - low) / (high - low)`` as
    ``(1 - s) f / factor + s f``."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * math.pi / f
        s_ = (orig / wl - low) / (high - low) if high != low else torch.zeros_like(f)
        f = torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, (1.0 - s_) * f / factor + s_ * f))
    return f.float().to(device)


def _rotate(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, dims: int) -> torch.Tensor:
    """x ``[..., n]`` float, pos broadcastable to x's leading dims: rotate-half on the first ``dims`` coordinates."""
    half = dims // 2
    ang = pos.float()[..., None] * inv_freq
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def latent_kv_store(kv: torch.Tensor, nw: torch.Tensor, eps: float, inv_freq: torch.Tensor, dims: int, pos0: torch.Tensor,
                    lens: torch.Tensor, slots: torch.Tensor, cache: Optional[torch.Tensor], want_rows: bool) -> Optional[torch.Tensor]:
    """``kv [B,S,C+R]``: RMS-norm (weight ``nw [C]``) of the first C numbers, rotation of the next ``dims`` at positions
    ``pos0[b] + t``.  The last ``ring`` real tokens of each row go to ``cache [slots, ring, C+R]`` at row ``position mod ring``;
    with ``want_rows`` the prepared rows come back as ``[B,S,C+R]``."""
    if _cuda(kv):
        _ext.count_launch()
        rows = ext().latent_kv_store(kv, nw, eps, inv_freq, dims, _i32(pos0), _i32(lens), _i32(slots), cache, want_rows)
        return rows if want_rows else None
    B, S, _ = kv.shape
    C = nw.numel()
    f = kv.float()
    c = f[..., :C]
    c = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * nw
    pos = pos0.long()[:, None] + torch.arange(S)[None, :]
    rows = torch.cat([c, _rotate(f[..., C:], pos, inv_freq, dims)], -1).to(kv.dtype)
    if cache is not None:
        ring = cache.shape[1]
        for b in range(B):
            n = int(lens[b])
            for t in range(max(0, n - ring), n):
                cache[int(slots[b]), int(pos[b, t]) % ring] = rows[b, t]
    return rows if want_rows else None


def rope_q_(q: torch.Tensor, off: int, dims: int, inv_freq: torch.Tensor, pos0: torch.Tensor) -> torch.Tensor:
    """``q [B,S,H,Dq]``: coordinates ``[off, off+dims)`` of every head rotated in place at positions ``pos0[b] + t``."""
    if _cuda(q):
        _ext.count_launch()
        ext().rope_q_(q, off, dims, inv_freq, _i32(pos0))
        return q
    S = q.shape[1]
    pos = (pos0.long()[:, None] + torch.arange(S)[None, :])[:, :, None]
    q[..., off:off + dims] = _rotate(q[..., off:off + dims].float(), pos, inv_freq, dims).to(q.dtype)
    return q


LATENT_ROW_MAX = 640        # widest key-store row (latent + rotated part) the attention kernels take


def latent_window_attention(qa: torch.Tensor, q: torch.Tensor, off: int, keys: torch.Tensor, key_index: Optional[torch.Tensor],
                            pos0: torch.Tensor, lens: torch.Tensor, window: int, scale: float) -> torch.Tensor:
    """``qa [H, B*S, C]`` absorbed queries, ``q [B,S,H,Dq]`` whose coordinates from ``off`` are the rotated part, ``keys
    [blocks, ring, C+R]`` (row ``j mod ring`` of block ``key_index[b]``, or of block b, holds position j).  Position p sees
    ``p - window < j <= p``.  Returns the attention-weighted sum of the latents ``[H, B*S, C]``; padded rows give zeros."""
    if _cuda(qa):
        _ext.count_launch()
        return ext().latent_window_attention(qa, q, off, keys, None if key_index is None else _i32(key_index), _i32(pos0), _i32(lens),
                                             window, scale)
    H, N, C = qa.shape
    B, S = q.shape[:2]
    ring, R = keys.shape[1], keys.shape[2] - C
    kb = keys[key_index.long()] if key_index is not None else keys                                  # [B, ring, C+R]
    qq = torch.cat([qa.float().view(H, B, S, C).permute(1, 2, 0, 3), q[..., off:off + R].float()], -1)  # [B,S,H,C+R]
    sc = torch.einsum("bshc,brc->bshr", qq, kb.float()) * scale
    p = pos0.long()[:, None] + torch.arange(S)[None, :]                                              # [B,S]
    r = torch.arange(ring)
    j = p[..., None] - torch.remainder(p[..., None] - r, ring)                                       # position held by ring row r
    ok = (j >= 0) & (j > p[..., None] - window)
    sc = sc.masked_fill(~ok[:, :, None, :], float("-inf"))
    o = torch.einsum("bshr,brc->bshc", torch.softmax(sc, -1), kb.float()[..., :C])
    o = torch.where((torch.arange(S)[None, :] < lens[:, None])[..., None, None], o, torch.zeros_like(o))
    return o.permute(2, 0, 1, 3).reshape(H, N, C).to(qa.dtype)


def latent_prompt_fused_ok(q: torch.Tensor, D: int, R: int, CR: int, VD: int) -> bool:
    """True when the one-kernel prompt attention takes this call: bfloat16 on the GPU, sizes in whole 16s (8s for the parts)."""
    return _cuda(q) and q.dtype == torch.bfloat16 and ext().latent_prompt_attention_fits(D, R, CR, VD)


def latent_prompt_attention(q: torch.Tensor, kx: torch.Tensor, rows: torch.Tensor, v: torch.Tensor, lens: torch.Tensor, D: int, R: int,
                            VD: int, window: int, scale: float) -> torch.Tensor:
    """Prompts that start at position 0, expanded form, one kernel (GPU, bfloat16): ``q [B,S,H,D+R]`` rotated queries, ``kx
    [B,S,H*D]`` every head's unrotated keys, ``rows [B,S,CR]`` whose last R numbers are the rotated key part all heads share, ``v
    [B,S,H*VD]``.  Query i sees ``i - window < j <= i``.  Returns the heads' outputs ``[B*S, H*VD]``; padded rows give zeros."""
    _ext.count_launch()
    return ext().latent_prompt_attention(q, kx.contiguous(), rows, v.contiguous(), _i32(lens), D, R, VD, window, scale)


def window_softmax(scores: torch.Tensor, scale: float, ring_mode: bool, H: int, Qb: int, nblk: int, w_eff: int, window: int,
                   pos0: torch.Tensor, lens: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Softmax over the visible keys of float score rows made by block matrix products; masked entries come out as zeros.
    Band mode: ``scores [B, nblk, Qb*H, span]``, column kk of block ``blk`` is position ``blk*Qb - (w_eff-1) + kk``; the query of
    row ``(t, h)`` sits at ``i = blk*Qb + t`` and sees ``max(0, i-window+1) <= j <= i``; rows with ``i >= lens[b]`` are zeros.
    Ring mode: ``scores [B, H, ring]`` of single tokens at ``pos0[b]``; ring row kk holds position ``p - ((p - kk) mod ring)``."""
    if _cuda(scores):
        _ext.count_launch()
        return ext().window_softmax(scores, scale, ring_mode, H, Qb, nblk, w_eff, window, _i32(pos0), _i32(lens), out_dtype == torch.bfloat16)
    span = scores.shape[-1]
    kk = torch.arange(span)
    if ring_mode:
        p = pos0.long()[:, None]
        m = torch.remainder(p - kk, span)
        ok = ((p - m >= 0) & (m < window))[:, None, :] & (lens > 0)[:, None, None]                    # [B,1,ring]
    else:
        blk, t = torch.arange(nblk)[:, None, None], torch.arange(Qb)[None, :, None]
        i, j = blk * Qb + t, blk * Qb - (w_eff - 1) + kk[None, None, :]                                # [nblk,Qb,1], [nblk,1,span]
        ok = (j >= 0) & (j <= i) & (j > i - window)                                                   # [nblk,Qb,span]
        ok = ok[None] & (i[None] < lens.long()[:, None, None, None])                                  # [B,nblk,Qb,span]
        ok = ok[:, :, :, None, :].expand(-1, -1, -1, H, -1).reshape(scores.shape)
    sc = (scores.float() * scale).masked_fill(~ok.expand(scores.shape), float("-inf"))
    return torch.nan_to_num(torch.softmax(sc, -1), nan=0.0).to(out_dtype)


SMALL_LINEAR_ROWS = 16        # up to this many rows a float-result product runs as one warp per output


def linear_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x [N, I]`` (row stride free) times ``w [O, I]`` → float ``[N, O]``: the operands as they are stored, float accumulation and
    a float result (router logits; per-head scalars that enter a recurrence)."""
    if _cuda(x) and x.shape[0] <= SMALL_LINEAR_ROWS and x.stride(-1) == 1:
        _ext.count_launch()
        return ext().small_linear_f32(x, w)
    if x.dtype == torch.float32 or not x.is_cuda:
        return F.linear(x.float(), w.float())
    return torch.bmm(x[None], w.to(x.dtype).t()[None], out_dtype=torch.float32)[0]


ROUTE_MAX_EXPERTS = 256
ROUTE_KINDS = {"sigmoid": 0, "softmax": 1, "softmax_top": 2}


def route_topk(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, n_real: int, act: str = "softmax", scale: float = 1.0):
    """Float router logits ``[N, E]`` → ``(weights [N, top] float, expert ids [N, top] int64, identity share [N] float)``.
    ``scores = softmax / sigmoid(logits)``; the ``top`` largest of ``scores + correction`` are chosen (descending); a chosen expert
    below ``n_real`` gets weight ``score * scale``, a chosen expert from ``n_real`` on (an identity expert) gets weight 0 and adds its
    score to the row's identity share.  ``act="softmax_top"``: the ``top`` largest LOGITS are chosen and the weights are the softmax
    over the chosen logits only (times ``scale``); no correction, no identity experts."""
    if _cuda(logits) and logits.shape[1] <= ROUTE_MAX_EXPERTS:
        _ext.count_launch()
        w, idx, ident = ext().route_topk(logits.contiguous(), correction, top, n_real, ROUTE_KINDS[act], float(scale))
        return w, idx, ident
    if act == "softmax_top":
        val, idx = torch.topk(logits.float(), top, dim=-1)
        return torch.softmax(val, -1) * scale, idx, torch.zeros(logits.shape[0], device=logits.device)
    scores = torch.softmax(logits.float(), -1) if act == "softmax" else torch.sigmoid(logits.float())
    idx = torch.topk(scores if correction is None else scores + correction, top, dim=-1).indices
    w = scores.gather(1, idx)
    real = idx < n_real
    ident = torch.where(real, torch.zeros_like(w), w).sum(1)
    return torch.where(real, w * scale, torch.zeros_like(w)), idx, ident


def matmul_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched ``a @ b`` with a float result (float accumulation of bfloat16 operands is kept, not rounded)."""
    if a.dtype == torch.float32:
        return torch.bmm(a, b)
    if a.is_cuda:
        return torch.bmm(a, b, out_dtype=torch.float32)
    return torch.bmm(a.float(), b.float())


# -------------------------------------------------------------------------------------------------------------------- recurrences
def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, zbias: torch.Tensor, tau: float, state: torch.Tensor,
             slots: torch.Tensor, lens: torch.Tensor, fresh: bool) -> torch.Tensor:
    """``q, k [B,S,H,D]``, ``v [B,S,H,V]``, decay logits ``z [B,S,H*D]`` (+ ``zbias``) → float ``[B,S,H,V]``:
    ``alpha = sigmoid(z)^(1/tau)``; ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``; ``o_t = S_t^T q_t / sqrt(D)``.  ``state
    [slots,H,D,V]`` float is read (unless ``fresh``) and left at each row's last real token."""
    if _cuda(q):
        _ext.count_launch()
        return ext().gla_scan(q, k, v, z, zbias, tau, state, _i32(slots), _i32(lens), fresh)
    B, S, H, D = q.shape
    V = v.shape[-1]
    alpha = torch.exp(F.logsigmoid(z.float() + zbias) / tau).view(B, S, H, D)
    qf, kf, vf = q.float() * D ** -0.5, k.float(), v.float()
    st = torch.zeros(B, H, D, V) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, H, V)
    for t in range(S):
        live = (t < lens)[:, None, None, None]
        new = alpha[:, t, :, :, None] * st + kf[:, t, :, :, None] * vf[:, t, :, None, :]
        st = torch.where(live, new, st)
        out[:, t] = torch.where(live[..., 0], torch.einsum("bhdv,bhd->bhv", st, qf[:, t]), out[:, t])
    state[slots.long()] = st
    return out


def rglru_scan(u: torch.Tensor, gr: torch.Tensor, gi: torch.Tensor, rbias: torch.Tensor, ibias: torch.Tensor, lam_sp: torch.Tensor,
               y: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, lens: torch.Tensor, fresh: bool) -> torch.Tensor:
    """``u [B,S,W]``; gate pre-activations ``gr, gi`` float ``[blocks, B*S, W/blocks]``; ``y [B,S,W]`` (pre-activation of the
    gelu branch) → ``[B,S,W]``: ``a = exp(-8 sigmoid(gr + rbias) lam_sp)``, ``h_t = a h_(t-1) + sqrt(1 - a^2) sigmoid(gi + ibias)
    u_t``, ``out = h_t * gelu_tanh(y_t)``.  ``state [slots, W]`` float."""
    if _cuda(u):
        _ext.count_launch()
        return ext().rglru_scan(u, gr, gi, rbias, ibias, lam_sp, y, state, _i32(slots), _i32(lens), fresh)
    B, S, W = u.shape
    nb, _, wb = gr.shape
    r = torch.sigmoid(gr.view(nb, B, S, wb).permute(1, 2, 0, 3).reshape(B, S, W) + rbias)
    g = torch.sigmoid(gi.view(nb, B, S, wb).permute(1, 2, 0, 3).reshape(B, S, W) + ibias)
    la = -8.0 * r * lam_sp
    a, mult = torch.exp(la), torch.sqrt(-torch.expm1(2.0 * la))
    h = torch.zeros(B, W) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, W)
    for t in range(S):
        live = (t < lens)[:, None]
        h = torch.where(live, a[:, t] * h + mult[:, t] * g[:, t] * u[:, t].float(), h)
        out[:, t] = torch.where(live, h * F.gelu(y[:, t].float(), approximate="tanh"), out[:, t])
    state[slots.long()] = h
    return out.to(u.dtype)


def mingru_scan(z: torch.Tensor, u: torch.Tensor, g: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, lens: torch.Tensor,
                fresh: bool) -> torch.Tensor:
    """Minimal gated recurrent unit whose gates read only the current token.  Pre-activations ``z, u, g [B,S,W]`` (views with the same
    strides) → ``[B,S,W]``: ``zt = sigmoid(z)``, candidate ``c = u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` below,
    ``h_t = (1 - zt) h_(t-1) + zt c`` per channel, ``out = h_t * silu(g)``.  ``state [slots, W]`` float is read (unless ``fresh``) and
    left at each row's last real token; gates, candidate and state are float."""
    if _cuda(z):
        _ext.count_launch()
        return ext().mingru_scan(z, u, g, state, _i32(slots), _i32(lens), fresh)
    B, S, W = z.shape
    zf, uf, gf = z.float(), u.float(), g.float()
    keep, take = torch.sigmoid(-zf), torch.sigmoid(zf)
    cand = torch.where(uf >= 0, uf + 0.5, torch.sigmoid(uf))
    h = torch.zeros(B, W) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, W)
    for t in range(S):
        live = (t < lens)[:, None]
        h = torch.where(live, keep[:, t] * h + take[:, t] * cand[:, t], h)
        out[:, t] = torch.where(live, h * F.silu(gf[:, t]), out[:, t])
    state[slots.long()] = h
    return out.to(z.dtype)


# -------------------------------------------------------------------------------------------------- activations, routed small batch
def xielu(x: torch.Tensor, ap: float, an: float) -> torch.Tensor:
    """``z > 0: ap z^2 + z/2``; ``z <= 0: an (exp(z) - 1 - z) + z/2``."""
    if _cuda(x):
        _ext.count_launch()
        return ext().xielu(x.contiguous(), ap, an)
    z = x.float()
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(z) - z) + 0.5 * z).to(x.dtype)


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    if _cuda(x):
        _ext.count_launch()
        return ext().gelu_erf(x.contiguous())
    return F.gelu(x.float()).to(x.dtype)


def relu_sq(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0)^2``."""
    if _cuda(x):
        _ext.count_launch()
        return ext().relu_sq(x.contiguous())
    return torch.relu(x.float()).pow(2).to(x.dtype)


GEMV_ACTS = {None: 0, "none": 0, "gelu": 1, "silu_glu": 2, "relu_sq": 3}


def indexed_gemv(w: torch.Tensor, sel: torch.Tensor, x: torch.Tensor, act) -> torch.Tensor:
    """``w [E,O,I]``, ``sel [M]``, ``x [M,I]`` → ``act(w[sel[m]] @ x[m])`` (float accumulation).  ``act``: ``None``, ``"gelu"`` (erf
    form; ``True`` means the same), ``"relu_sq"`` (the square of relu) or ``"silu_glu"``: the matrix stacks gate rows over up rows and the result is
    ``silu(gate) * up``, ``[M, O/2]``.  Rows whose ``sel`` names no matrix (``< 0`` or ``>= E``) give zeros."""
    kind = GEMV_ACTS["gelu" if act is True else (None if act is False else act)]
    if _cuda(x):
        _ext.count_launch()
        return ext().indexed_gemv(w, _i32(sel), x, kind)
    ok = (sel >= 0) & (sel < w.shape[0])
    y = torch.einsum("moi,mi->mo", w[sel.long().clamp(0, w.shape[0] - 1)].float(), x.float())
    if kind == 1:
        y = F.gelu(y)
    elif kind == 2:
        half = y.shape[1] // 2
        y = F.silu(y[:, :half]) * y[:, half:]
    elif kind == 3:
        y = torch.relu(y).pow(2)
    return torch.where(ok[:, None], y, torch.zeros_like(y)).to(x.dtype)


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    """``gu [M, 2F]`` (gate columns, then up columns) → ``silu(gate) * up`` ``[M, F]``."""
    if _cuda(gu):
        _ext.count_launch()
        return ext().silu_mul(gu)
    half = gu.shape[1] // 2
    return (F.silu(gu[:, :half].float()) * gu[:, half:].float()).to(gu.dtype)


def moe_combine(rows: torch.Tensor, src: torch.Tensor, weight: torch.Tensor, base: Optional[torch.Tensor],
                base_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[n] = base_weight[n] * base[n] + sum_k weight[n,k] * rows[src[n,k]]`` summed in float; ``rows [M,C]``, ``src, weight
    [N,top]``, ``base [N,C]`` (optional; ``base_weight [N]`` float, one when absent)."""
    if _cuda(rows):
        _ext.count_launch()
        return ext().moe_combine(rows, _i32(src), weight, base, base_weight)
    y = (rows.float()[src.long()] * weight[..., None]).sum(1)
    if base is not None:
        y = y + (base.float() if base_weight is None else base.float() * base_weight[:, None])
    return y.to(rows.dtype)


# ------------------------------------------------------------------------------------------------- embedding with sinusoid positions
def sinusoid_inv_freq(width: int, base: float, device=None) -> torch.Tensor:
    """``base^(-2i/width)`` for i < ceil(width/2), rounded once from float64."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / width).float().to(device)


def embed_sinusoid(tokens: torch.Tensor, table: torch.Tensor, scale: float, inv_freq: torch.Tensor, pos0: torch.Tensor) -> torch.Tensor:
    """``tokens [B,S]`` → float ``[B,S,W]``: ``table[token] * scale`` plus interleaved sinusoids of the position ``p = pos0[b] + t``
    (coordinate 2i: ``sin(p f_i)``, 2i+1: ``cos(p f_i)``; angles in float)."""
    if _cuda(table):
        _ext.count_launch()
        return ext().embed_sinusoid(tokens.contiguous(), table, float(scale), inv_freq, _i32(pos0))
    B, S = tokens.shape
    W = table.shape[1]
    ang = (pos0.long()[:, None] + torch.arange(S)[None, :]).float()[..., None] * inv_freq          # [B,S,ceil(W/2)]
    pe = torch.stack([torch.sin(ang), torch.cos(ang)], -1).reshape(B, S, -1)[..., :W]
    return table[tokens].float() * scale + pe


def embed_bigram(tokens: torch.Tensor, table: torch.Tensor, scale: float, pairs: Optional[torch.Tensor], mul_prev: int, mul_cur: int,
                 prev: Optional[torch.Tensor], slots: torch.Tensor, lens: torch.Tensor, fresh: bool, want_lowp: bool = False):
    """``tokens [B,S]`` → float ``[B,S,W]`` (and a copy in the table's dtype with ``want_lowp``): ``table[token] * scale`` plus
    ``pairs[r]``, a table of ``buckets + 1`` rows indexed by a hash of the token and the one before it,
    ``r = (previous * mul_prev + token * mul_cur) mod buckets``; a sequence's first token takes the last row.  ``prev [slots]``
    (int64) carries each sequence's last token between calls: read for a row's first token unless ``fresh``, and left at the row's
    last real token."""
    if _cuda(table):
        _ext.count_launch()
        out, lp = ext().embed_bigram(tokens.contiguous(), table, float(scale), pairs, int(mul_prev), int(mul_cur), prev, _i32(slots), _i32(lens),
                                     fresh, want_lowp)
        return (out, lp) if want_lowp else (out, None)
    B, S = tokens.shape
    tok = tokens.long().clamp(0, table.shape[0] - 1)
    out = table[tok].float() * scale
    if pairs is not None:
        buckets = pairs.shape[0] - 1
        first = torch.full((B,), -1, dtype=torch.long) if (fresh or prev is None) else prev[slots.long()].clone()
        before = torch.cat([first[:, None], tok[:, :-1]], 1)
        row = torch.where(before < 0, torch.full_like(tok, buckets), (before * mul_prev + tok * mul_cur) % buckets)
        out = out + pairs[row].float()
    if prev is not None:
        n = lens.long().clamp(max=S)
        last = tok.gather(1, (n - 1).clamp(min=0)[:, None])[:, 0]
        old = prev[slots.long()]
        prev[slots.long()] = torch.where(n > 0, last, old)
    return out, (out.to(table.dtype) if want_lowp else None)


# ------------------------------------------------------------------------------------------------------------- grouped gated norm
def group_rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, groups: int, eps: float, gate_first: bool,
                         out: Optional[torch.Tensor] = None, out_scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
                         gate_act: str = "silu") -> torch.Tensor:
    """Rows of ``x [rows, C]`` in ``groups`` equal parts, each divided by its own root mean square, with a ``silu(gate)`` factor
    (``gate_act="sigmoid"``: a ``sigmoid(gate)`` factor):
    ``gate_first``: ``rms_g(x * silu(gate)) * w`` (the gate enters the statistics); otherwise ``rms_g(x) * w * silu(gate)``.
    ``w`` holds ``C`` numbers or ``C / groups`` (shared by the groups).  The result times ``out_scale`` goes to ``out`` (any row
    stride) or a new ``[rows, C]`` tensor of ``out_dtype``."""
    rows, C = x.shape
    if out is None:
        out = torch.empty(rows, C, dtype=out_dtype or gate.dtype, device=x.device)
    if _cuda(x):
        _ext.count_launch()
        ext().group_rms_norm_gated(x, gate, w, groups, eps, gate_first, out, out_scale, gate_act == "sigmoid")
        return out
    xf, g = x.float(), (torch.sigmoid(gate.float()) if gate_act == "sigmoid" else F.silu(gate.float()))
    if gate_first:
        xf = xf * g
    xg = xf.view(rows, groups, C // groups)
    y = (xg / torch.sqrt(xg.pow(2).mean(-1, keepdim=True) + eps)).view(rows, C) * (w if w.numel() == C else w.repeat(groups))
    if not gate_first:
        y = y * g
    out.copy_((y * out_scale).to(out.dtype))
    return out


# ------------------------------------------------------------------------------------- grouped-query sliding-window attention
def window_qk_prepare(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], qw: Optional[torch.Tensor],
                      kw: Optional[torch.Tensor], eps: float, pos0: torch.Tensor, lens: torch.Tensor, slots: torch.Tensor,
                      kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], norm_all: bool = False,
                      inv_freq: Optional[torch.Tensor] = None, rot_dims: int = 0) -> None:
    """``q [B,S,H,D]``, ``k [B,S,G,D]``, ``v [B,S,G,V]`` (views; last dim contiguous), all IN PLACE.  Norm: every head's query and key
    is divided by its root mean square and multiplied by ``qw`` / ``kw`` (``[D]`` float; ``None``: left as they are); with
    ``norm_all`` the root mean square is taken over ALL heads of the token's queries (keys) at once and the weights hold ``H*D``
    (``G*D``) numbers.  Rotation (``inv_freq [rot_dims/2]`` given): afterwards the first ``rot_dims`` coordinates of every query and
    key head are rotated at position ``pos0[b] + t``, coordinate ``i`` paired with ``i + rot_dims/2``, angles in float.  The last
    ``ring`` real tokens of each row go to ``kcache [slots, ring, G, D]`` / ``vcache [slots, ring, G, V]`` at row
    ``position mod ring``.  ``k`` None (then ``v`` and the caches too): only the queries are prepared."""
    if _cuda(q):
        _ext.count_launch()
        ext().window_qk_prepare(q, k, v, qw, kw, norm_all, eps, inv_freq, rot_dims if inv_freq is not None else 0, _i32(pos0), _i32(lens),
                                _i32(slots), kcache, vcache)
        return
    B, S = q.shape[:2]
    pos = (pos0.long()[:, None] + torch.arange(S)[None, :])[:, :, None]

    def prep(x, w):
        f = x.float()
        if w is not None and norm_all:
            flat = f.flatten(2)
            f = (flat / torch.sqrt(flat.pow(2).mean(-1, keepdim=True) + eps) * w).view(f.shape)
        elif w is not None:
            f = f / torch.sqrt(f.pow(2).mean(-1, keepdim=True) + eps) * w
        if inv_freq is not None and rot_dims:
            f = _rotate(f, pos, inv_freq, rot_dims)
        return f.to(x.dtype)

    if qw is not None or inv_freq is not None:
        q.copy_(prep(q, qw))
    if k is None:
        return
    if kw is not None or inv_freq is not None:
        k.copy_(prep(k, kw))
    ring = kcache.shape[1]
    for b in range(B):
        n, p0, sl = int(lens[b]), int(pos0[b]), int(slots[b])
        for t in range(max(0, n - ring), n):
            kcache[sl, (p0 + t) % ring] = k[b, t]
            vcache[sl, (p0 + t) % ring] = v[b, t]


def _capped(sc: torch.Tensor, softcap: float) -> torch.Tensor:
    return softcap * torch.tanh(sc / softcap) if softcap > 0 else sc


def _window_weights(sc: torch.Tensor, ok: torch.Tensor, score_bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``sc [B,H,...,keys]`` scores, ``ok`` broadcastable → weights: a softmax over the visible keys, or with ``score_bias [H]``
    ``sigmoid(score + bias[h])`` of every visible key by itself."""
    if score_bias is None:
        return torch.nan_to_num(torch.softmax(sc.masked_fill(~ok, float("-inf")), -1), nan=0.0)
    bias = score_bias.view((1, -1) + (1,) * (sc.dim() - 2))
    return torch.sigmoid(sc + bias) * ok


def window_attention_prompt(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: Optional[torch.Tensor], lens: torch.Tensor,
                            window: int, scale: float, softcap: float, out: torch.Tensor, out_scale: float = 1.0,
                            score_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prompts that start at position 0: ``q [B,S,H,D]``, ``k [B,S,G,D]``, ``v [B,S,G,V]`` (views), query head h uses key/value head
    ``h // (H/G)``; query i sees ``i - window < j <= i``.  Scores ``q.k * scale``, capped as ``softcap * tanh(score / softcap)``
    when ``softcap > 0``, softmax in float; with ``score_bias [H]`` (float) the weight of a visible key is
    ``sigmoid(score + score_bias[h])`` instead, not normalised over the keys.  Each head's result is multiplied by
    ``sigmoid(gate[b,s,h])`` (if given) and ``out_scale`` and written to ``out [B*S, >= H*V]`` (row stride free); padded rows give
    zeros."""
    if _cuda(q):
        _ext.count_launch()
        ext().window_attention_prompt(q, k, v, gate, _i32(lens), window, scale, softcap, score_bias, out, out_scale)
        return out
    B, S, H, D = q.shape
    G, V = k.shape[2], v.shape[3]
    kk, vv = k.float().repeat_interleave(H // G, 2), v.float().repeat_interleave(H // G, 2)
    sc = _capped(torch.einsum("bihd,bjhd->bhij", q.float(), kk) * scale, softcap)
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    real = (torch.arange(S)[None, :] < lens[:, None])
    vv = torch.where(real[..., None, None], vv, torch.zeros(()))
    sc = torch.where(real[:, None, None, :], sc, torch.zeros(()))                               # padded rows hold anything
    o = torch.einsum("bhij,bjhv->bihv", _window_weights(sc, ((j <= i) & (j > i - window))[None, None], score_bias), vv)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())[..., None]
    o = torch.where((torch.arange(S)[None, :] < lens[:, None])[..., None, None], o * out_scale, torch.zeros_like(o))
    out[:, :H * V] = o.reshape(B * S, H * V).to(out.dtype)
    return out


def window_attention_token(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, gate: Optional[torch.Tensor], slots: torch.Tensor,
                           pos0: torch.Tensor, lens: torch.Tensor, window: int, scale: float, softcap: float, out: torch.Tensor,
                           out_scale: float = 1.0, score_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single tokens ``q [B,1,H,D]`` at positions ``pos0`` against their slots' rings (``kcache [slots, ring, G, D]``, ``vcache
    [slots, ring, G, V]``; row ``j mod ring`` holds position j, the token's own row included; ``ring >= window``).  Same scores,
    weights, gate and output layout as :func:`window_attention_prompt`; rows with ``lens == 0`` give zeros."""
    if _cuda(q):
        _ext.count_launch()
        ext().window_attention_token(q, kcache, vcache, gate, _i32(slots), _i32(pos0), _i32(lens), window, scale, softcap, score_bias, out,
                                     out_scale)
        return out
    B, _, H, D = q.shape
    ring, G, V = kcache.shape[1], kcache.shape[2], vcache.shape[3]
    kb = kcache[slots.long()].float().repeat_interleave(H // G, 2)                                  # [B, ring, H, D]
    vb = vcache[slots.long()].float().repeat_interleave(H // G, 2)
    sc = _capped(torch.einsum("bhd,brhd->bhr", q[:, 0].float(), kb) * scale, softcap)
    p = pos0.long()[:, None]
    m = torch.remainder(p - torch.arange(ring)[None, :], ring)                                      # distance back of ring row r
    ok = (p - m >= 0) & (m < window)
    sc = torch.where(ok[:, None, :], sc, torch.zeros(()))
    vb = torch.where(ok[:, :, None, None], vb, torch.zeros_like(vb))                               # rows never written hold anything
    o = torch.einsum("bhr,brhv->bhv", _window_weights(sc, ok[:, None, :], score_bias), vb)
    if gate is not None:
        o = o * torch.sigmoid(gate.float()).view(B, H, 1)
    o = torch.where((lens > 0)[:, None, None], o * out_scale, torch.zeros_like(o))
    out[:, :H * V] = o.reshape(B, H * V).to(out.dtype)
    return out


# ---------------------------------------------------------------------------------------------- matrix-state recurrences (scalar decay)
def gated_delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, braw: torch.Tensor, araw: torch.Tensor, a_log: torch.Tensor,
                     dt_bias: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, lens: torch.Tensor, fresh: bool) -> torch.Tensor:
    """Gated delta rule.  ``q, k [B,S,G,D]``, ``v [B,S,H,V]`` (views), ``braw, araw [B,S,H]`` float pre-activations → float
    ``[B,S,H,V]``.  Head h reads q/k head ``h // (H/G)``; q and k are made unit vectors (``x / sqrt(sum x^2 + 1e-6)``), q also
    times ``D^-1/2``; ``beta = sigmoid(braw)``, ``g = exp(-exp(a_log) softplus(araw + dt_bias))``; per token
    ``M <- g M; u = beta (v - M^T k); M <- M + k u^T; o = M^T q``.  ``state [slots,H,D,V]`` float.  With ``araw [B,S,H,D]`` and
    ``dt_bias [H*D]`` the decay is one number per head AND key channel, ``g [H,D]``, which scales the rows of M."""
    if _cuda(q):
        _ext.count_launch()
        return ext().gated_delta_scan(q, k, v, braw, araw, a_log, dt_bias, state, _i32(slots), _i32(lens), fresh)
    B, S, G, D = q.shape
    H, V = v.shape[2], v.shape[3]
    qf, kf = q.float(), k.float()
    qf = (qf / torch.sqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5).repeat_interleave(H // G, 2)
    kf = (kf / torch.sqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, 2)
    vf, beta = v.float(), torch.sigmoid(braw.float())
    if araw.dim() == 4:
        g = torch.exp(-torch.exp(a_log)[:, None] * F.softplus(araw.float() + dt_bias.view(H, D)))[..., None]      # [B,S,H,D,1]
    else:
        g = torch.exp(-torch.exp(a_log) * F.softplus(araw.float() + dt_bias))[..., None, None]                    # [B,S,H,1,1]
    st = torch.zeros(B, H, D, V) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, H, V)
    for t in range(S):
        live = (t < lens)[:, None, None, None]
        M = g[:, t] * st
        u = beta[:, t, :, None] * (vf[:, t] - torch.einsum("bhdv,bhd->bhv", M, kf[:, t]))
        M = M + kf[:, t, :, :, None] * u[:, :, None, :]
        st = torch.where(live, M, st)
        out[:, t] = torch.where(live[..., 0], torch.einsum("bhdv,bhd->bhv", st, qf[:, t]), out[:, t])
    state[slots.long()] = st
    return out


def ssd_scan(x: torch.Tensor, bm: torch.Tensor, cm: torch.Tensor, dtraw: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
             dskip: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, lens: torch.Tensor, fresh: bool) -> torch.Tensor:
    """Selective state space recurrence with a scalar decay per head.  ``x [B,S,H,V]``, ``bm, cm [B,S,G,N]`` (views), ``dtraw
    [B,S,H]`` float → float ``[B,S,H,V]``: ``dt = softplus(dtraw + dt_bias)``, ``M_t = exp(-exp(a_log) dt) M_(t-1) + dt b_t x_t^T``,
    ``y_t = M_t^T c_t + dskip x_t`` with head h reading group ``h // (H/G)``.  ``state [slots,H,N,V]`` float."""
    if _cuda(x):
        _ext.count_launch()
        return ext().ssd_scan(x, bm, cm, dtraw, a_log, dt_bias, dskip, state, _i32(slots), _i32(lens), fresh)
    B, S, H, V = x.shape
    G, N = bm.shape[2], bm.shape[3]
    xf = x.float()
    bf, cf = bm.float().repeat_interleave(H // G, 2), cm.float().repeat_interleave(H // G, 2)
    dt = F.softplus(dtraw.float() + dt_bias)
    dec = torch.exp(-torch.exp(a_log) * dt)
    st = torch.zeros(B, H, N, V) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, H, V)
    for t in range(S):
        live = (t < lens)[:, None, None, None]
        M = dec[:, t, :, None, None] * st + (dt[:, t, :, None] * bf[:, t])[..., None] * xf[:, t, :, None, :]
        st = torch.where(live, M, st)
        y = torch.einsum("bhnv,bhn->bhv", st, cf[:, t]) + dskip[None, :, None] * xf[:, t]
        out[:, t] = torch.where(live[..., 0], y, out[:, t])
    state[slots.long()] = st
    return out


# ------------------------------------------------------------------------------------------------ gated feed-forward, output gates
def clamped_glu(gu: torch.Tensor, limit: float, slope: float) -> torch.Tensor:
    """``gu [M, 2F]`` (gate columns, then up columns) → ``[M, F]``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``,
    ``g * sigmoid(slope * g) * (u + 1)``."""
    if _cuda(gu):
        _ext.count_launch()
        return ext().clamped_glu(gu, float(limit), float(slope))
    half = gu.shape[1] // 2
    g, u = gu[:, :half].float().clamp(max=limit), gu[:, half:].float().clamp(-limit, limit)
    return (g * torch.sigmoid(slope * g) * (u + 1.0)).to(gu.dtype)


def sigmoid_gate_mul_(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``x [N, C]`` (contiguous) times ``sigmoid(gate [N, Cg])`` in place, each gate number covering ``C / Cg`` consecutive
    coordinates of its row (``Cg = C``: one gate per coordinate; ``Cg = heads``: one per head).  ``gate``'s row stride is free."""
    if _cuda(x):
        _ext.count_launch()
        ext().sigmoid_gate_mul_(x, gate)
        return x
    N, C = x.shape
    rep = C // gate.shape[1]
    x.copy_((x.float().view(N, -1, rep) * torch.sigmoid(gate.float())[..., None]).view(N, C).to(x.dtype))
    return x


# ------------------------------------------------------------------------------------------------------- retention (fixed decay)
def rotary_qkv_f32(p: torch.Tensor, hq: int, hk: int, D: int, dims: int, inv_freq: torch.Tensor, pos0: torch.Tensor, q_scale: float,
                   k_scale: float) -> torch.Tensor:
    """``p [B,S,C]`` (a stacked projection: ``hq`` query heads of D numbers, ``hk`` key heads of D numbers, then anything) → float
    ``[B,S,C]``: the first ``dims`` coordinates of every query and key head rotated (rotate-half pairs) at positions
    ``pos0[b] + t`` in float, queries times ``q_scale``, keys times ``k_scale``, the rest copied."""
    if _cuda(p):
        _ext.count_launch()
        return ext().rotary_qkv_f32(p, hq, hk, D, dims, inv_freq, _i32(pos0), float(q_scale), float(k_scale))
    B, S, C = p.shape
    f = p.float()
    pos = (pos0.long()[:, None] + torch.arange(S)[None, :])[:, :, None]
    q = _rotate(f[..., :hq * D].reshape(B, S, hq, D), pos, inv_freq, dims) * q_scale
    k = _rotate(f[..., hq * D:(hq + hk) * D].reshape(B, S, hk, D), pos, inv_freq, dims) * k_scale
    return torch.cat([q.reshape(B, S, -1), k.reshape(B, S, -1), f[..., (hq + hk) * D:]], -1)


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
                   lens: torch.Tensor, fresh: bool) -> torch.Tensor:
    """Linear attention with ONE fixed decay per head: float ``q, k [B,S,H,D]``, ``v [B,S,H,V]`` (views), ``decay [H]`` float → float
    ``[B,S,H,V]``: ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` (no softmax, no denominator; scales are the
    caller's).  ``state [slots,H,D,V]`` float is read (unless ``fresh``) and left at each row's last real token."""
    if _cuda(q):
        _ext.count_launch()
        return ext().retention_scan(q, k, v, decay, state, _i32(slots), _i32(lens), fresh)
    B, S, H, D = q.shape
    V = v.shape[-1]
    qf, kf, vf = q.float(), k.float(), v.float()
    st = torch.zeros(B, H, D, V) if fresh else state[slots.long()].clone()
    out = torch.zeros(B, S, H, V)
    for t in range(S):
        live = (t < lens)[:, None, None, None]
        st = torch.where(live, decay[None, :, None, None] * st + kf[:, t, :, :, None] * vf[:, t, :, None, :], st)
        out[:, t] = torch.where(live[..., 0], torch.einsum("bhdv,bhd->bhv", st, qf[:, t]), out[:, t])
    state[slots.long()] = st
    return out


# -------------------------------------------------------------- softmax attention with scores mixed across heads and a sink term
# The mixing is linear in the queries, so it is moved onto them: with ``score_g = c_g q_g . k_kv(g)`` and ``s_h = sum_g T[h,g]
# score_g``, head h's mixed query against key head c is ``Q'[h,c,:] = sum_{g in group c} T[h,g] c_g q_g`` and ``s_h = sum_c Q'[h,c,:] .
# k_c``: one dot product of length G*D between head h's row of Q' and the position's keys with all key heads side by side.
def headmix_qk_prepare(q: torch.Tensor, k: torch.Tensor, mixw: torch.Tensor, dims: int, inv_freq: torch.Tensor, pos0: torch.Tensor,
                       lens: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, want_rows: bool):
    """Queries to be mixed across heads and keys that double as values: ``q [B,S,H,D]``, ``k [B,S,G,D]`` (views; last dim contiguous),
    ``mixw [H,H]`` float (``T[h,g] * c_g``).  Queries and keys are rotated on their first ``dims`` coordinates (rotate-half pairs, in
    float, at positions ``pos0[b] + t``).  Returns ``(Q' [B,S,H,G*D], rotated keys [B,S,G,D] or None)``.  The keys as they come are
    the VALUES: the last ``ring`` real tokens of each row go to ``kcache`` (rotated) and ``vcache`` (as they come), both ``[slots,
    ring, G, D]``, at row ``position mod ring``.  Rows past ``lens`` are left unwritten."""
    if _cuda(k):
        _ext.count_launch()
        qmix, rows = ext().headmix_qk_prepare(q, k, mixw, dims, inv_freq, _i32(pos0), _i32(lens), _i32(slots), kcache, vcache, want_rows)
        return qmix, (rows if want_rows else None)
    B, S, H, D = q.shape
    G = k.shape[2]
    pos = pos0.long()[:, None] + torch.arange(S)[None, :]
    qr = _rotate(q.float(), pos[:, :, None], inv_freq, dims).view(B, S, G, H // G, D)
    qmix = torch.einsum("hcr,bscrd->bshcd", mixw.view(H, G, H // G), qr).reshape(B, S, H, G * D).to(q.dtype)
    rows = _rotate(k.float(), pos[:, :, None], inv_freq, dims).to(k.dtype)
    ring = kcache.shape[1]
    for b in range(B):
        n = int(lens[b])
        for t in range(max(0, n - ring), n):
            kcache[int(slots[b]), int(pos[b, t]) % ring] = rows[b, t]
            vcache[int(slots[b]), int(pos[b, t]) % ring] = k[b, t]
    return qmix, (rows if want_rows else None)


def _visible(i: torch.Tensor, j: torch.Tensor, chunk: int, window: int) -> torch.Tensor:
    ok = (j <= i) & (j >= 0)
    if chunk > 0:
        ok = ok & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    if window > 0:
        ok = ok & (i - j < window)
    return ok


def _sink_softmax(sc: torch.Tensor, sink: Optional[torch.Tensor], ok: torch.Tensor) -> torch.Tensor:
    """``sc [B,H,Q,K]`` scores, ``ok`` broadcastable → weights: softmax over the visible keys whose denominator also holds
    ``exp(sink_h)``."""
    sc = sc.masked_fill(~ok, float("-inf"))
    if sink is not None:
        sc = torch.cat([sc, sink.view(1, -1, 1, 1).expand(sc.shape[0], -1, sc.shape[2], 1)], -1)
    p = torch.nan_to_num(torch.softmax(sc, -1), nan=0.0)
    return p[..., :-1] if sink is not None else p


def headmix_attention_prompt(qmix: torch.Tensor, krows: torch.Tensor, v: torch.Tensor, sink: Optional[torch.Tensor],
                             gate: Optional[torch.Tensor], lens: torch.Tensor, chunk: int, window: int, out: torch.Tensor) -> torch.Tensor:
    """Prompts that start at position 0: mixed queries ``qmix [B,S,H,G*D]``, rotated keys ``krows [B,S,G,D]``, values ``v [B,S,G,D]``
    (a view); head h reads value head ``h // (H/G)``.  Score of head h for (i, j): ``qmix[i,h] . krows[j]`` over all ``G*D`` numbers
    (float).  Query i sees ``j <= i`` of its own aligned chunk of ``chunk`` positions (0: no chunks) and within ``window`` positions
    back (0: no window).  Softmax in float with ``exp(sink[h])`` added to the denominator (no key, no value).  The heads' results
    times ``sigmoid(gate [B,S,H*D])`` go to ``out [B*S, H*D]`` (row stride free); padded rows give zeros."""
    if _cuda(qmix):
        _ext.count_launch()
        ext().headmix_attention_prompt(qmix, krows, v, sink, gate, _i32(lens), chunk, window, out)
        return out
    B, S, H, DK = qmix.shape
    G, D = krows.shape[2], krows.shape[3]
    real = torch.arange(S)[None, :] < lens[:, None]
    kk = torch.where(real[..., None], krows.float().reshape(B, S, DK), torch.zeros(()))              # padded rows hold anything
    vv = torch.where(real[..., None, None], v.float(), torch.zeros(())).repeat_interleave(H // G, 2)
    qq = torch.where(real[..., None, None], qmix.float(), torch.zeros(()))
    sc = torch.einsum("bihx,bjx->bhij", qq, kk)
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    p = _sink_softmax(sc, sink, _visible(i, j, chunk, window)[None, None])
    o = torch.einsum("bhij,bjhv->bihv", p, vv).reshape(B, S, H * D)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    o = torch.where(real[..., None], o, torch.zeros_like(o))
    out[:, :H * D] = o.reshape(B * S, H * D).to(out.dtype)
    return out


def headmix_attention_token(qmix: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, sink: Optional[torch.Tensor],
                            gate: Optional[torch.Tensor], slots: torch.Tensor, pos0: torch.Tensor, lens: torch.Tensor, chunk: int, window: int,
                            out: torch.Tensor) -> torch.Tensor:
    """Single tokens' mixed queries ``qmix [B,1,H,G*D]`` at positions ``pos0`` against their slots' rings (``kcache, vcache [slots,
    ring, G, D]``; row ``j mod ring`` holds position j, the token's own row included; the ring is at least as long as the longest
    visible stretch).  Scores, sink, gate and output layout as :func:`headmix_attention_prompt`; rows with ``lens == 0`` give zeros."""
    if _cuda(qmix):
        _ext.count_launch()
        ext().headmix_attention_token(qmix, kcache, vcache, sink, gate, _i32(slots), _i32(pos0), _i32(lens), chunk, window, out)
        return out
    B, _, H, DK = qmix.shape
    ring, G, D = kcache.shape[1], kcache.shape[2], kcache.shape[3]
    p_ = pos0.long()[:, None]
    back = torch.remainder(p_ - torch.arange(ring)[None, :], ring)                                   # distance back of ring row r
    ok = _visible(p_, p_ - back, chunk, window)                                                      # [B, ring]
    kb = torch.where(ok[..., None], kcache[slots.long()].float().reshape(B, ring, DK), torch.zeros(()))   # rows never written hold anything
    vb = torch.where(ok[..., None, None], vcache[slots.long()].float(), torch.zeros(())).repeat_interleave(H // G, 2)
    sc = torch.einsum("bhx,brx->bhr", qmix[:, 0].float(), kb)
    w = _sink_softmax(sc[:, :, None, :], sink, ok[:, None, None, :])[:, :, 0]                        # [B,H,ring]
    o = torch.einsum("bhr,brhv->bhv", w, vb).reshape(B, H * D)
    if gate is not None:
        o = o * torch.sigmoid(gate.float()).view(B, H * D)
    o = torch.where((lens > 0)[:, None], o, torch.zeros_like(o))
    out[:, :H * D] = o.to(out.dtype)
    return out


if __name__ == "__main__":
    for _so in build(verbose="-v" in sys.argv):
        print(_so)
