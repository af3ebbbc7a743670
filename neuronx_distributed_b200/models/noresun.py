"""Noresun: a decoder-only language model that alternates two kinds of sequence mixer — a minimal gated recurrent unit
(``modules/recurrent/mingru.py``) and grouped-query sliding-window attention with rotary positions, one RMS norm over the whole
query / key projection and independent sigmoid weights with a bias per head instead of a softmax
(``modules/attention/window_attention.py``), optionally reading another layer's cached keys and values — each followed by a routed
feed-forward of squared-relu experts whose weights are the softmax over the chosen logits (``modules/moe/routed_ffn.py``), or none.

Block shape: the norm comes after the residual sum, and every sublayer's result passes a sigmoid gate per coordinate projected from
the sublayer's input: ``x <- norm1(alpha x + sigmoid(W_g1 x + b) * mixer(x))`` then ``x <- norm2(alpha x + sigmoid(W_g2 x + b) * ff(x))``
(``modules/rms_norm.py:GatedPostRMSNorm``).  The sublayers read the normed stream itself; the mixer's gate rides on the mixer's
stacked input projection.  The embedding is scaled and a hashed embedding of the (previous token, token) pair is added; the previous
token is part of a sequence's state.  The logits reuse the embedding table.  The residual stream ``x`` is float; the sublayers
compute in the model dtype from a rounded copy that the closing kernel of the block before leaves.  ``config.json`` lists the layers
in order (``type``, ``mixer`` sizes, ``mlp`` or null), so any order and any sizes load without code changes.  Rotations pair
neighbouring coordinates in the checkpoint; the projections and norm weights are reordered at load so that the kernels pair the two
halves of the rotated stretch.

Serving is the slot-based wrapper shared with the other stateful families (``inference/slot_serving.py``)."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..inference.slot_serving import SlotServingModel
from ..inference.state_cache import SequenceStateManager, StepContext
from ..modules.attention.utils import deinterleave_index
from ..modules.attention.window_attention import GatedWindowAttention
from ..modules.moe.routed_ffn import RoutedFFN
from ..modules.recurrent import MinGRU
from ..modules.rms_norm import GatedPostRMSNorm
from ..ops import seqmix
from ..utils.sampling import Sampler


@dataclasses.dataclass
class NoresunConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]                    # [{"type", "mixer": {...}, "mlp": {...} | None}, ...] as in config.json
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    embedding_scale: float = 1.0
    bigram: Optional[Dict[str, int]] = None         # {"buckets", "mul_prev", "mul_cur"} or None: no pair embedding
    dtype: torch.dtype = torch.bfloat16
    device: Any = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **overrides) -> "NoresunConfig":
        emb = d.get("embedding") or {}
        big = emb.get("bigram")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=list(d["layers"]), norm_eps=float(d["norm"]["eps"]),
                   postln_alpha=float(d.get("postln_alpha", 1.0)), embedding_scale=float(emb.get("scale", 1.0)),
                   bigram={k: int(big[k]) for k in ("buckets", "mul_prev", "mul_cur")} if big else None, **overrides)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "NoresunConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f), **overrides)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _kv_key(owner: int):
    return ("window_kv", owner)


def _kv_source(spec: Dict[str, Any]) -> Optional[int]:
    src = spec["mixer"].get("kv_from") if spec["type"] == "attention" else None
    return None if src is None else int(src)


def _build_mixer(cfg: NoresunConfig, index: int, max_seq_len: int) -> nn.Module:
    spec = cfg.layers[index]
    m, kind = spec["mixer"], spec["type"]
    if kind == "mingru":
        return MinGRU(cfg.width, int(m["width"]), dtype=cfg.dtype, device=cfg.device, extra_rows=cfg.width)
    if kind == "attention":
        src = _kv_source(spec)
        borrowers = [s["mixer"] for s in cfg.layers if _kv_source(s) == index]
        if src is not None:
            owner = cfg.layers[src] if 0 <= src < index else None
            if owner is None or owner["type"] != "attention" or _kv_source(owner) is not None:
                raise ValueError(f"layer {index} borrows keys from layer {src}, which keeps none of its own before it")
            if any(owner["mixer"].get(k) != m.get(k) for k in ("kv_heads", "dim", "vdim")):
                raise ValueError(f"layer {index} and the layer it borrows keys from differ in key/value heads or sizes")
        rot = m.get("rot") or {}
        return GatedWindowAttention(cfg.width, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), window=int(m["mask"]["size"]),
                                    scale=float(m["scale"]), eps=cfg.norm_eps, qk_norm="all", head_gate=False, dtype=cfg.dtype, device=cfg.device,
                                    max_seq_len=max_seq_len, bias=True, weights="sigmoid", rot_dims=int(rot.get("dims", 0)),
                                    rot_base=float(rot.get("base", 10000.0)), rot_scaling=rot.get("scaling"),
                                    kv_key=_kv_key(src) if src is not None else (_kv_key(index) if borrowers else None), shares_kv=src is not None,
                                    ring_window=max([int(b["mask"]["size"]) for b in borrowers], default=0), extra_rows=cfg.width)
    raise ValueError(f"unknown mixer type {kind!r}")


def _build_ffn(cfg: NoresunConfig, f: Optional[Dict[str, Any]]) -> Optional[nn.Module]:
    if not f:
        return None
    if f["kind"] == "moe":
        r = f["router"]
        return RoutedFFN(cfg.width, int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), router_act="softmax_top", router_bias=True,
                         expert_act="relu_sq", dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


class NoresunLayer(nn.Module):
    def __init__(self, cfg: NoresunConfig, index: int, max_seq_len: int):
        super().__init__()
        spec = cfg.layers[index]
        self.kind, self.dtype = spec["type"], cfg.dtype
        src = _kv_source(spec)
        self.state_layer = index if src is None else src                 # whose state entries the mixer reads and writes
        self.mixer = _build_mixer(cfg, index, max_seq_len)               # its stacked projection carries the first gate's rows
        self.norm1 = GatedPostRMSNorm(cfg.width, cfg.postln_alpha, cfg.norm_eps, cfg.device)
        self.mlp = _build_ffn(cfg, spec.get("mlp"))
        if self.mlp is not None:
            self.gate2 = nn.Parameter(torch.zeros(cfg.width, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
            self.gate2_bias = nn.Parameter(torch.zeros(cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
            self.norm2 = GatedPostRMSNorm(cfg.width, cfg.postln_alpha, cfg.norm_eps, cfg.device)

    def state_spec(self):
        return self.mixer.state_spec()

    def forward(self, x: torch.Tensor, h: torch.Tensor, ctx: StepContext, st: Dict[str, torch.Tensor]):
        """``x [B,S,width]`` float residual stream, updated in place; ``h``: the same numbers in the model dtype (``x`` itself when
        that is float), the sublayers' input, updated in place as well."""
        B, S, W = x.shape
        lowp = None if h is x else h
        y, gate = self.mixer(h, ctx, st)
        self.norm1.apply_(x, y, gate, lowp)
        if self.mlp is not None:
            rows = h.view(B * S, W)
            gate = F.linear(rows, self.gate2, self.gate2_bias)
            self.norm2.apply_(x, self.mlp(rows), gate, lowp)
        return x


class NoresunForCausalLM(nn.Module):
    def __init__(self, cfg: NoresunConfig, max_seq_len: int = 1 << 30):
        super().__init__()
        self.cfg = self.config = cfg
        mk = lambda *s: nn.Parameter(torch.zeros(*s, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
        self.embed = mk(cfg.vocab, cfg.width)
        self.pairs = mk(cfg.bigram["buckets"] + 1, cfg.width) if cfg.bigram else None
        self.layers = nn.ModuleList([NoresunLayer(cfg, i, max_seq_len) for i in range(len(cfg.layers))])
        self.norm_weight = nn.Parameter(torch.ones(cfg.width, dtype=torch.float32, device=cfg.device), requires_grad=False)

    def state_specs(self):
        """One entry per layer, then the embedding's: the sequence's last token (the pair embedding of the next one needs it)."""
        return [layer.state_spec() for layer in self.layers] + [{"prev": ((), torch.int64)} if self.pairs is not None else {}]

    def body(self, input_ids: torch.Tensor, ctx: StepContext, states: SequenceStateManager, tap=None) -> torch.Tensor:
        big = self.cfg.bigram or {"mul_prev": 0, "mul_cur": 0}
        lowp = self.cfg.dtype != torch.float32
        x, h = seqmix.embed_bigram(input_ids, self.embed, self.cfg.embedding_scale, self.pairs, big["mul_prev"], big["mul_cur"],
                                   states.layer(len(self.layers)).get("prev"), ctx.slots, ctx.lens, ctx.fresh, want_lowp=lowp)
        h = h if lowp else x
        for i, layer in enumerate(self.layers):
            x = layer(x, h, ctx, states.layer(layer.state_layer))
            if tap is not None:
                tap(i, x)
        ctx.scratch.clear()
        return x

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """Residual rows ``[n, width]`` float → float logits ``[n, vocab]`` (the embedding table is the output matrix)."""
        return F.linear(seqmix.rms_norm(rows, self.norm_weight, self.cfg.norm_eps, None, self.cfg.dtype), self.embed).float()


# --------------------------------------------------------------------------------------------------------------- checkpoint names
def convert_state_dict(cfg: NoresunConfig, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (``embed``, ``bigram``, ``l<i>.norm1|norm2``, ``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``,
    ``final.norm``; linear weights ``[out, in]``) → this module's parameters: the projections that read the mixer's input, the first
    residual gate among them, are stacked (missing biases are zeros), rotated rows of queries and keys are de-interleaved together
    with their norm weights, experts are stacked, and everything the kernels read as float is float."""
    W = cfg.width
    out: Dict[str, torch.Tensor] = {"embed": sd["embed"], "norm_weight": sd["final.norm"]}
    if cfg.bigram:
        out["pairs"] = sd["bigram"]
    for i, spec in enumerate(cfg.layers):
        p, o, m = f"l{i}.", f"layers.{i}.", spec["mixer"]
        x = lambda n: sd[p + "mix." + n]
        a = o + "mixer."
        out[o + "norm1.weight"] = sd[p + "norm1"]
        if spec["type"] == "mingru":
            R = int(m["width"])
            out[a + "in_proj"] = torch.cat([x("z"), x("x"), x("g"), sd[p + "rg1"]], 0)
            out[a + "in_bias"] = torch.cat([x("z.b").float(), x("x.b").float(), torch.zeros(R), sd[p + "rg1.b"].float()], 0)
            out[a + "o"] = x("o")
        elif spec["type"] == "attention":
            H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            dims = int((m.get("rot") or {}).get("dims", 0))
            iq, ik = deinterleave_index(H, D, 0, dims), deinterleave_index(G, D, 0, dims)
            own = m.get("kv_from") is None
            parts = [x("q")[iq]] + ([x("k")[ik], x("v")] if own else []) + [sd[p + "rg1"]]
            rows = GatedWindowAttention.stacked_rows(H, G if own else 0, D, V, False, W)
            stack = torch.cat(parts, 0)
            out[a + "in_proj"] = torch.cat([stack, stack.new_zeros(rows - stack.shape[0], stack.shape[1])], 0)
            bias = torch.zeros(rows)                                       # q, k, v have no biases; the gate's rows have one
            bias[stack.shape[0] - W:stack.shape[0]] = sd[p + "rg1.b"].float()
            out[a + "in_bias"] = bias
            out[a + "q_norm"] = x("q.norm")[iq]
            if own:
                out[a + "k_norm"] = x("k.norm")[ik]
            out[a + "score_bias"], out[a + "o"] = x("pb"), x("o")
        f = spec.get("mlp")
        if not f:
            continue
        out[o + "norm2.weight"] = sd[p + "norm2"]
        out[o + "gate2"], out[o + "gate2_bias"] = sd[p + "rg2"], sd[p + "rg2.b"]
        y = lambda n: sd[p + "mlp." + n]
        E = int(f["router"]["experts"])
        out[o + "mlp.router.linear_router.weight"], out[o + "mlp.router.linear_router.bias"] = y("router"), y("router.b")
        out[o + "mlp.up"] = torch.stack([y(f"e{e}.up") for e in range(E)], 0)
        out[o + "mlp.down"] = torch.stack([y(f"e{e}.down") for e in range(E)], 0)
    return out


def load_noresun_weights(model: NoresunForCausalLM, sd: Dict[str, torch.Tensor]) -> None:
    conv = convert_state_dict(model.cfg, sd)
    params = dict(model.named_parameters())
    missing, extra = sorted(set(params) - set(conv)), sorted(set(conv) - set(params))
    if missing or extra:
        raise KeyError(f"checkpoint does not fit the model: missing {missing[:6]}, unexpected {extra[:6]}")
    with torch.no_grad():
        for k, v in conv.items():
            if tuple(params[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != {tuple(params[k].shape)}")
            params[k].copy_(v.to(params[k].dtype))


# ------------------------------------------------------------------------------------------------------------------------ serving
class NoresunForInference(SlotServingModel):
    def __init__(self, cfg: NoresunConfig, batch_size: int = 1, max_seq_len: int = 2048, on_device_sampling: bool = True,
                 sampler: Optional[Sampler] = None):
        super().__init__(cfg, NoresunForCausalLM(cfg, max_seq_len=max_seq_len), batch_size=batch_size, max_seq_len=max_seq_len,
                         on_device_sampling=on_device_sampling, sampler=sampler)

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "NoresunForInference":
        from ..utils.safetensors_utils import load_state_dict_safetensors

        sd = load_state_dict_safetensors(os.path.join(path, "model.safetensors"))
        model = cls(NoresunConfig.from_pretrained(path, dtype=dtype, device=device), **kw)
        load_noresun_weights(model.lm, sd)
        return model.eval()

    def load_checkpoint_tensors(self, sd) -> None:
        load_noresun_weights(self.lm, sd)
