"""Pulenex: a decoder-only language model that mixes three kinds of sequence mixer — latent sliding-window attention with direct
queries, a sigmoid gate per head and optional borrowing of another layer's cached latents (``modules/attention/latent_attention.py``),
retention (``modules/recurrent/retention.py``), and a pair side by side: chunked softmax attention whose heads' scores are mixed
before a softmax with a sink (``modules/attention/headmix_attention.py``) next to a gated delta rule with a decay per key channel
(``modules/recurrent/delta_rule.py``), each RMS-normed over the width and averaged (``modules/parallel_mixers.py``) — with a dense
clamped gated feed-forward (``modules/gated_ffn.py``) or none.

Block shape: a layer norm (gain, no bias) on both sides of every sublayer, ``x += norm1b(mixer(norm1(x)))`` then
``x += norm2b(ff(norm2(x)))``.  The residual stream ``x`` is float; the sublayers compute in the model dtype, and everything that
enters a recurrence, a score or a norm's statistics is float.  ``config.json`` lists the layers in order (``type``, ``mixer`` sizes,
``mlp`` or null), so any order and any sizes load without code changes.  Rotations pair neighbouring coordinates in the checkpoint;
the projections are reordered at load so that the kernels pair the two halves of the rotated stretch.

Serving is the slot-based wrapper shared with the other stateful families (``inference/slot_serving.py``)."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from ..inference.slot_serving import SlotServingModel
from ..inference.state_cache import SequenceStateManager, StepContext
from ..modules.attention.headmix_attention import HeadMixAttention
from ..modules.attention.latent_attention import LatentWindowAttention
from ..modules.attention.utils import deinterleave_index, deinterleave_rows
from ..modules.gated_ffn import ClampedGatedFFN
from ..modules.parallel_mixers import NormedParallelMixers
from ..modules.recurrent import GatedDeltaRule, Retention
from ..modules.rms_norm import GainOnlyLayerNorm
from ..utils.sampling import Sampler

GATE_SLOPE = 1.702          # the feed-forward's gate is g * sigmoid(1.702 g)


@dataclasses.dataclass
class PulenexConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]                    # [{"type", "mixer": {...}, "mlp": {...} | None}, ...] as in config.json
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    dtype: torch.dtype = torch.bfloat16
    device: Any = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **overrides) -> "PulenexConfig":
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), layers=list(d["layers"]), norm_eps=float(d["norm"]["eps"]),
                   logit_scale=float(d.get("logit_scale", 1.0)), **overrides)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "PulenexConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f), **overrides)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _latent_key(owner: int):
    return ("latent", owner)


def _build_mixer(cfg: PulenexConfig, index: int, max_seq_len: int) -> nn.Module:
    spec = cfg.layers[index]
    m, kind = spec["mixer"], spec["type"]
    if kind == "latent_attention":
        borrowers = [s["mixer"] for s in cfg.layers if s["type"] == "latent_attention" and s["mixer"].get("kv_from") == index]
        shares = m.get("kv_from") is not None
        if shares:
            owner = cfg.layers[int(m["kv_from"])]
            if owner["type"] != "latent_attention" or owner["mixer"].get("kv_from") is not None or int(m["kv_from"]) >= index:
                raise ValueError(f"layer {index} borrows keys from layer {m['kv_from']}, which keeps none of its own before it")
        return LatentWindowAttention(cfg.width, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), 0,
                                     window=int(m["mask"]["size"]), scale=float(m["scale"]), rot_base=float(m["rot"]["base"]),
                                     rot_dims=int(m["rot"]["dims"]), eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device,
                                     max_seq_len=max_seq_len, head_gate=True, shares_kv=shares,
                                     kv_key=_latent_key(int(m["kv_from"])) if shares else (_latent_key(index) if borrowers else None),
                                     ring_window=max([int(b["mask"]["size"]) for b in borrowers], default=0))
    if kind == "retention":
        return Retention(cfg.width, int(m["heads"]), int(m["dim"]), int(m["vdim"]), [float(d) for d in m["decay"]],
                         rot_base=float(m["rot"]["base"]), rot_dims=int(m["rot"]["dims"]), eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device)
    if kind == "parallel":
        l, r = m["left"], m["right"]
        if int(l["vdim"]) != int(l["dim"]):
            raise ValueError("the attention branch's values are its keys: vdim must equal dim")
        left = HeadMixAttention(cfg.width, int(l["heads"]), int(l["kv_heads"]), int(l["dim"]), int(l["conv"]), scale=float(l["scale"]),
                                rot_base=float(l["rot"]["base"]), rot_dims=int(l["rot"]["dims"]), chunk=int(l["mask"]["size"]),
                                dtype=cfg.dtype, device=cfg.device, max_seq_len=max_seq_len)
        right = GatedDeltaRule(cfg.width, int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r["conv"]),
                               eps=cfg.norm_eps, dtype=cfg.dtype, device=cfg.device, channel_decay=True, decay_rank=int(r["decay_rank"]),
                               gate_rank=int(r["gate_rank"]), gate_act="sigmoid")
        return NormedParallelMixers({"left": left, "right": right}, [0.5, 0.5], cfg.width, cfg.norm_eps, cfg.device)
    raise ValueError(f"unknown mixer type {kind!r}")


def _build_ffn(cfg: PulenexConfig, f: Optional[Dict[str, Any]]) -> Optional[nn.Module]:
    if not f:
        return None
    if f["kind"] == "dense":
        return ClampedGatedFFN(cfg.width, int(f["ff"]), float(f["limit"]), GATE_SLOPE, bias=True, dtype=cfg.dtype, device=cfg.device)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


class PulenexLayer(nn.Module):
    def __init__(self, cfg: PulenexConfig, index: int, max_seq_len: int):
        super().__init__()
        spec = cfg.layers[index]
        self.kind, self.dtype = spec["type"], cfg.dtype
        src = spec["mixer"].get("kv_from") if spec["type"] == "latent_attention" else None
        self.state_layer = index if src is None else int(src)           # whose state entries the mixer reads and writes
        mk = lambda: GainOnlyLayerNorm(cfg.width, cfg.norm_eps, cfg.device)
        self.norm1, self.norm1b = mk(), mk()
        self.mixer = _build_mixer(cfg, index, max_seq_len)
        self.mlp = _build_ffn(cfg, spec.get("mlp"))
        if self.mlp is not None:
            self.norm2, self.norm2b = mk(), mk()

    def state_spec(self):
        return self.mixer.state_spec()

    def forward(self, x: torch.Tensor, ctx: StepContext, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        """``x [B,S,width]`` float residual stream, updated in place."""
        B, S, W = x.shape
        self.norm1b.add_to(x, self.mixer(self.norm1(x, out_dtype=self.dtype), ctx, st))
        if self.mlp is not None:
            self.norm2b.add_to(x, self.mlp(self.norm2(x, out_dtype=self.dtype).view(B * S, W)))
        return x


class PulenexForCausalLM(nn.Module):
    def __init__(self, cfg: PulenexConfig, max_seq_len: int = 1 << 30):
        super().__init__()
        self.cfg = self.config = cfg
        self.embed = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)
        self.layers = nn.ModuleList([PulenexLayer(cfg, i, max_seq_len) for i in range(len(cfg.layers))])
        self.norm = GainOnlyLayerNorm(cfg.width, cfg.norm_eps, cfg.device)
        self.head = nn.Parameter(torch.zeros(cfg.vocab, cfg.width, dtype=cfg.dtype, device=cfg.device), requires_grad=False)

    def state_specs(self):
        return [layer.state_spec() for layer in self.layers]

    def body(self, input_ids: torch.Tensor, ctx: StepContext, states: SequenceStateManager, tap=None) -> torch.Tensor:
        x = F.embedding(input_ids, self.embed).float()
        for i, layer in enumerate(self.layers):
            x = layer(x, ctx, states.layer(layer.state_layer))
            if tap is not None:
                tap(i, x)
        ctx.scratch.clear()
        return x

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """Residual rows ``[n, width]`` float → float logits ``[n, vocab]``."""
        return F.linear(self.norm(rows, out_dtype=self.cfg.dtype), self.head).float() * self.cfg.logit_scale


# --------------------------------------------------------------------------------------------------------------- checkpoint names
def convert_state_dict(cfg: PulenexConfig, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``;
    linear weights ``[out, in]``) → this module's parameters: projections that read the same input are stacked, the convolutions of
    one mixer are stacked, per-head matrices get a head axis, rotated rows are de-interleaved (and with them, where the values are
    the keys, the gate's rows and the output projection's columns), and everything the kernels read as float is float.  Branch
    gains are returned under ``*.gain`` keys and scaled by the loader."""
    out: Dict[str, torch.Tensor] = {"embed": sd["embed"], "head": sd["head"], "norm.weight": sd["final.norm"]}
    for i, spec in enumerate(cfg.layers):
        p, o, m = f"l{i}.", f"layers.{i}.", spec["mixer"]
        out[o + "norm1.weight"], out[o + "norm1b.weight"] = sd[p + "norm1"], sd[p + "norm1b"]
        x = lambda n: sd[p + "mix." + n]
        a = o + "mixer."
        if spec["type"] == "latent_attention":
            H, D, R, C, dims = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["kv_rank"]), int(m["rot"]["dims"])
            out[a + "q_proj"] = deinterleave_rows(x("q"), H, D + R, D, dims)
            if m.get("kv_from") is None:
                out[a + "dkv"], out[a + "dkv_norm"] = deinterleave_rows(x("dkv"), 1, C + R, C, dims), x("dkv.norm")
            out[a + "uk"], out[a + "uv"] = x("uk").view(H, D, C), x("uv").view(H, int(m["vdim"]), C)
            out[a + "head_gate"], out[a + "o"] = x("g"), x("o")
        elif spec["type"] == "retention":
            out[a + "in_proj"], out[a + "o"] = torch.cat([x("q"), x("k"), x("v"), x("g")], 0), x("o")
        elif spec["type"] == "parallel":
            l, b = a + "branches.left.", a + "branches.right."
            ml = m["left"]
            H, G, D, dims = int(ml["heads"]), int(ml["kv_heads"]), int(ml["dim"]), int(ml["rot"]["dims"])
            iq, ik = deinterleave_index(H, D, 0, dims), deinterleave_index(G, D, 0, dims)
            out[l + "in_proj"] = torch.cat([x("left.q")[iq], x("left.k")[ik], x("left.g")[iq]], 0)
            out[l + "conv.weight"] = torch.cat([x("left.q.conv")[iq], x("left.k.conv")[ik]], 0)
            out[l + "talk"], out[l + "temp"], out[l + "sink"] = x("left.talk"), x("left.temp"), x("left.sink")
            out[l + "o"] = x("left.o")[:, iq]
            out[b + "in_proj"] = torch.cat([x("right.q"), x("right.k"), x("right.v"), x("right.g1"), x("right.a1")], 0)
            out[b + "ba_proj"], out[b + "gate_up"], out[b + "decay_up"] = x("right.b"), x("right.g2"), x("right.a2")
            out[b + "conv.weight"] = torch.cat([x("right.q.conv"), x("right.k.conv"), x("right.v.conv")], 0)
            out[b + "a_log"], out[b + "dt_bias"] = x("right.A_log"), x("right.dt_bias")
            out[b + "norm"], out[b + "o"] = x("right.norm"), x("right.o")
            out[a + "out_norms.left.gain"], out[a + "out_norms.right.gain"] = x("left.out"), x("right.out")
        f = spec.get("mlp")
        if not f:
            continue
        out[o + "norm2.weight"], out[o + "norm2b.weight"] = sd[p + "norm2"], sd[p + "norm2b"]
        y = lambda n: sd[p + "mlp." + n]
        out[o + "mlp.up"], out[o + "mlp.up_bias"] = torch.cat([y("gate"), y("up")], 0), torch.cat([y("gate.b"), y("up.b")], 0)
        out[o + "mlp.down"], out[o + "mlp.down_bias"] = y("down"), y("down.b")
    return out


def complete_config(d: Dict[str, Any], shapes: Dict[str, Sequence[int]]) -> Dict[str, Any]:
    """Sizes that ``config.json`` leaves to the tensors' shapes: the ranks of the delta rule's low-rank decay and gate projections,
    and the taps of the short convolutions when they are not listed."""
    d = json.loads(json.dumps(d))
    for i, spec in enumerate(d["layers"]):
        if spec["type"] != "parallel":
            continue
        l, r = spec["mixer"]["left"], spec["mixer"]["right"]
        r.setdefault("decay_rank", int(shapes[f"l{i}.mix.right.a1"][0]))
        r.setdefault("gate_rank", int(shapes[f"l{i}.mix.right.g1"][0]))
        r.setdefault("conv", int(shapes[f"l{i}.mix.right.q.conv"][1]))
        l.setdefault("conv", int(shapes[f"l{i}.mix.left.q.conv"][1]))
    return d


def load_pulenex_weights(model: PulenexForCausalLM, sd: Dict[str, torch.Tensor]) -> None:
    conv = convert_state_dict(model.cfg, sd)
    gains = {k[: -len(".gain")]: conv.pop(k) for k in [k for k in conv if k.endswith(".gain")]}
    params = dict(model.named_parameters())
    have = set(conv) | set(gains)
    missing, extra = sorted(set(params) - have), sorted(have - set(params))
    if missing or extra:
        raise KeyError(f"checkpoint does not fit the model: missing {missing[:6]}, unexpected {extra[:6]}")
    with torch.no_grad():
        for k, v in conv.items():
            if tuple(params[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != {tuple(params[k].shape)}")
            params[k].copy_(v.to(params[k].dtype))
        for k, v in gains.items():
            mixer, _, name = k.rpartition(".out_norms.")
            model.get_submodule(mixer).set_gain(name, v)


# ------------------------------------------------------------------------------------------------------------------------ serving
class PulenexForInference(SlotServingModel):
    def __init__(self, cfg: PulenexConfig, batch_size: int = 1, max_seq_len: int = 2048, on_device_sampling: bool = True,
                 sampler: Optional[Sampler] = None):
        super().__init__(cfg, PulenexForCausalLM(cfg, max_seq_len=max_seq_len), batch_size=batch_size, max_seq_len=max_seq_len,
                         on_device_sampling=on_device_sampling, sampler=sampler)

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "PulenexForInference":
        from ..utils.safetensors_utils import load_state_dict_safetensors

        sd = load_state_dict_safetensors(os.path.join(path, "model.safetensors"))
        with open(os.path.join(path, "config.json")) as f:
            d = complete_config(json.load(f), {k: tuple(v.shape) for k, v in sd.items()})
        model = cls(PulenexConfig.from_dict(d, dtype=dtype, device=device), **kw)
        load_pulenex_weights(model.lm, sd)
        return model.eval()

    def load_checkpoint_tensors(self, sd) -> None:
        load_pulenex_weights(self.lm, sd)
