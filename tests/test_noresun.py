"""Noresun serving path against the plain oracle (tests/noresun_oracle.py): every mechanism alone, whole prompts, prompt + token by
token decoding, unequal batches, reused slots, window edges in prompts and in decoding, borrowed keys, far tokens through the
recurrent state, the first tokens, long decoding, other sizes, greedy generation through the serving entry points, the registry /
checkpoint reader, the trace runner and the generation command line.  Configurations and weights are made here (random, seeded)."""
import io
import json
import math
import os
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import noresun_oracle as oracle  # noqa: E402

from neuronx_distributed_b200.inference.hf_adapter import HuggingFaceGenerationAdapter  # noqa: E402
from neuronx_distributed_b200.inference.trace_replay import TraceReplayer  # noqa: E402
from neuronx_distributed_b200.models import registry  # noqa: E402
from neuronx_distributed_b200.models.noresun import NoresunConfig, NoresunForInference, load_noresun_weights  # noqa: E402
from neuronx_distributed_b200.modules.attention.utils import deinterleave_index  # noqa: E402
from neuronx_distributed_b200.ops import seqmix  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
TOL32 = 2e-4
F64 = torch.float64


# ------------------------------------------------------------------------------------------------------------------ model making
def moe(ff=24, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def gru(width=40, mlp="default"):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": moe() if mlp == "default" else mlp}


def attn(heads=4, kv_heads=2, dim=16, vdim=24, window=7, dims=8, base=5000.0, scaling=None, scale=None, kv_from=None, mlp="default"):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


SCALING = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 24}


def make_cfg(layers, vocab=50, width=48, eps=1e-5, alpha=1.7, scale=3.0, bigram=(37, 5, 11)):
    e = {"scale": scale}
    if bigram:
        e["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Noresun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "embedding": e, "layers": layers}


def random_checkpoint(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.to(torch.bfloat16).float()
    lin = lambda o, i, s=1.0: bf(torch.randn(o, i, generator=g) * s / math.sqrt(i))
    vec = lambda n, s=1.0, m=0.0: bf(torch.randn(n, generator=g) * s + m)
    W, w = cfg["width"], {}
    w["embed"], w["final.norm"] = bf(torch.randn(cfg["vocab"], W, generator=g) * 0.5), vec(W, 0.2, 1.0)
    big = cfg["embedding"].get("bigram")
    if big:
        w["bigram"] = bf(torch.randn(big["buckets"] + 1, W, generator=g))
    for i, L in enumerate(cfg["layers"]):
        p, m, q = f"l{i}.", L["mixer"], f"l{i}.mix."
        w[p + "norm1"], w[p + "rg1"], w[p + "rg1.b"] = vec(W, 0.2, 1.0), lin(W, W, 2.0), vec(W, 0.5)
        if L["type"] == "mingru":
            R = m["width"]
            w.update({q + "z": lin(R, W, 2.0), q + "z.b": vec(R, 0.5), q + "x": lin(R, W, 2.0), q + "x.b": vec(R, 0.5), q + "g": lin(R, W, 2.0),
                      q + "o": lin(W, R)})
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w.update({q + "q": lin(H * D, W, 2.0), q + "q.norm": vec(H * D, 0.3, 1.0), q + "pb": vec(H, 1.0, -1.0), q + "o": lin(W, H * V)})
            if m.get("kv_from") is None:
                w.update({q + "k": lin(G * D, W, 2.0), q + "k.norm": vec(G * D, 0.3, 1.0), q + "v": lin(G * V, W, 2.0)})
        f = L.get("mlp")
        if not f:
            continue
        w[p + "norm2"], w[p + "rg2"], w[p + "rg2.b"] = vec(W, 0.2, 1.0), lin(W, W, 2.0), vec(W, 0.5)
        y, E = p + "mlp.", f["router"]["experts"]
        w[y + "router"], w[y + "router.b"] = lin(E, W, 4.0), vec(E, 0.5)
        for e in range(E):
            w[y + f"e{e}.up"], w[y + f"e{e}.down"] = lin(f["expert"]["ff"], W, 2.0), lin(W, f["expert"]["ff"])
    return w


def build(cfg, weights, device, dtype=torch.float32, max_seq_len=4096, batch_size=1):
    m = NoresunForInference(NoresunConfig.from_dict(cfg, dtype=dtype, device=torch.device(device)), batch_size=batch_size, max_seq_len=max_seq_len,
                            on_device_sampling=False)
    load_noresun_weights(m.lm, weights)
    return m.eval()


def tokens_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_cut(model, toks, prompt):
    """Prompt of ``prompt`` tokens in one step, the rest one by one → logits at every position [S, vocab] (float, cpu)."""
    mgr = model.states
    slot = mgr.alloc()
    dev = next(model.parameters()).device
    x = model.forward_step(torch.tensor([toks[:prompt]], device=dev), [prompt], [slot], [0], True)
    mgr.advance([slot], [prompt])
    out = [model.logits(x[0])]
    for p in range(prompt, len(toks)):
        x = model.forward_step(torch.tensor([[toks[p]]], device=dev), [1], [slot], [p], False)
        mgr.advance([slot], [1])
        out.append(model.logits(x[0]))
    mgr.free(slot)
    return torch.cat(out).cpu()


def close(got, want, tol):
    """Mean-free difference relative to the spread of the expected values, per position."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = (want - want.mean(-1, keepdim=True)).double().pow(2).mean().sqrt()
    err = (d.pow(2).mean(-1).sqrt() / ref).max().item()
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def i32(v, device):
    return torch.tensor(v, dtype=torch.int32, device=device)


# ------------------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rows,C,gated", [(7, 48, True), (3, 37, True), (300, 64, False), (2, 1024, True), (5, 1030, True), (1200, 2048, True),
                                          (1190, 2304, True), (3, 8192, True), (2, 20480, False)])
def test_norm_after_the_gated_residual_sum(device, rows, C, gated):
    g = torch.Generator().manual_seed(rows + C)
    x, y, gate = (torch.randn(rows, C, generator=g) for _ in range(3))
    w = torch.randn(C, generator=g)
    alpha, eps = 2.25, 1e-5
    v = alpha * x.double() + (torch.sigmoid(gate.double()) if gated else 1.0) * y.double()
    want = oracle.rms(v, w.double(), eps)
    xs = x.clone().to(device)
    both = torch.cat([y, gate], 1).to(device)                         # views into one buffer, as a stacked projection gives them
    seqmix.postnorm_gated_(xs, both[:, :C], both[:, C:] if gated else None, w.to(device), alpha, eps)
    assert (xs.cpu().double() - want).abs().max() < 1e-5
    if device == "cuda":
        xs, low = x.clone().to(device), torch.empty(rows, C, dtype=torch.bfloat16, device=device)
        yb, gb = y.to(device).bfloat16(), gate.to(device).bfloat16()
        seqmix.postnorm_gated_(xs, yb, gb if gated else None, w.to(device), alpha, eps, low)
        v = alpha * x.double() + (torch.sigmoid(gb.cpu().double()) if gated else 1.0) * yb.cpu().double()
        assert (xs.cpu().double() - oracle.rms(v, w.double(), eps)).abs().max() < 1e-5
        assert torch.equal(low, xs.bfloat16())


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("W,buckets,pairs", [(48, 37, True), (33, 2, True), (64, 7, False)])
def test_pair_hash_embedding_and_the_carried_token(device, W, buckets, pairs):
    g = torch.Generator().manual_seed(W)
    vocab, scale, mp, mc = 29, 2.5, 7, 13
    table = torch.randn(vocab, W, generator=g)
    pt = torch.randn(buckets + 1, W, generator=g) if pairs else None
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (9, 4, 1)]

    def want(s):
        x = table.double()[s] * scale
        return x + pt.double()[oracle.pair_rows(s, buckets, mp, mc)] if pairs else x

    prev = torch.full((6,), 17, dtype=torch.int64, device=device)     # slots hold leftovers of earlier sequences
    slots, cut = [4, 1, 5], [5, 3, 1]
    ids = torch.zeros(3, 5, dtype=torch.long)
    for b, s in enumerate(seqs):
        ids[b, :cut[b]] = torch.tensor(s[:cut[b]])
    out, _ = seqmix.embed_bigram(ids.to(device), table.to(device), scale, None if pt is None else pt.to(device), mp, mc, prev, i32(slots, device),
                                 i32(cut, device), True)
    for b, s in enumerate(seqs):
        assert (out[b, :cut[b]].cpu().double() - want(s)[:cut[b]]).abs().max() < 1e-5
    assert prev.cpu().tolist() == [17, seqs[1][2], 17, 17, seqs[0][4], seqs[2][0]]
    for t in range(5, 9):                                             # row 0 goes on one token at a time; row 1 too, while it lasts
        live = [b for b in (0, 1) if t - 5 + cut[b] < len(seqs[b])]
        step = torch.tensor([[seqs[b][t - 5 + cut[b]]] for b in live])
        out, _ = seqmix.embed_bigram(step.to(device), table.to(device), scale, None if pt is None else pt.to(device), mp, mc, prev,
                                     i32([slots[b] for b in live], device), i32([1] * len(live), device), False)
        for j, b in enumerate(live):
            assert (out[j, 0].cpu().double() - want(seqs[b])[t - 5 + cut[b]]).abs().max() < 1e-5


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("W,S", [(40, 21), (64, 150), (33, 1), (70, 700), (40, 2100)])
def test_mingru_scan_rows_of_many_lengths_and_a_carried_state(device, W, S):
    g = torch.Generator().manual_seed(W + S)
    B = 3
    p = torch.randn(B, S, 3 * W + 5, generator=g) * 2.0               # z | u | gate inside a wider projection
    lens = [S, max(1, S // 3), max(1, S - 1)]
    z, u, gt = p[..., :W].double(), p[..., W:2 * W].double(), p[..., 2 * W:3 * W].double()

    def want(b, n, s0):
        s, rows = s0.clone(), []
        for t in range(n):
            zz = torch.sigmoid(z[b, t])
            s = (1 - zz) * s + zz * torch.where(u[b, t] >= 0, u[b, t] + 0.5, torch.sigmoid(u[b, t]))
            rows.append(s * gt[b, t] * torch.sigmoid(gt[b, t]))
        return torch.stack(rows), s

    state = torch.randn(5, W, generator=g).to(device)                 # leftovers that a fresh call must ignore
    slots = [3, 0, 4]
    pd = p.to(device)
    out = seqmix.mingru_scan(pd[..., :W], pd[..., W:2 * W], pd[..., 2 * W:3 * W], state, i32(slots, device), i32(lens, device), True)
    ends = []
    for b in range(B):
        rows, s = want(b, lens[b], torch.zeros(W, dtype=F64))
        ends.append(s)
        assert (out[b, :lens[b]].cpu().double() - rows).abs().max() < 2e-5
        assert (out[b, lens[b]:] == 0).all()
        assert (state[slots[b]].cpu().double() - s).abs().max() < 2e-5
    out = seqmix.mingru_scan(pd[:, :1, :W], pd[:, :1, W:2 * W], pd[:, :1, 2 * W:3 * W], state, i32(slots, device), i32([1, 1, 0], device), False)
    for b in range(2):
        rows, s = want(b, 1, ends[b])
        assert (out[b, 0].cpu().double() - rows[0]).abs().max() < 2e-5 and (state[slots[b]].cpu().double() - s).abs().max() < 2e-5
    assert (state[slots[2]].cpu().double() - ends[2]).abs().max() < 2e-5   # a row without tokens leaves its state alone


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("N,E,top", [(5, 7, 3), (40, 5, 1), (3, 4, 4), (70, 33, 2), (9, 40, 35)])
def test_router_softmax_over_the_chosen_logits(device, N, E, top):
    logits = torch.randn(N, E, generator=torch.Generator().manual_seed(N)) * 3
    w, idx, _ = seqmix.route_topk(logits.to(device), None, top, E, "softmax_top")
    val, want_idx = torch.topk(logits.double(), top, -1)
    assert torch.equal(idx.cpu(), want_idx)
    assert (w.cpu().double() - torch.softmax(val, -1)).abs().max() < 1e-6


@pytest.mark.parametrize("device", DEVICES)
def test_squared_relu_alone_and_in_the_indexed_products(device):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 33, generator=g)
    assert (seqmix.relu_sq(x.to(device)).cpu() - torch.relu(x) ** 2).abs().max() < 1e-6
    w, sel = torch.randn(4, 10, 33, generator=g), torch.tensor([2, 0, 3, 3, 1, 2, 0], dtype=torch.int32)
    got = seqmix.indexed_gemv(w.to(device), sel.to(device), x.to(device), "relu_sq").cpu()
    want = torch.relu(torch.einsum("moi,mi->mo", w[sel.long()].double(), x.double())) ** 2
    assert (got.double() - want).abs().max() < 1e-4


def test_rescaled_rotation_frequencies():
    for dims, base, sc in [(8, 5000.0, SCALING), (16, 100.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}), (4, 10.0, None)]:
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = sc
        want = torch.tensor(oracle.frequencies(rot), dtype=F64)
        got = seqmix.rotary_inv_freq(dims, base, None, sc).double()
        assert ((got - want).abs() / want).max() < 1e-6
        if sc:                                                        # the three regimes are all there
            plain = torch.tensor(oracle.frequencies({"dims": dims, "base": base}), dtype=F64)
            ratio = want / plain
            assert (ratio == 1).any() and ((ratio - 1 / sc["factor"]).abs() < 1e-12).any()


def _attention_case(H, G, D, V, window, dims, S, seed, scaling=None):
    g = torch.Generator().manual_seed(seed)
    m = attn(H, G, D, V, window, dims, 300.0, scaling)["mixer"]
    W = 24
    w = {"q": torch.randn(H * D, W, generator=g), "k": torch.randn(G * D, W, generator=g), "v": torch.randn(G * V, W, generator=g),
         "q.norm": torch.randn(H * D, generator=g) * 0.3 + 1, "k.norm": torch.randn(G * D, generator=g) * 0.3 + 1, "pb": torch.randn(H, generator=g) - 1,
         "o": torch.eye(H * V)}
    h = torch.randn(S, W, generator=g, dtype=F64)
    k, v = oracle.attention_keys(m, w, "", h, 1e-5)
    return m, w, h, oracle.sigmoid_window_attention(m, w, "", h, 1e-5, k, v)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,D,V,window,dims", [(4, 2, 16, 24, 7, 8), (6, 1, 32, 16, 20, 32), (2, 2, 10, 5, 3, 4), (3, 3, 64, 64, 100, 16),
                                                 (8, 2, 16, 16, 1, 2), (2, 1, 12, 40, 9, 0)])
def test_sigmoid_window_attention_prompt_and_ring(device, H, G, D, V, window, dims):
    """Whole-projection norms, rotation (neighbour pairs in the oracle, halves after the load-time reordering here), the ring store,
    independent sigmoid weights with a bias per head: a prompt in one call, then the same tokens one by one against the ring."""
    S = 23
    m, w, h, want = _attention_case(H, G, D, V, window, dims, S, H * 100 + D, SCALING if dims >= 8 else None)
    iq, ik = deinterleave_index(H, D, 0, dims), deinterleave_index(G, D, 0, dims)
    dv = lambda t: t.float().to(device)
    q0 = (h @ w["q"].double().T)[:, iq].view(1, S, H, D)
    k0 = (h @ w["k"].double().T)[:, ik].view(1, S, G, D)
    v0 = (h @ w["v"].double().T).view(1, S, G, V)
    qw, kw, pb = dv(w["q.norm"][iq]), dv(w["k.norm"][ik]), dv(w["pb"])
    inv = seqmix.rotary_inv_freq(dims, 300.0, device, m["rot"].get("scaling")) if dims else None
    ring = window
    kc, vc = torch.full((3, ring, G, D), 9.0, device=device), torch.full((3, ring, G, V), 9.0, device=device)
    q, k, v = dv(q0), dv(k0), dv(v0)
    one, slot = i32([S], device), i32([2], device)
    seqmix.window_qk_prepare(q, k, v, qw, kw, 1e-5, i32([0], device), one, slot, kc, vc, norm_all=True, inv_freq=inv, rot_dims=dims)
    out = torch.empty(S, H * V, device=device)
    seqmix.window_attention_prompt(q, k, v, None, one, window, m["scale"], 0.0, out, 1.0, pb)
    assert (out.cpu().double() - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    kc.fill_(9.0), vc.fill_(9.0)
    for t in range(S):
        q, k, v = dv(q0[:, t:t + 1]), dv(k0[:, t:t + 1]), dv(v0[:, t:t + 1])
        seqmix.window_qk_prepare(q, k, v, qw, kw, 1e-5, i32([t], device), i32([1], device), slot, kc, vc, norm_all=True, inv_freq=inv, rot_dims=dims)
        o1 = torch.empty(1, H * V, device=device)
        seqmix.window_attention_token(q, kc, vc, None, slot, i32([t], device), i32([1], device), window, m["scale"], 0.0, o1, 1.0, pb)
        assert (o1[0].cpu().double() - want[t]).abs().max() < 2e-4 * max(1.0, want.abs().max().item()), t


@pytest.mark.parametrize("device", DEVICES)
def test_softmax_window_attention_is_unchanged_by_the_new_options(device):
    """The softmax form with a norm per head and no rotation (what the older family uses) through the same entry points."""
    g = torch.Generator().manual_seed(5)
    H, G, D, V, S, window = 4, 2, 16, 8, 19, 6
    q, k, v = torch.randn(1, S, H, D, generator=g), torch.randn(1, S, G, D, generator=g), torch.randn(1, S, G, V, generator=g)
    qw, kw = torch.rand(D, generator=g) + 0.5, torch.rand(D, generator=g) + 0.5
    qn, kn = oracle.rms(q.double(), qw.double(), 1e-5), oracle.rms(k.double(), kw.double(), 1e-5)
    sc = torch.einsum("ihd,jhd->hij", qn[0], kn[0].repeat_interleave(2, 1)) * 0.3
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    p = torch.softmax(sc.masked_fill(~((j <= i) & (j > i - window)), float("-inf")), -1)
    want = torch.einsum("hij,jhv->ihv", p, v[0].double().repeat_interleave(2, 1)).reshape(S, H * V)
    kc, vc = torch.zeros(1, window, G, D, device=device), torch.zeros(1, window, G, V, device=device)
    qd, kd, vd = q.to(device), k.to(device), v.to(device)
    seqmix.window_qk_prepare(qd, kd, vd, qw.to(device), kw.to(device), 1e-5, i32([0], device), i32([S], device), i32([0], device), kc, vc)
    out = torch.empty(S, H * V, device=device)
    seqmix.window_attention_prompt(qd, kd, vd, None, i32([S], device), window, 0.3, 0.0, out)
    assert (out.cpu().double() - want).abs().max() < 1e-4


# ------------------------------------------------------------------------------------------------------------------ whole models
SINGLE = {
    "mingru": [gru()],
    "mingru_bare": [gru(width=48, mlp=None)],
    "attention": [attn()],
    "attention_scaled_rotation": [attn(dims=16, scaling=SCALING, mlp=None)],
    "attention_one_key_head": [attn(heads=5, kv_heads=1, dim=8, vdim=8, window=5, dims=4, mlp=moe(top=1))],
    "attention_every_head_its_keys": [attn(heads=3, kv_heads=3, dim=12, vdim=20, window=40, dims=12, mlp=moe(experts=3, top=3))],
    "attention_no_rotation": [attn(dims=0, window=1, mlp=None)],
}
MIXED = [gru(), attn(window=9), gru(width=24, mlp=None), attn(heads=2, window=5, kv_from=1, scale=0.4), attn(heads=2, kv_heads=1, dim=8, vdim=8, window=6, dims=8),
         attn(heads=4, window=12, kv_from=1, mlp=moe(ff=16, experts=4, top=3))]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_single_layer_models(device, name):
    cfg = make_cfg(SINGLE[name], bigram=None if name == "mingru_bare" else (37, 5, 11), alpha=1.0 if name == "attention" else 1.7)
    w = random_checkpoint(cfg, seed=len(name))
    toks = tokens_for(cfg, 30, 5)
    want = oracle.forward(cfg, w, toks)
    close(run_cut(build(cfg, w, device), toks, 30), want, TOL32)
    close(run_cut(build(cfg, w, device), toks, 11), want, TOL32)


@pytest.fixture(scope="module")
def mixed():
    cfg = make_cfg(MIXED)
    w = random_checkpoint(cfg, seed=11)
    toks = tokens_for(cfg, 48, 7)
    stream = []
    want = oracle.forward(cfg, w, toks, taps=stream)
    return cfg, w, toks, want, stream


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [48, 1, 2, 6, 31])
def test_prompt_then_decode_matches_oracle(device, mixed, prompt):
    cfg, w, toks, want, _ = mixed
    close(run_cut(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_residual_stream_after_every_layer(device, mixed):
    cfg, w, toks, _, stream = mixed
    model = build(cfg, w, device)
    seen = {}
    model.forward_step(torch.tensor([toks], device=device), [len(toks)], [model.states.alloc()], [0], True, tap=lambda i, x: seen.__setitem__(i, x[0].cpu().clone()))
    for i in range(len(MIXED)):
        close(seen[i], stream[i], TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_unequal_batch_against_each_alone_and_reused_slots(device, mixed):
    cfg, w, toks, _, _ = mixed
    model = build(cfg, w, device)
    reqs = [tokens_for(cfg, n, 20 + n) for n in (1 + 6, 7 + 6, 23 + 6, 2 + 6)]
    prompts, steps = [1, 7, 23, 2], [0, 6, 3, 6]                      # row 0 ends with its prompt, row 2 leaves early
    mgr = model.states
    warm = [mgr.alloc() for _ in range(3)]                            # dirty a few slots first, then give them back
    model.forward_step(torch.randint(0, 50, (3, 9), device=device), [9, 9, 9], warm, [0, 0, 0], True)
    for s in warm:
        mgr.free(s)
    slots = [mgr.alloc() for _ in reqs]
    assert set(warm) <= set(slots)
    S = max(prompts)
    ids = torch.zeros(len(reqs), S, dtype=torch.long)
    for b, (r, p) in enumerate(zip(reqs, prompts)):
        ids[b, :p] = torch.tensor(r[:p])
    x = model.forward_step(ids.to(device), prompts, slots, [0] * len(reqs), True)
    got = [[model.logits(x[b, :p]).cpu()] for b, p in enumerate(prompts)]
    live = [b for b in range(len(reqs)) if steps[b] > 0]
    mgr.free(slots[0])
    for k in range(max(steps)):
        live = [b for b in live if k < steps[b]]
        step_ids = torch.tensor([[reqs[b][prompts[b] + k]] for b in live], device=device)
        x = model.forward_step(step_ids, [1] * len(live), [slots[b] for b in live], [prompts[b] + k for b in live], False)
        lg = model.logits(x[:, 0]).cpu()
        for j, b in enumerate(live):
            got[b].append(lg[j:j + 1])
    for b, r in enumerate(reqs):
        n = prompts[b] + steps[b]
        close(torch.cat(got[b]), oracle.forward(cfg, w, r[:n]), TOL32)
    fresh = build(cfg, w, device)
    close(torch.cat(got[2]), run_cut(fresh, reqs[2][:26], 23), 1e-5)        # the batch changes nothing beyond rounding


# ------------------------------------------------------------------------------------- edges, far tokens, first tokens, long decoding
def _needle_model(layers, vocab=40, width=48, seed=3, **kw):
    """Token 0 is the needle: its embedding is large and unlike the others, so wherever a layer can still see it the logits move."""
    cfg = make_cfg(layers, vocab=vocab, width=width, **kw)
    w = random_checkpoint(cfg, seed=seed)
    w["embed"][0] = (w["embed"][0] * 12).to(torch.bfloat16).float()
    return cfg, w


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [40, 12, 1])
def test_window_edges_with_a_needle_and_borrowed_keys(device, prompt):
    """Attention only, no feed-forwards, no pair embedding: layer 0 (window 6) and layer 1, which borrows layer 0's keys and values
    with window 4.  They are made from layer 0's input, so the needle at position 9 is a key for 9..14 in layer 0 and for 9..12 in
    layer 1, and nothing moves from position 15 on.  Checked in a prompt, and with both borders passing over decoded tokens."""
    at = 9
    cfg, w = _needle_model([attn(window=6, mlp=None), attn(heads=2, window=4, kv_from=0, mlp=None)], bigram=None)
    toks = [1 + t % 7 for t in range(40)]
    plain = list(toks)
    toks[at] = 0
    want, base = oracle.forward(cfg, w, toks), oracle.forward(cfg, w, plain)
    moved = (want - base).abs().amax(-1)
    assert (moved[at:at + 6] > 1e-3).all() and (moved[at + 6:] < 1e-9).all() and (moved[:at] < 1e-9).all()
    close(run_cut(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [60, 30, 1])
def test_borrower_with_the_wider_window_and_one_loud_key(device, prompt):
    """The borrower's window (33) is wider than the lender's (5), so the lender's ring must keep 33 rows.  One key far back is made
    loud: the lender's query bias is very negative (its weights vanish), the borrower's is large only through that key, whose
    coordinates and the matching query coordinates are scaled up; a ring that is too short, or a window that is one off, loses it."""
    cfg, w = _needle_model([attn(heads=2, kv_heads=1, window=5, dims=4, mlp=None), attn(heads=2, kv_heads=1, window=33, dims=4, kv_from=0, mlp=None)], bigram=None)
    w["l1.mix.pb"] = torch.tensor([-6.0, -6.0])
    toks = [1 + t % 7 for t in range(60)]
    plain = list(toks)
    toks[20] = 0
    want, base = oracle.forward(cfg, w, toks), oracle.forward(cfg, w, plain)
    moved = (want - base).abs().amax(-1)
    assert (moved[20:53] > 1e-6).all() and (moved[53:] < 1e-9).all()
    model = build(cfg, w, device)
    assert model.states.layer(0)["k"].shape[1] == 33 and model.states.layer(1) == {}
    close(run_cut(model, toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("prompt", [300, 150, 2])
def test_far_token_through_the_recurrent_state(device, prompt):
    """minGRU only: the update gates' biases are very negative, so the state forgets slowly and a needle at position 3 still moves
    the logits hundreds of tokens later; a state that is dropped or reset between steps loses it."""
    cfg, w = _needle_model([gru(mlp=None)], bigram=None)
    w["l0.mix.z.b"] = torch.full_like(w["l0.mix.z.b"], -5.0)
    toks = [1 + t % 7 for t in range(300)]
    plain = list(toks)
    toks[3] = 0
    want, base = oracle.forward(cfg, w, toks), oracle.forward(cfg, w, plain)
    assert ((want - base).abs().amax(-1)[3:] > 1e-4).all()
    close(run_cut(build(cfg, w, device), toks, prompt), want, TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_first_tokens_and_the_pair_embedding_across_steps(device):
    """The pair table is made loud, so a wrong previous token (a prompt's last token not carried into decoding, the first token not
    taking the extra row, a reused slot's leftover) shows at once."""
    cfg = make_cfg([gru(mlp=None), attn(window=3, mlp=None)], bigram=(5, 3, 7))
    w = random_checkpoint(cfg, seed=4)
    w["bigram"] = (w["bigram"] * 6).to(torch.bfloat16).float()
    model = build(cfg, w, device)
    for seed, prompt in [(1, 1), (2, 4), (3, 2), (4, 9)]:              # the same slot again and again
        toks = tokens_for(cfg, 9, seed)
        close(run_cut(model, toks, prompt), oracle.forward(cfg, w, toks), TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_from_one_token(device):
    cfg = make_cfg([attn(window=40), gru(), attn(window=50, kv_from=0), attn(heads=2, kv_heads=2, window=16, mlp=None)])
    w = random_checkpoint(cfg, seed=21)
    toks = tokens_for(cfg, 130, 9)
    close(run_cut(build(cfg, w, device), toks, 1), oracle.forward(cfg, w, toks), TOL32)


@pytest.mark.parametrize("device", DEVICES)
def test_window_larger_than_the_cache_limit(device):
    """``max_seq_len`` below the window: the rings are only as long as sequences can get."""
    cfg = make_cfg([attn(window=400), attn(window=500, kv_from=0)])
    w = random_checkpoint(cfg, seed=2)
    toks = tokens_for(cfg, 30, 3)
    model = build(cfg, w, device, max_seq_len=30)
    assert model.states.layer(0)["k"].shape[1] == 30
    close(run_cut(model, toks, 11), oracle.forward(cfg, w, toks), TOL32)


def test_lender_must_come_first_and_match(mixed):
    cfg, w, _, _, _ = mixed
    model = build(cfg, w, "cpu")
    assert model.states.layer(1)["k"].shape[1] == 12 and model.states.layer(3) == {} and model.states.layer(5) == {}
    assert model.states.layer(len(MIXED))["prev"].dtype == torch.int64
    with pytest.raises(ValueError):
        build(make_cfg([attn(kv_from=1), attn()]), w, "cpu")
    with pytest.raises(ValueError):
        build(make_cfg([attn(), attn(kv_heads=1, kv_from=0)]), w, "cpu")


def test_continuing_step_carries_one_token(mixed):
    cfg, w, toks, _, _ = mixed
    model = build(cfg, w, "cpu")
    s = model.states.alloc()
    model.forward_step(torch.tensor([toks[:4]]), [4], [s], [0], True)
    with pytest.raises(ValueError):
        model.forward_step(torch.tensor([toks[4:7]]), [3], [s], [4], False)


# ---------------------------------------------------------------------------------------------- generation, registry, command lines
def _oracle_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(oracle.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_serving_entry_points(device, mixed):
    cfg, w, _, _, _ = mixed
    prompts = [tokens_for(cfg, 9, 31), tokens_for(cfg, 4, 32)]
    want = [_oracle_greedy(cfg, w, p, 5) for p in prompts]
    model = build(cfg, w, device, batch_size=2)
    model.on_device_sampling = True
    ids = torch.zeros(2, 9, dtype=torch.long)
    mask = torch.zeros(2, 9, dtype=torch.long)
    for b, p in enumerate(prompts):
        ids[b, :len(p)], mask[b, :len(p)] = torch.tensor(p), 1
    out = model.generate(ids.to(device), 5, prompt_lens=mask.sum(1).to(device))
    assert out.cpu().tolist() == want
    out = HuggingFaceGenerationAdapter(model, pad_token_id=0).generate(ids.to(device), attention_mask=mask.to(device), max_new_tokens=5)
    assert out[:, 9:].cpu().tolist() == want


def _save_model_dir(path, cfg, w):
    from neuronx_distributed_b200.utils.safetensors_utils import save_state_dict_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_state_dict_safetensors({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))


def _trace(cfg):
    a, b, c = tokens_for(cfg, 14, 41), tokens_for(cfg, 5, 42), tokens_for(cfg, 9, 43)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []}]
    for k in range(4):
        ent = [{"id": "a", "tokens": [a[10 + k]], "want": [0]}]
        if k < 2:
            ent.append({"id": "b", "tokens": [b[3 + k]], "want": [] if k == 0 else [0]})
        steps.append({"step": k + 1, "entries": ent, "end": (["b"] if k == 1 else []) + (["a"] if k == 3 else [])})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [8]}], "end": ["c"]})
    rows = {0: [("a", 0), ("a", 9), ("b", 2)], 1: [("a", 10)], 2: [("a", 11), ("b", 4)], 3: [("a", 12)], 4: [("a", 13)], 5: [("c", 8)]}
    return {"a": a, "b": b, "c": c}, steps, rows


@pytest.mark.parametrize("device", DEVICES)
def test_registry_checkpoint_reader_and_trace_replay(device, mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    model = registry.load_for_serving(str(tmp_path / "m"), dtype=torch.float32, device=torch.device(device), max_seq_len=64, on_device_sampling=False)
    assert isinstance(model, NoresunForInference)
    reqs, steps, rows = _trace(cfg)
    out = tmp_path / "o"
    os.makedirs(out)
    log = io.StringIO()
    TraceReplayer(model, str(out)).run([json.dumps(s) for s in steps], log)
    assert log.getvalue().split() == [x for s in steps for x in ("done", str(s["step"]))]
    assert model.states.in_use == 0
    for n, want_rows in rows.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(want_rows), cfg["vocab"]).copy())
        for j, (rid, pos) in enumerate(want_rows):
            close(got[j:j + 1], oracle.forward(cfg, w, reqs[rid][:pos + 1])[-1:], TOL32)


def test_trace_runner_command_line(mixed, tmp_path):
    import numpy as np

    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    reqs, steps, rows = _trace(cfg)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(tmp_path / "o"),
                        "--max-tokens", "40"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got = np.fromfile(tmp_path / "o" / "5.f32", dtype="<f4")
    close(torch.from_numpy(got.copy())[None], oracle.forward(cfg, w, reqs["c"])[8:9], TOL32)


def test_generate_command_line(mixed, tmp_path):
    cfg, w, _, _, _ = mixed
    _save_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = [tokens_for(cfg, 6, 51), tokens_for(cfg, 3, 52)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    args = [os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--max-new-tokens", "4"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(args, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(t) for t in line.split(",")] for line in r.stdout.strip().splitlines()[-2:]]
    assert got == [_oracle_greedy(cfg, w, p, 4) for p in prompts]


# ---------------------------------------------------------------------------------------------------------------- bfloat16 (GPU)
@pytest.mark.gpu
def test_bfloat16_serving_close_to_the_oracle():
    cfg = make_cfg([gru(width=64), attn(heads=4, kv_heads=2, dim=32, vdim=16, window=9, dims=16), gru(width=32, mlp=None),
                    attn(heads=4, kv_heads=2, dim=32, vdim=16, window=20, dims=16, kv_from=1, mlp=moe(ff=64, experts=4, top=2))], width=64)
    w = random_checkpoint(cfg, seed=13)
    toks = tokens_for(cfg, 40, 3)
    want = oracle.forward(cfg, w, toks)
    model = build(cfg, w, "cuda", dtype=torch.bfloat16)
    ref = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    for prompt in (25, 40):                          # rounding noise of a small model with large weights: a few percent, no outliers
        d = run_cut(model, toks, prompt).double() - want
        err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / ref
        assert err.mean() < 4e-2 and err.max() < 0.2, (err.mean().item(), err.max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("B,W,S", [(2, 4800, 70), (2, 70, 300), (3, 4737, 20), (1, 9600, 1), (2, 70, 1500), (1, 2400, 1100), (1, 130, 4200)])
def test_bfloat16_mingru_scan_channel_pairs_and_singles(B, W, S):
    """The bfloat16 instantiation (two channels per thread where the row is wide enough to fill the GPU that way, hardware
    exponential and reciprocal) against float64 on the same rounded inputs, prompt then one more token."""
    g = torch.Generator().manual_seed(W + S)
    p = (torch.randn(B, S + 1, 3 * W + 6, generator=g) * 2).bfloat16()
    z, u, gt = (p[..., k * W:(k + 1) * W].double() for k in range(3))
    zz = torch.sigmoid(z)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s, rows = torch.zeros(B, W, dtype=F64), []
    for t in range(S + 1):
        s = (1 - zz[:, t]) * s + zz[:, t] * cand[:, t]
        rows.append(s * gt[:, t] * torch.sigmoid(gt[:, t]))
    want = torch.stack(rows, 1)
    pd, state = p.cuda(), torch.ones(B, W, device="cuda")
    slots = i32(list(range(B)), "cuda")
    cut = lambda a, b: (pd[:, a:b, :W], pd[:, a:b, W:2 * W], pd[:, a:b, 2 * W:3 * W])
    out = seqmix.mingru_scan(*cut(0, S), state, slots, i32([S] * B, "cuda"), True)
    nxt = seqmix.mingru_scan(*cut(S, S + 1), state, slots, i32([1] * B, "cuda"), False)
    got = torch.cat([out, nxt], 1).cpu().double()
    assert (got - want).abs().max() < 1e-2 * max(1.0, want.abs().max().item())
    assert (state.cpu().double() - s).abs().max() < 1e-4 * max(1.0, s.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,D,V", [(4, 2, 16, 16), (6, 3, 64, 48), (2, 1, 128, 128), (4, 4, 64, 64), (8, 2, 128, 64), (2, 2, 256, 256), (3, 1, 24, 40)])
@pytest.mark.parametrize("window", [1, 7, 64, 100, 1000])
def test_bfloat16_prompt_attention_in_one_kernel(H, G, D, V, window):
    """The fused tensor-core prompt kernel with sigmoid weights (and the scalar kernel, for sizes it does not take) against float64
    on the same bfloat16 inputs: unequal rows, windows below, at and above the tile sizes."""
    g = torch.Generator().manual_seed(H * D + window)
    B, S = 2, 200
    lens = [200, 77]
    q, k, v = (torch.randn(B, S, n, generator=g).bfloat16() for n in (H * D, G * D, G * V))
    pb = torch.randn(H, generator=g) - 2
    scale = 1.0 / math.sqrt(D)
    sc = torch.einsum("bihd,bjhd->bhij", q.double().view(B, S, H, D), k.double().view(B, S, G, D).repeat_interleave(H // G, 2)) * scale
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    p = torch.sigmoid(sc + pb.double()[None, :, None, None]) * ((j <= i) & (j > i - window))
    want = torch.einsum("bhij,bjhv->bihv", p, v.double().view(B, S, G, V).repeat_interleave(H // G, 2)).reshape(B, S, H * V)
    out = torch.empty(B * S, H * V, dtype=torch.bfloat16, device="cuda")
    seqmix.window_attention_prompt(q.cuda().view(B, S, H, D), k.cuda().view(B, S, G, D), v.cuda().view(B, S, G, V), None, i32(lens, "cuda"), window,
                                   scale, 0.0, out, 1.0, pb.cuda())
    got = out.view(B, S, H * V).cpu().double()
    for b in range(B):
        n = lens[b]
        ref = want[b, :n].abs().max().item()
        assert (got[b, :n] - want[b, :n]).abs().max() < 2e-2 * max(ref, 1.0)
        assert (got[b, n:] == 0).all()
