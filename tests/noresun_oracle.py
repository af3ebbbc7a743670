"""Plain, slow statement of the Noresun design in float64: one function per mechanism, whole sequences at once, no caches, no
kernels, nothing shared with the serving path.  Weights come as a dict of checkpoint tensors (``l<i>.mix.*`` etc.), configurations
as the ``config.json`` dict."""
import math

import torch

F64 = torch.float64


def rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every position: a hash of (token before, token); the first position takes the extra last row."""
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * mul_prev + b * mul_cur) % buckets)
    return rows


def embed(cfg, w, tokens):
    e = cfg.get("embedding") or {}
    x = w["embed"].to(F64)[tokens] * float(e.get("scale", 1.0))
    if e.get("bigram"):
        g = e["bigram"]
        x = x + w["bigram"].to(F64)[pair_rows(tokens, g["buckets"], g["mul_prev"], g["mul_cur"])]
    return x


def frequencies(rot):
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wave >= sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate_neighbours(x, freqs):
    """x [S, heads, D]: coordinates (2i, 2i+1) of every head turned by the angle position * freqs[i]; the rest untouched."""
    y = x.clone()
    for t in range(x.shape[0]):
        for i, f in enumerate(freqs):
            c, s = math.cos(t * f), math.sin(t * f)
            a, b = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            y[t, :, 2 * i], y[t, :, 2 * i + 1] = a * c - b * s, b * c + a * s
    return y


def attention_keys(m, w, p, h, eps):
    """The prepared keys [S, G, D] and the values [S, G, V] of a layer that has its own."""
    S = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = rms(h @ w[p + "k"].to(F64).T, w[p + "k.norm"].to(F64), eps).view(S, G, D)
    return rotate_neighbours(k, frequencies(m["rot"])), (h @ w[p + "v"].to(F64).T).view(S, G, V)


def sigmoid_window_attention(m, w, p, h, eps, k, v):
    S = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate_neighbours(rms(h @ w[p + "q"].to(F64).T, w[p + "q.norm"].to(F64), eps).view(S, H, D), frequencies(m["rot"]))
    out = torch.zeros(S, H, V, dtype=F64)
    for i in range(S):
        for hd in range(H):
            g = hd // (H // G)
            for j in range(max(0, i - m["mask"]["size"] + 1), i + 1):
                weight = torch.sigmoid((q[i, hd] @ k[j, g]) * m["scale"] + w[p + "pb"].to(F64)[hd])
                out[i, hd] += weight * v[j, g]
    return out.view(S, H * V) @ w[p + "o"].to(F64).T


def mingru(m, w, p, h):
    z = torch.sigmoid(h @ w[p + "z"].to(F64).T + w[p + "z.b"].to(F64))
    u = h @ w[p + "x"].to(F64).T + w[p + "x.b"].to(F64)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w[p + "g"].to(F64).T
    gate = gate * torch.sigmoid(gate)
    s = torch.zeros(m["width"], dtype=F64)
    rows = []
    for t in range(h.shape[0]):
        s = (1 - z[t]) * s + z[t] * cand[t]
        rows.append(s * gate[t])
    return torch.stack(rows) @ w[p + "o"].to(F64).T


def routed_ffn(f, w, p, h):
    r = f["router"]
    logits = h @ w[p + "router"].to(F64).T + w[p + "router.b"].to(F64)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(r["experts"]), key=lambda e: -float(logits[t, e]))[: r["top"]]
        share = torch.softmax(logits[t, chosen], 0)
        for s, e in zip(share, chosen):
            mid = torch.relu(w[p + f"e{e}.up"].to(F64) @ h[t]) ** 2
            out[t] += s * (w[p + f"e{e}.down"].to(F64) @ mid)
    return out


def forward(cfg, w, tokens, taps=None):
    """Logits [S, vocab] (float64) of one sequence; ``taps`` collects the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    x = embed(cfg, w, tokens)
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        if L["type"] == "mingru":
            y = mingru(m, w, p + "mix.", x)
        else:
            if m.get("kv_from") is None:
                kept[i] = attention_keys(m, w, p + "mix.", x, eps)
            k, v = kept[i if m.get("kv_from") is None else m["kv_from"]]
            y = sigmoid_window_attention(m, w, p + "mix.", x, eps, k, v)
        g = torch.sigmoid(x @ w[p + "rg1"].to(F64).T + w[p + "rg1.b"].to(F64))
        x = rms(alpha * x + g * y, w[p + "norm1"].to(F64), eps)
        if L.get("mlp"):
            y = routed_ffn(L["mlp"], w, p + "mlp.", x)
            g = torch.sigmoid(x @ w[p + "rg2"].to(F64).T + w[p + "rg2.b"].to(F64))
            x = rms(alpha * x + g * y, w[p + "norm2"].to(F64), eps)
        if taps is not None:
            taps.append(x.clone())
    return rms(x, w["final.norm"].to(F64), eps) @ w["embed"].to(F64).T
