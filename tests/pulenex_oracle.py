"""Plain, slow restatement of the Pulenex decoder for the numerics tests: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batching), float64 by default.  It shares no code with the served model:
weights come in as a ``{checkpoint name: tensor}`` dict and the configuration as the parsed ``config.json`` dict."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def centred_norm(x, w, eps):
    """Layer norm with a gain and no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def causal_conv(h, w):
    """h [S, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    S, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(S):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate(x, dims, base, interleaved, first_pos=0):
    """x [S, heads, n]: the first ``dims`` coordinates of every head turn by angle p * base^(-2i/dims); pair i is (i, i + dims/2) or,
    interleaved, (2i, 2i + 1)."""
    out = x.clone()
    half = dims // 2
    for p in range(x.shape[0]):
        for i in range(half):
            a = (first_pos + p) * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            ia, ib = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
            u, v = x[p, :, ia], x[p, :, ib]
            out[p, :, ia] = u * c - v * s
            out[p, :, ib] = v * c + u * s
    return out


def retention(h, P, m, eps):
    """Linear attention with one fixed decay per head: S <- decay S + k v^T, o = S^T q; no softmax, no denominator."""
    S = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ P["q"].T).reshape(S, H, D), m["rot"]["dims"], m["rot"]["base"], False)
    k = rotate((h @ P["k"].T).reshape(S, H, D), m["rot"]["dims"], m["rot"]["base"], False) * D ** -0.5
    v = (h @ P["v"].T).reshape(S, H, V)
    out = torch.zeros(S, H, V, dtype=h.dtype)
    for hd in range(H):
        M = torch.zeros(D, V, dtype=h.dtype)
        for t in range(S):
            M = m["decay"][hd] * M + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = M.T @ q[t, hd]
    out = rms(out, eps).reshape(S, H * V) * silu(h @ P["g"].T)
    return out @ P["o"].T


def chunked_attention(h, P, m):
    """Softmax attention inside aligned chunks of positions, keys doubling as values, with convolved queries and keys, a per-head
    temperature, score mixing across heads and a sink term in the denominator."""
    S = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    assert m["vdim"] == D, "values are the keys"
    q = causal_conv(h @ P["q"].T, P["q.conv"]).reshape(S, H, D)
    kc = causal_conv(h @ P["k"].T, P["k.conv"]).reshape(S, G, D)
    v = kc
    q = rotate(q, m["rot"]["dims"], m["rot"]["base"], True)
    k = rotate(kc, m["rot"]["dims"], m["rot"]["base"], True)
    size = m["mask"]["size"]
    heads = torch.zeros(S, H, D, dtype=h.dtype)
    for i in range(S):
        lo = (i // size) * size
        raw = torch.stack([(k[lo:i + 1, hd // (H // G)] @ q[i, hd]) * m["scale"] * P["temp"][hd] for hd in range(H)])   # [H, n]
        sc = P["talk"] @ raw
        for hd in range(H):
            top = max(float(sc[hd].max()), float(P["sink"][hd]))
            e = torch.exp(sc[hd] - top)
            heads[i, hd] = (e / (e.sum() + math.exp(float(P["sink"][hd]) - top))) @ v[lo:i + 1, hd // (H // G)]
    return (heads.reshape(S, H * D) * sigmoid(h @ P["g"].T)) @ P["o"].T


def channel_delta_rule(h, P, m, eps):
    """Gated delta rule with one decay per head and key channel, low-rank decay and gate projections."""
    S = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ P["q"].T, P["q.conv"])).reshape(S, G, D)
    k = silu(causal_conv(h @ P["k"].T, P["k.conv"])).reshape(S, G, D)
    v = silu(causal_conv(h @ P["v"].T, P["v.conv"])).reshape(S, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ P["b"].T)                                                                   # [S, H]
    step = softplus((h @ P["a1"].T) @ P["a2"].T + P["dt_bias"]).reshape(S, H, D)
    g = torch.exp(-torch.exp(P["A_log"])[None, :, None] * step)
    gate = sigmoid((h @ P["g1"].T) @ P["g2"].T).reshape(S, H, V)
    out = torch.zeros(S, H, V, dtype=h.dtype)
    for hd in range(H):
        M = torch.zeros(D, V, dtype=h.dtype)
        kh = hd // (H // G)
        for t in range(S):
            M = g[t, hd][:, None] * M
            u = beta[t, hd] * (v[t, hd] - M.T @ k[t, kh])
            M = M + torch.outer(k[t, kh], u)
            out[t, hd] = M.T @ q[t, kh]
    out = rms(out, eps) * P["norm"] * gate
    return out.reshape(S, H * V) @ P["o"].T


def parallel(h, P, m, eps):
    sub = lambda side: {k[len(side) + 1:]: v for k, v in P.items() if k.startswith(side + ".")}
    a = rms(chunked_attention(h, sub("left"), m["left"]), eps) * P["left.out"]
    b = rms(channel_delta_rule(h, sub("right"), m["right"], eps), eps) * P["right.out"]
    return 0.5 * (a + b)


def latent_keys(h, P, m, eps):
    """The cached part of latent attention: the normed latent c [S, kv_rank] and the rotated shared key part [S, rot_dim]."""
    S, C, R = h.shape[0], m["kv_rank"], m["rot_dim"]
    d = h @ P["dkv"].T
    c = rms(d[:, :C], eps) * P["dkv.norm"]
    kr = rotate(d[:, C:].reshape(S, 1, R), m["rot"]["dims"], m["rot"]["base"], True).reshape(S, R)
    return c, kr


def latent_attention(h, P, m, eps, shared=None):
    """Sliding-window softmax attention whose keys and values are expanded from a cached latent; ``shared`` = (c, rotated key
    part) of another layer when this one has no down-projection of its own."""
    S = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = shared if shared is not None else latent_keys(h, P, m, eps)
    q = (h @ P["q"].T).reshape(S, H, D + R)
    qr = rotate(q[..., D:], m["rot"]["dims"], m["rot"]["base"], True)
    ku = (c @ P["uk"].T).reshape(S, H, D)
    vu = (c @ P["uv"].T).reshape(S, H, V)
    win = m["mask"]["size"]
    heads = torch.zeros(S, H, V, dtype=h.dtype)
    for i in range(S):
        lo = max(0, i - win + 1)
        for hd in range(H):
            sc = (ku[lo:i + 1, hd] @ q[i, hd, :D] + kr[lo:i + 1] @ qr[i, hd]) * m["scale"]
            heads[i, hd] = torch.softmax(sc, 0) @ vu[lo:i + 1, hd]
    heads = heads * sigmoid(h @ P["g"].T)[..., None]
    return heads.reshape(S, H * V) @ P["o"].T


def clamped_ffn(h, P, f):
    g = torch.clamp(h @ P["gate"].T + P["gate.b"], max=f["limit"])
    u = torch.clamp(h @ P["up"].T + P["up.b"], -f["limit"], f["limit"])
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ P["down"].T + P["down.b"]


def forward(cfg, sd, tokens, dtype=torch.float64, taps=None):
    """tokens: a list of ids → logits [S, vocab]; ``taps`` (a list) receives the residual stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    latents = {}
    for i, spec in enumerate(cfg["layers"]):
        pre = f"l{i}."
        P = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        m, h = spec["mixer"], centred_norm(x, W[pre + "norm1"], eps)
        if spec["type"] == "retention":
            y = retention(h, P, m, eps)
        elif spec["type"] == "parallel":
            y = parallel(h, P, m, eps)
        elif spec["type"] == "latent_attention":
            if "kv_from" in m:
                y = latent_attention(h, P, m, eps, latents[int(m["kv_from"])])
            else:
                latents[i] = latent_keys(h, P, m, eps)
                y = latent_attention(h, P, m, eps, latents[i])
        else:
            raise ValueError(spec["type"])
        x = x + centred_norm(y, W[pre + "norm1b"], eps)
        if spec.get("mlp"):
            F = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            y = clamped_ffn(centred_norm(x, W[pre + "norm2"], eps), F, spec["mlp"])
            x = x + centred_norm(y, W[pre + "norm2b"], eps)
        if taps is not None:
            taps.append(x.clone())
    return (centred_norm(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]
