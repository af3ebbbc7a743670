"""``bench.py --mode noresun``: serving throughput of the Noresun design at layer sizes that resemble a real model (random weights),
beside the framework's closest existing models at equal width and depth — Pinirax (grouped-query window attention and a routed
feed-forward, whose kernels Noresun's attention and experts extend) and Naguzen (whose real-gated LRU scan is the like of the
minGRU scan) — plus every kernel the design added or extended, timed alone against the measured copy bandwidth / GEMM throughput,
beside the like kernel of those paths.  One GPU, bfloat16.  Device time (CUDA events), >= 3 warm-up iterations; the weights of
every model exceed L2, and the kernel timings flush L2 (a 512 MiB write) between iterations; every kernel row is replayed from a
CUDA graph.

Layers (width 2048): minGRU of 4096 channels + 32 squared-relu experts of 1024, 4 chosen | sigmoid window attention, 16 heads / 4 KV
heads of 128, value 128, window 1024, 64 rotated coordinates with rescaled frequencies + the same experts | minGRU + experts |
attention borrowing the second layer's keys and values + experts."""
from __future__ import annotations

import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tools"))

import bench_naguzen as base  # noqa: E402
import bench_pinirax as pin  # noqa: E402

WIDTH, VOCAB = base.WIDTH, base.VOCAB
SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}


def noresun_layers():
    moe = {"kind": "moe", "expert": {"ff": 1024}, "router": {"experts": 32, "top": 4}}
    gru = {"type": "mingru", "mlp": moe, "mixer": {"width": 4096}}
    att = lambda src: {"type": "attention", "mlp": moe,
                       "mixer": dict({"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 1.0 / math.sqrt(128),
                                      "rot": {"base": 500000.0, "dims": 64, "scaling": SCALING}}, **({} if src is None else {"kv_from": src}))}
    return [gru, att(None), gru, att(1)]


def build_noresun(dev, batch, max_len):
    import torch

    from neuronx_distributed_b200.models.noresun import NoresunConfig, NoresunForInference

    cfg = NoresunConfig(vocab=VOCAB, width=WIDTH, layers=noresun_layers(), norm_eps=1e-6, postln_alpha=2.0, embedding_scale=8.0,
                        bigram={"buckets": 65521, "mul_prev": 31, "mul_cur": 17}, dtype=torch.bfloat16, device=dev)
    m = NoresunForInference(cfg, batch_size=batch, max_seq_len=max_len).eval()
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dtype == torch.bfloat16 or "router" in name:
                p.normal_(0.0, 0.02 if p.dim() > 1 else 0.0, generator=g)
                if "router" in name:                       # as a checkpoint stored in bfloat16 would hold it
                    p.copy_(p.to(torch.bfloat16).float())
            # norm gains (1) and score biases (0) keep their initial values
        m.lm.embed.normal_(0.0, 1.0, generator=g)
    return m


def kernel_table(dev, steps, warmup):
    """Each kernel the design added or extended, alone at the sizes of the model above (4 x 2048 prompt tokens; 8 decoding rows) →
    time, achieved GB/s or TFLOP/s, fraction of the measured peak; the like kernel of the Pinirax / Naguzen path is timed the same way
    in the row after it."""
    import torch

    from neuronx_distributed_b200.ops import seqmix

    hbm, tfl, src = base._peaks()
    flush = torch.empty(128 << 20, dtype=torch.float32, device=dev)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    B, S, W = 4, 2048, WIDTH
    N = B * S
    rnd = lambda *s, dtype=bf: torch.randn(*s, device=dev, dtype=f32).to(dtype)
    lens, slots, pos0 = torch.full((B,), S, dtype=i32, device=dev), torch.arange(B, dtype=i32, device=dev), torch.zeros(B, dtype=i32, device=dev)
    Bd = 8
    l1, s8, p8 = torch.ones(Bd, dtype=i32, device=dev), torch.arange(Bd, dtype=i32, device=dev), torch.full((Bd,), 2047, dtype=i32, device=dev)
    rows = []

    def replayed(fn):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g.replay
        except Exception:
            torch.cuda.synchronize()
            return fn

    def add(name, fn, bytes_=0, flops=0, like=None):
        ms = base._timed(replayed(fn), steps, warmup, flush)
        r = {"kernel": name, "ms": round(ms, 4)}
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            r["frac_bf16_gemm"] = round(flops / ms / 1e9 / tfl, 4)
        if like:
            r["like_of"] = like
        rows.append(r)

    # embedding
    ids = torch.randint(0, VOCAB, (B, S), device=dev)
    table, pairs, prev = rnd(VOCAB, W), rnd(65522, W), torch.zeros(B, dtype=torch.int64, device=dev)
    add("embed_bigram (token + hashed pair rows -> f32 stream + bf16 copy)",
        lambda: seqmix.embed_bigram(ids, table, 8.0, pairs, 31, 17, prev, slots, lens, True, True), N * W * (2 + 2 + 4 + 2))
    inv_w = seqmix.sinusoid_inv_freq(W, 10000.0, dev)
    add("pinirax embed_sinusoid (token rows + sinusoids -> f32 stream)", lambda: seqmix.embed_sinusoid(ids, table, 8.0, inv_w, pos0), N * W * (2 + 4),
        like="embed_bigram")
    # the closing step of a block
    x32, yg, wW, low = rnd(N, W, dtype=f32), rnd(N, 2 * W), torch.ones(W, device=dev), torch.empty(N, W, dtype=bf, device=dev)
    add("postnorm_gated_ (stream <- norm(alpha stream + sigmoid(gate) y), f32 in place + bf16 copy)",
        lambda: seqmix.postnorm_gated_(x32, yg[:, :W], yg[:, W:], wW, 2.0, 1e-6, low), N * W * (4 + 2 + 2 + 4 + 2))
    y16 = rnd(N, W)
    add("pinirax stream += rms_norm(bf16), then rms_norm f32 -> bf16 (closing norm + the next sublayer's opening norm)",
        lambda: (seqmix.add_rms_norm_(x32, y16, wW, 1e-6), seqmix.rms_norm(x32, wW, 1e-6, None, bf)), N * W * (10 + 6), like="postnorm_gated_")
    # minGRU beside the real-gated LRU
    R = 4096
    p = rnd(B, S, 3 * R + W)
    st = torch.zeros(B, R, device=dev)
    add("mingru_scan prompt (4096 channels; z, u, gate read in place from the stacked projection)",
        lambda: seqmix.mingru_scan(p[..., :R], p[..., R:2 * R], p[..., 2 * R:3 * R], st, slots, lens, True), N * R * (5 * 2 + 2))
    Rl, nb = 2048, 8
    u, yv = rnd(B, S, Rl), rnd(B, S, Rl)
    gr, gi = rnd(nb, N, Rl // nb, dtype=f32), rnd(nb, N, Rl // nb, dtype=f32)
    rb, lam, stl = torch.zeros(Rl, device=dev), torch.full((Rl,), 0.5, device=dev), torch.zeros(B, Rl, device=dev)
    add("naguzen rglru_scan prompt (2048 channels, float gate pre-activations)",
        lambda: seqmix.rglru_scan(u, gr, gi, rb, rb, lam, yv, stl, slots, lens, True), N * Rl * (2 * (2 + 4 + 4) + 2 + 2), like="mingru_scan prompt")
    p1, st8 = rnd(Bd, 1, 3 * R + W), torch.zeros(Bd, R, device=dev)
    add("mingru_scan decode (8 rows)", lambda: seqmix.mingru_scan(p1[..., :R], p1[..., R:2 * R], p1[..., 2 * R:3 * R], st8, s8, l1, False),
        Bd * R * (6 + 8 + 2))
    u1, y1 = rnd(Bd, 1, Rl), rnd(Bd, 1, Rl)
    gr1, gi1, stl8 = rnd(nb, Bd, Rl // nb, dtype=f32), rnd(nb, Bd, Rl // nb, dtype=f32), torch.zeros(Bd, Rl, device=dev)
    add("naguzen rglru_scan decode (8 rows)", lambda: seqmix.rglru_scan(u1, gr1, gi1, rb, rb, lam, y1, stl8, s8, l1, False), Bd * Rl * (4 + 8 + 8 + 2),
        like="mingru_scan decode")
    # attention
    H, G, D, win, dims = 16, 4, 128, 1024, 64
    q, k, v = rnd(B, S, H, D), rnd(B, S, G, D), rnd(B, S, G, D)
    qwa, kwa, qwh = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev), torch.ones(D, device=dev)
    inv = seqmix.rotary_inv_freq(dims, 500000.0, dev, SCALING)
    kc, vc = torch.zeros(B, win, G, D, dtype=bf, device=dev), torch.zeros(B, win, G, D, dtype=bf, device=dev)
    prep_bytes = N * (H + G) * D * 4 + B * win * G * 2 * D * 4
    add("window_qk_prepare (one norm over all heads + rotation of 64 coordinates in place + ring store)",
        lambda: seqmix.window_qk_prepare(q, k, v, qwa, kwa, 1e-6, pos0, lens, slots, kc, vc, norm_all=True, inv_freq=inv, rot_dims=dims), prep_bytes)
    add("pinirax window_qk_prepare (head norms in place + ring store)", lambda: seqmix.window_qk_prepare(q, k, v, qwh, qwh, 1e-6, pos0, lens, slots, kc, vc),
        prep_bytes, like="window_qk_prepare")
    out = torch.empty(N, H * D, dtype=bf, device=dev)
    pb = torch.full((H,), -2.0, device=dev)
    pairs_w = B * H * sum(min(t + 1, win) for t in range(S))
    add("window_attention_prompt, sigmoid weights + head bias (GQA 16/4 x 128, window 1024)",
        lambda: seqmix.window_attention_prompt(q, k, v, None, lens, win, 0.088, 0.0, out, 1.0, pb), flops=pairs_w * 2 * (D + D))
    hgate = rnd(B, S, H)
    add("pinirax window_attention_prompt, softmax (same sizes, cap, gate)",
        lambda: seqmix.window_attention_prompt(q, k, v, hgate, lens, win, 0.088, 30.0, out, 0.8), flops=pairs_w * 2 * (D + D), like="window_attention_prompt")
    add("window_attention_prompt, softmax without cap and gate (same sizes)",
        lambda: seqmix.window_attention_prompt(q, k, v, None, lens, win, 0.088, 0.0, out, 1.0), flops=pairs_w * 2 * (D + D), like="window_attention_prompt")
    q1, kc8, vc8 = rnd(Bd, 1, H, D), rnd(Bd, win, G, D), rnd(Bd, win, G, D)
    o1, hg1 = torch.empty(Bd, H * D, dtype=bf, device=dev), rnd(Bd, 1, H)
    add("window_attention_token, sigmoid weights (8 rows, ring 1024, 4 KV heads)",
        lambda: seqmix.window_attention_token(q1, kc8, vc8, None, s8, p8, l1, win, 0.088, 0.0, o1, 1.0, pb), bytes_=Bd * win * G * D * 4)
    add("pinirax window_attention_token, softmax (8 rows, ring 1024, 4 KV heads)",
        lambda: seqmix.window_attention_token(q1, kc8, vc8, hg1, s8, p8, l1, win, 0.088, 30.0, o1, 0.8), bytes_=Bd * win * G * D * 4,
        like="window_attention_token")
    # router and experts
    E, top, FF = 32, 4, 1024
    lg = rnd(N, E, dtype=f32)
    add("route_topk, softmax over the chosen logits (32 experts, 4 chosen)", lambda: seqmix.route_topk(lg, None, top, E, "softmax_top"),
        N * (E * 4 + top * 12))
    add("pinirax route_topk, softmax over all (32 experts, 4 chosen)", lambda: seqmix.route_topk(lg, None, top, E, "softmax"), N * (E * 4 + top * 12),
        like="route_topk")
    mid = rnd(N * top, FF)
    add("relu_sq [N x 4, 1024]", lambda: seqmix.relu_sq(mid), N * top * FF * 4)
    add("naguzen gelu_erf [N x 4, 1024]", lambda: seqmix.gelu_erf(mid), N * top * FF * 4, like="relu_sq")
    up, sel, xs = rnd(E, FF, W), torch.randint(0, E, (Bd * top,), dtype=i32, device=dev), rnd(Bd * top, W)
    add("indexed_gemv up, squared relu (8 rows x 4 experts)", lambda: seqmix.indexed_gemv(up, sel, xs, "relu_sq"), Bd * top * FF * W * 2)
    add("naguzen indexed_gemv up, gelu (8 rows x 4 experts)", lambda: seqmix.indexed_gemv(up, sel, xs, "gelu"), Bd * top * FF * W * 2, like="indexed_gemv")
    return {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src}, "rows": rows}


def main(args) -> int:
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29541")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    from neuronx_distributed_b200.parallel_layers import parallel_state as ps

    ps.initialize_model_parallel(tensor_model_parallel_size=1)
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    out = {"mode": "noresun", "dtype": "bf16", "data": "synthetic", "steps": steps, "warmup": warmup, "n_gpus": 1,
           "l2": "weights of every model exceed L2; kernel rows flush L2 between iterations"}
    shapes = [(4, 2048), (1, 8192), (8, 512)]
    for name, make in (("noresun", build_noresun), ("pinirax", pin.build_pinirax), ("naguzen", base.build_naguzen)):
        res = []
        for B, S in shapes:
            model = make(dev, B, S + 64)
            res.append(base.throughput(model, dev, B, S, S, steps, warmup))
            del model
            torch.cuda.empty_cache()
        out[name] = res
    out["kernels"] = kernel_table(dev, max(steps, 5), warmup)
    print(json.dumps(out), flush=True)
    dist.destroy_process_group()
    return 0
