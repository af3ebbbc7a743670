"""``bench.py --mode pulenex``: serving throughput of the Pulenex design at layer sizes that resemble a real model (random weights),
beside the framework's closest existing models at equal width and depth — Naguzen (latent window attention + a gated linear
recurrence, whose kernels Pulenex's latent attention and retention extend) and Pinirax (attention next to a delta rule in one layer,
norms on both sides of every sublayer) — plus every kernel the design added, timed alone against the measured copy bandwidth / GEMM
throughput, beside the like kernel of those paths.  One GPU, bfloat16.  Device time (CUDA events), >= 3 warm-up iterations; the
weights of every model exceed L2, and the kernel timings flush L2 (a 512 MiB write) between iterations; every kernel row is replayed
from a CUDA graph.

Layers (width 2048): latent attention 16 heads of 128 + 64 rotated, value 128, latent 512, window 1024, head gates + dense ff 8192 |
retention 8 heads of 256 x 256, no feed-forward | parallel [head-mixing attention 16 heads / 4 KV heads of 128, chunk 1024, 4 taps |
delta rule 16 value heads of 128 over 4 q/k heads of 128, a decay per key channel through rank 64, gate through rank 128, 4 taps] +
dense ff 8192 | latent attention borrowing the first layer's latents + dense ff 8192."""
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


def pulenex_layers():
    dense = {"kind": "dense", "ff": 8192, "limit": 7.0}
    lat = lambda src: {"type": "latent_attention", "mlp": dense,
                       "mixer": dict({"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "mask": {"size": 1024},
                                      "rot": {"base": 10000.0, "dims": 64}, "scale": 1.0 / math.sqrt(192)}, **({} if src is None else {"kv_from": src}))}
    ret = {"type": "retention", "mlp": None,
           "mixer": {"heads": 8, "dim": 256, "vdim": 256, "decay": [1.0 - 2.0 ** (-5 - h) for h in range(8)], "rot": {"base": 10000.0, "dims": 256}}}
    par = {"type": "parallel", "mlp": dense,
           "mixer": {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "conv": 4, "mask": {"size": 1024}, "rot": {"base": 10000.0, "dims": 128},
                              "scale": 1.0 / math.sqrt(128)},
                     "right": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 128}}}
    return [lat(None), ret, par, lat(0)]


def build_pulenex(dev, batch, max_len):
    import torch

    from neuronx_distributed_b200.models.pulenex import PulenexConfig, PulenexForInference

    cfg = PulenexConfig(vocab=VOCAB, width=WIDTH, layers=pulenex_layers(), norm_eps=1e-6, logit_scale=0.5, dtype=torch.bfloat16, device=dev)
    m = PulenexForInference(cfg, batch_size=batch, max_seq_len=max_len).eval()
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dtype == torch.bfloat16:
                p.normal_(0.0, 0.02 if p.dim() > 1 else 0.0, generator=g)
            elif "conv.weight" in name:
                p.normal_(0.0, 0.2, generator=g)
            elif name.endswith("a_log"):
                p.fill_(-1.0)
            elif name.endswith("right.norm"):
                p.fill_(1.0)
            elif name.endswith("talk"):
                p.copy_(torch.eye(p.shape[0], device=dev) + 0.1 * torch.randn(p.shape, device=dev, generator=g))
            # norm gains, temperatures (1) and sinks (0) keep their initial values
        m.lm.embed.normal_(0.0, 1.0, generator=g)
    return m


def kernel_table(dev, steps, warmup):
    """Each kernel the design added, alone at the sizes of the model above (4 x 2048 prompt tokens; 8 decoding rows) → time, achieved
    GB/s or TFLOP/s, fraction of the measured peak; the like kernel of the Naguzen / Pinirax path is timed the same way in the row
    after it."""
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

    # norms of the sandwich block
    x32, y16, wW = rnd(N, W, dtype=f32), rnd(N, W), torch.ones(W, device=dev)
    add("layer norm (gain only) f32 -> bf16", lambda: seqmix.rms_norm(x32, wW, 1e-6, None, bf, center=True), N * W * 6)
    add("rms_norm f32 -> bf16", lambda: seqmix.rms_norm(x32, wW, 1e-6, None, bf), N * W * 6, like="layer norm")
    add("stream += layer norm(bf16)", lambda: seqmix.add_rms_norm_(x32, y16, wW, 1e-6, center=True), N * W * 10)
    add("stream += rms_norm(bf16)", lambda: seqmix.add_rms_norm_(x32, y16, wW, 1e-6), N * W * 10, like="stream += layer norm")
    # feed-forward activation, head gates
    FF = 8192
    gu = rnd(N, 2 * FF)
    add("clamped_glu [N, 2 x 8192]", lambda: seqmix.clamped_glu(gu, 7.0, 1.702), N * FF * 6)
    add("pinirax silu_mul [N, 2 x 8192]", lambda: seqmix.silu_mul(gu), N * FF * 6, like="clamped_glu")
    hv, hg = rnd(N, 2048), rnd(N, 16, dtype=f32)
    add("sigmoid_gate_mul_ (16 head gates over [N, 2048])", lambda: seqmix.sigmoid_gate_mul_(hv, hg), N * 2048 * 4)
    gu2 = rnd(N, 4096)
    add("pinirax silu_mul [N, 2 x 2048]", lambda: seqmix.silu_mul(gu2), N * 2048 * 6, like="sigmoid_gate_mul_")
    # retention
    Hr, Dr, Vr = 8, 256, 256
    pr = rnd(B, S, 2 * Hr * Dr + 2 * Hr * Vr)
    invr = seqmix.rotary_inv_freq(Dr, 10000.0, dev)
    nqk = 2 * Hr * Dr + Hr * Vr
    add("rotary_qkv_f32 (8 + 8 heads of 256 rotated, values copied; bf16 -> f32)",
        lambda: seqmix.rotary_qkv_f32(pr[..., :nqk], Hr, Hr, Dr, Dr, invr, pos0, 1.0, Dr ** -0.5), N * nqk * 6)
    Cl, R = 512, 64
    kvl, nw, invl = rnd(B, S, Cl + R), torch.ones(Cl, device=dev), seqmix.rotary_inv_freq(R, 10000.0, dev)
    cachel = torch.zeros(B, 1024, Cl + R, dtype=bf, device=dev)
    add("naguzen latent_kv_store (norm + rotation + ring append)", lambda: seqmix.latent_kv_store(kvl, nw, 1e-6, invl, R, pos0, lens, slots, cachel, True),
        N * (Cl + R) * 4 + B * 1024 * (Cl + R) * 2, like="rotary_qkv_f32")
    fr = rnd(B, S, nqk, dtype=f32)
    qr, kr = fr[..., :Hr * Dr].unflatten(-1, (Hr, Dr)), fr[..., Hr * Dr:2 * Hr * Dr].unflatten(-1, (Hr, Dr))
    vr = fr[..., 2 * Hr * Dr:].unflatten(-1, (Hr, Vr))
    dec = torch.tensor([1.0 - 2.0 ** (-5 - h) for h in range(Hr)], device=dev)
    str_ = torch.zeros(B, Hr, Dr, Vr, device=dev)
    add("retention_scan prompt (8 heads, 256 x 256 state)", lambda: seqmix.retention_scan(qr, kr, vr, dec, str_, slots, lens, True),
        bytes_=N * (nqk * 4 + Hr * Vr * 4), flops=N * Hr * Dr * Vr * 4)
    Hg, Dg, Vg = 4, 256, 512
    pg = rnd(B, S, 2 * Hg * Dg + Hg * Vg)
    qg, kg = pg[..., :Hg * Dg].unflatten(-1, (Hg, Dg)), pg[..., Hg * Dg:2 * Hg * Dg].unflatten(-1, (Hg, Dg))
    vg, zg = pg[..., 2 * Hg * Dg:].unflatten(-1, (Hg, Vg)), rnd(B, S, Hg * Dg)
    zb, stg = torch.full((Hg * Dg,), 3.0, device=dev), torch.zeros(B, Hg, Dg, Vg, device=dev)
    add("naguzen gla_scan prompt (4 heads, 256 x 512 state)", lambda: seqmix.gla_scan(qg, kg, vg, zg, zb, 16.0, stg, slots, lens, True),
        bytes_=N * (3 * Hg * Dg * 2 + Hg * Vg * 2 + Hg * Vg * 4), flops=N * Hg * Dg * Vg * 4, like="retention_scan prompt")
    f1 = rnd(Bd, 1, nqk, dtype=f32)
    q1r, k1r = f1[..., :Hr * Dr].unflatten(-1, (Hr, Dr)), f1[..., Hr * Dr:2 * Hr * Dr].unflatten(-1, (Hr, Dr))
    v1r, st8r = f1[..., 2 * Hr * Dr:].unflatten(-1, (Hr, Vr)), torch.zeros(Bd, Hr, Dr, Vr, device=dev)
    add("retention_scan decode (8 rows)", lambda: seqmix.retention_scan(q1r, k1r, v1r, dec, st8r, s8, l1, False), bytes_=Bd * Hr * Dr * Vr * 8)
    p1g, z1g, stg8 = rnd(Bd, 1, 2 * Hg * Dg + Hg * Vg), rnd(Bd, 1, Hg * Dg), torch.zeros(Bd, Hg, Dg, Vg, device=dev)
    q1g, k1g = p1g[..., :Hg * Dg].unflatten(-1, (Hg, Dg)), p1g[..., Hg * Dg:2 * Hg * Dg].unflatten(-1, (Hg, Dg))
    v1g = p1g[..., 2 * Hg * Dg:].unflatten(-1, (Hg, Vg))
    add("naguzen gla_scan decode (8 rows)", lambda: seqmix.gla_scan(q1g, k1g, v1g, z1g, zb, 16.0, stg8, s8, l1, False), bytes_=Bd * Hg * Dg * Vg * 8,
        like="retention_scan decode")
    # delta rule: a decay per key channel beside the one-decay-per-head form
    Hd, Gd, Dd, Vd = 16, 4, 128, 128
    qd, kd, vd = rnd(B, S, Gd, Dd), rnd(B, S, Gd, Dd), rnd(B, S, Hd, Vd)
    braw, araw_c, araw_h = rnd(B, S, Hd, dtype=f32), rnd(B, S, Hd, Dd, dtype=f32), rnd(B, S, Hd, dtype=f32)
    al, db_c, db_h = torch.full((Hd,), -1.0, device=dev), torch.zeros(Hd * Dd, device=dev), torch.zeros(Hd, device=dev)
    std = torch.zeros(B, Hd, Dd, Vd, device=dev)
    io = N * (2 * Gd * Dd * 2 + Hd * Vd * 2 + Hd * Vd * 4)
    add("gated_delta_scan prompt, decay per key channel (16 heads, 128 x 128 state)",
        lambda: seqmix.gated_delta_scan(qd, kd, vd, braw, araw_c, al, db_c, std, slots, lens, True), bytes_=io + N * Hd * Dd * 4, flops=N * Hd * Dd * Vd * 6)
    add("pinirax gated_delta_scan prompt, decay per head", lambda: seqmix.gated_delta_scan(qd, kd, vd, braw, araw_h, al, db_h, std, slots, lens, True),
        bytes_=io, flops=N * Hd * Dd * Vd * 6, like="gated_delta_scan per channel, prompt")
    q1d, k1d, v1d = rnd(Bd, 1, Gd, Dd), rnd(Bd, 1, Gd, Dd), rnd(Bd, 1, Hd, Vd)
    b1, a1c, a1h = rnd(Bd, 1, Hd, dtype=f32), rnd(Bd, 1, Hd, Dd, dtype=f32), rnd(Bd, 1, Hd, dtype=f32)
    st8 = torch.zeros(Bd, Hd, Dd, Vd, device=dev)
    add("gated_delta_scan decode, decay per key channel (8 rows)", lambda: seqmix.gated_delta_scan(q1d, k1d, v1d, b1, a1c, al, db_c, st8, s8, l1, False),
        bytes_=Bd * Hd * Dd * Vd * 8)
    add("pinirax gated_delta_scan decode, decay per head (8 rows)", lambda: seqmix.gated_delta_scan(q1d, k1d, v1d, b1, a1h, al, db_h, st8, s8, l1, False),
        bytes_=Bd * Hd * Dd * Vd * 8, like="gated_delta_scan per channel, decode")
    # head-mixing attention beside the window attention of Pinirax
    H, G, D, chunk = 16, 4, 128, 1024
    q, k = rnd(B, S, H, D), rnd(B, S, G, D)
    mixw = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev)) * D ** -0.5
    inv = seqmix.rotary_inv_freq(D, 10000.0, dev)
    kc, vc = torch.zeros(B, chunk, G, D, dtype=bf, device=dev), torch.zeros(B, chunk, G, D, dtype=bf, device=dev)
    add("headmix_qk_prepare (rotation, 16 x 16 mixing onto the queries, rings)",
        lambda: seqmix.headmix_qk_prepare(q, k, mixw, D, inv, pos0, lens, slots, kc, vc, True),
        N * (H * D * 2 + G * D * 2 + H * G * D * 2 + G * D * 2) + B * chunk * G * D * 4)
    v = rnd(B, S, G, D)
    qw = torch.ones(D, device=dev)
    add("pinirax window_qk_prepare (head norms in place + ring store)", lambda: seqmix.window_qk_prepare(q, k, v, qw, qw, 1e-6, pos0, lens, slots, kc, vc),
        N * (H + G) * D * 4 + B * chunk * G * 2 * D * 4, like="headmix_qk_prepare")
    qmix, krows = seqmix.headmix_qk_prepare(q, k, mixw, D, inv, pos0, lens, slots, kc, vc, True)
    sink, gate = torch.zeros(H, device=dev), rnd(B, S, H * D)
    out = torch.empty(N, H * D, dtype=bf, device=dev)
    pairs_c = B * H * sum((p % chunk) + 1 for p in range(S))
    add("headmix_attention_prompt (16 heads, key 4 x 128, value 128, chunk 1024, sink, gate)",
        lambda: seqmix.headmix_attention_prompt(qmix, krows, k, sink, gate, lens, chunk, 0, out), flops=pairs_c * 2 * (G * D + D))
    pairs_w = B * H * sum(min(p + 1, chunk) for p in range(S))
    hgate = rnd(B, S, H)
    add("pinirax window_attention_prompt (GQA 16/4 x 128, window 1024, cap, gate)",
        lambda: seqmix.window_attention_prompt(q, k, v, hgate, lens, chunk, 0.088, 30.0, out, 0.8), flops=pairs_w * 2 * (D + D), like="headmix_attention_prompt")
    qm1, g1 = rnd(Bd, 1, H, G * D), rnd(Bd, 1, H * D)
    kc8, vc8 = rnd(Bd, chunk, G, D), rnd(Bd, chunk, G, D)
    p8c = torch.full((Bd,), 2047, dtype=i32, device=dev)                      # the last position of a chunk: the whole ring is visible
    o1 = torch.empty(Bd, H * D, dtype=bf, device=dev)
    add("headmix_attention_token (8 rows, ring 1024, 4 KV heads)",
        lambda: seqmix.headmix_attention_token(qm1, kc8, vc8, sink, g1, s8, p8c, l1, chunk, 0, o1), bytes_=Bd * chunk * G * D * 4)
    q1, hg1 = rnd(Bd, 1, H, D), rnd(Bd, 1, H)
    add("pinirax window_attention_token (8 rows, ring 1024, 4 KV heads)",
        lambda: seqmix.window_attention_token(q1, kc8, vc8, hg1, s8, p8, l1, chunk, 0.088, 30.0, o1, 0.8), bytes_=Bd * chunk * G * D * 4,
        like="headmix_attention_token")
    return {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src}, "rows": rows}


def main(args) -> int:
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29539")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    from neuronx_distributed_b200.parallel_layers import parallel_state as ps

    ps.initialize_model_parallel(tensor_model_parallel_size=1)
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    out = {"mode": "pulenex", "dtype": "bf16", "data": "synthetic", "steps": steps, "warmup": warmup, "n_gpus": 1,
           "l2": "weights of every model exceed L2; kernel rows flush L2 between iterations"}
    shapes = [(4, 2048), (1, 8192), (8, 512)]
    for name, make in (("pulenex", build_pulenex), ("naguzen", base.build_naguzen), ("pinirax", pin.build_pinirax)):
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
