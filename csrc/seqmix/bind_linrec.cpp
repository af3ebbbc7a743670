// Python bindings of the gated linear recurrences with a decay per channel (gated linear attention, real-gated LRU).
#include "bind_common.h"

// q,k [B,S,H,D], v [B,S,H,V] (views with equal batch / token strides), z [B,S,H*D] → o float [B,S,H,V]; state [slots,H,D,V] float
// Runs of at least this many tokens take the chunked form (matrix products); shorter ones and single tokens the token by token scan.
static const int kGlaChunkedFrom = 32;

// Float matrix products stay true float here whatever the process-wide setting is: they carry the recurrence.
struct FloatProducts {
    bool was;
    FloatProducts() : was(at::globalContext().allowTF32CuBLAS()) { at::globalContext().setAllowTF32CuBLAS(false); }
    ~FloatProducts() { at::globalContext().setAllowTF32CuBLAS(was); }
};

static Tensor gla_scan_chunked(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const float* zbias, double tau,
                               float qscale, const float* decay, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), V = v.size(3), C = seqmix::gla_chunk_tokens();
    const auto f = q.options().dtype(at::kFloat);
    const long es = q.element_size();
    // the states before every chunk are materialised ([chunks, D, V] floats per head): long prompts go segment by segment
    const long per_chunk = (long)B * H * D * V * 4;
    const long seg_chunks = std::max<long>(1, (1L << 30) / per_chunk);
    const long seg = seg_chunks * C;
    Tensor out = at::empty({B, S, H, V}, f);
    FloatProducts guard;
    for (long s0 = 0; s0 < S; s0 += seg) {
        const int Sg = (int)std::min<long>(seg, S - s0), nC = (Sg + C - 1) / C;
        const long n = (long)B * H * nC;
        Tensor lens_g = s0 == 0 ? lens : (lens - (int)s0).clamp_min(0).to(at::kInt).contiguous();
        Tensor Qe = at::empty({n, C, D}, f), Ke = at::empty({n, C, D}, f), Bc = at::empty({n, C, D}, f), G = at::empty({n, D}, f);
        Tensor Vf = at::empty({n, C, V}, f), A = at::empty({n, C, C}, f);
        const char *qp = (const char*)q.data_ptr() + s0 * q.stride(1) * es, *kp = (const char*)k.data_ptr() + s0 * k.stride(1) * es;
        const char *vp = (const char*)v.data_ptr() + s0 * v.stride(1) * es, *zp = (const char*)z.data_ptr() + s0 * z.stride(1) * es;
        seqmix::gla_chunk_prep(qp, kp, vp, is_bf(q), q.stride(0), q.stride(1), zp, z.stride(0), z.stride(1), zbias, (float)(1.0 / tau),
                               qscale, decay, i32(lens_g), B, Sg, H, D, V, nC, Qe.data_ptr<float>(),
                               Ke.data_ptr<float>(), Bc.data_ptr<float>(), G.data_ptr<float>(), Vf.data_ptr<float>(), A.data_ptr<float>(),
                               stream());
        check_launch();
        Tensor Sl = at::bmm(Ke.transpose(1, 2), Vf);                                             // [n, D, V]
        seqmix::gla_carry(Sl.data_ptr<float>(), G.data_ptr<float>(), state.data_ptr<float>(), i32(slots), fresh && s0 == 0, B, nC, H, D, V,
                          stream());
        check_launch();
        Tensor O = at::baddbmm(at::bmm(A, Vf), Qe, Sl);                                          // [n, C, V]
        out.slice(1, s0, s0 + Sg).copy_(O.view({B, H, (long)nC * C, V}).slice(2, 0, Sg).permute({0, 2, 1, 3}));
    }
    return out;
}

static Tensor linear_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const float* zbias, double tau, float qscale,
                          const float* decay, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && v.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && z.stride(2) == 1,
                "bad recurrence operands");
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), V = v.size(3);
    TORCH_CHECK(H == 1 || (q.stride(2) == D && k.stride(2) == D && v.stride(2) == V), "heads must be laid out one after another");
    TORCH_CHECK((B == 1 || (q.stride(0) == k.stride(0) && q.stride(0) == v.stride(0))) &&
                    (S == 1 || (q.stride(1) == k.stride(1) && q.stride(1) == v.stride(1))),
                "q, k, v must share their batch and token strides");   // a stride of a dimension of size 1 is never used
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == H && state.size(2) == D && state.size(3) == V,
                "state must be float [slots,H,D,V]");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type() && q.scalar_type() == z.scalar_type(), "dtype mismatch");
    if (S >= kGlaChunkedFrom) return gla_scan_chunked(q, k, v, z, zbias, tau, qscale, decay, state, slots, lens, fresh);
    Tensor out = at::empty({B, S, H, V}, q.options().dtype(at::kFloat));
    if (S == 1 && seqmix::gla_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), is_bf(q), q.stride(0), z.data_ptr(), z.stride(0), zbias,
                                   (float)(1.0 / tau), qscale, decay, state.data_ptr<float>(), i32(slots), i32(lens),
                                   fresh, B, H, D, V, out.data_ptr<float>(), stream())) {
        check_launch();
        return out;
    }
    bool ok = seqmix::gla_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), is_bf(q), q.stride(0), q.stride(1), z.data_ptr(), z.stride(0),
                               z.stride(1), zbias, (float)(1.0 / tau), qscale, decay, state.data_ptr<float>(),
                               i32(slots), i32(lens), fresh, B, S, H, D, V, out.data_ptr<float>(), stream());
    TORCH_CHECK(ok, "linear scan: no launch shape for key size ", D, " and value size ", V);
    check_launch();
    return out;
}

Tensor gla_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const Tensor& zbias, double tau, Tensor state,
                const Tensor& slots, const Tensor& lens, bool fresh) {
    return linear_scan(q, k, v, z, f32(zbias), tau, (float)(1.0 / std::sqrt((double)q.size(3))), nullptr, state, slots, lens, fresh);
}

// Retention: the same scans with ONE fixed decay per head (decay float [H]) and no scale on the queries; q stands in for the unused z.
Tensor retention_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& decay, Tensor state, const Tensor& slots,
                      const Tensor& lens, bool fresh) {
    TORCH_CHECK(q.dim() == 4 && decay.numel() == q.size(2), "one decay per head");
    return linear_scan(q, k, v, q.flatten(2), nullptr, 1.0, 1.f, f32(decay), state, slots, lens, fresh);
}

// u [B,S,W] contiguous, gr / gi float [blocks, B*S, W/blocks], y [B,S,W] view (pre-activation) → out [B,S,W]; state [slots, W] float
Tensor rglru_scan(const Tensor& u, const Tensor& gr, const Tensor& gi, const Tensor& rbias, const Tensor& ibias, const Tensor& lam_sp,
                  const Tensor& y, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(u.is_cuda() && u.dim() == 3 && u.is_contiguous() && y.dim() == 3 && y.stride(2) == 1 && gr.dim() == 3, "bad operands");
    const int B = u.size(0), S = u.size(1), W = u.size(2), wb = gr.size(2);
    TORCH_CHECK(gr.size(0) * wb == W && gr.size(1) == (long)B * S && gi.sizes() == gr.sizes() && u.scalar_type() == y.scalar_type(), "bad gates");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == W, "state must be float [slots, W]");
    Tensor out = at::empty({B, S, W}, u.options());
    seqmix::rglru_scan(u.data_ptr(), is_bf(u), f32(gr), f32(gi), wb, f32(rbias), f32(ibias), f32(lam_sp), y.data_ptr(), y.stride(0), y.stride(1),
                       state.data_ptr<float>(), i32(slots), i32(lens), fresh, B, S, W, out.data_ptr(), stream());
    check_launch();
    return out;
}

// zraw, uraw, graw [B,S,W]: views with the same strides (parts of one stacked projection) → out [B,S,W]; state [slots, W] float
Tensor mingru_scan(const Tensor& z, const Tensor& u, const Tensor& g, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(z.is_cuda() && z.dim() == 3 && z.stride(2) == 1 && u.sizes() == z.sizes() && g.sizes() == z.sizes() && u.strides() == z.strides() &&
                    g.strides() == z.strides() && u.scalar_type() == z.scalar_type() && g.scalar_type() == z.scalar_type(),
                "z, u, g must be [B,S,W] views with the same strides and dtype");
    const int B = z.size(0), S = z.size(1), W = z.size(2);
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.dim() == 2 && state.size(1) == W, "state must be float [slots, W]");
    TORCH_CHECK(slots.numel() == B && lens.numel() == B, "one slot and one length per row");
    Tensor out = at::empty({B, S, W}, z.options());
    seqmix::mingru_scan(z.data_ptr(), u.data_ptr(), g.data_ptr(), is_bf(z), z.stride(0), z.stride(1), state.data_ptr<float>(), i32(slots),
                        i32(lens), fresh, B, S, W, out.data_ptr(), stream());
    check_launch();
    return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("mingru_scan", &mingru_scan);
    m.def("gla_scan", &gla_scan);
    m.def("retention_scan", &retention_scan);
    m.def("rglru_scan", &rglru_scan);
}
