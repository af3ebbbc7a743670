// Python bindings of the head-mixing attention (scores mixed across heads before a softmax with a sink; keys that double as values).
#include "bind_common.h"

// q [B,S,H,D], k [B,S,G,D] (views: last dim contiguous, heads one after another), mixw float [H,H] → {Q' [B,S,H,G*D], rotated key
// rows [B,S,G,D] or an empty tensor}; kcache / vcache [slots, ring, G, D]
std::vector<Tensor> headmix_qk_prepare(const Tensor& q, const Tensor& k, const Tensor& mixw, int64_t dims, const Tensor& inv_freq,
                                       const Tensor& pos0, const Tensor& lens, const Tensor& slots, Tensor kcache, Tensor vcache,
                                       bool want_rows) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1, "q, k must be [B,S,heads,D] views");
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), G = k.size(2);
    TORCH_CHECK(k.size(0) == B && k.size(1) == S && k.size(3) == D && H % G == 0 && (H == 1 || q.stride(2) == D) && (G == 1 || k.stride(2) == D),
                "heads must be laid out one after another");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && kcache.scalar_type() == k.scalar_type() && vcache.scalar_type() == k.scalar_type(), "dtype mismatch");
    TORCH_CHECK(dims % 2 == 0 && dims <= D && inv_freq.numel() == dims / 2 && mixw.numel() == (long)H * H, "bad rotary / mixing sizes");
    TORCH_CHECK(kcache.is_contiguous() && vcache.is_contiguous() && kcache.dim() == 4 && kcache.sizes() == vcache.sizes() && kcache.size(2) == G &&
                    kcache.size(3) == D, "rings must be [slots, ring, G, D]");
    TORCH_CHECK((size_t)H * D * 4 <= 96 * 1024, "query heads do not fit on chip");
    is_bf(q);
    Tensor qmix = at::empty({B, S, H, (long)G * D}, q.options());
    Tensor rows = want_rows ? at::empty({B, S, G, D}, q.options()) : at::empty({0}, q.options());
    seqmix::headmix_qk_prepare(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), is_bf(q), f32(mixw), (int)dims,
                               f32(inv_freq), i32(pos0), i32(lens), i32(slots), kcache.data_ptr(), vcache.data_ptr(), (int)kcache.size(1),
                               qmix.data_ptr(), want_rows ? rows.data_ptr() : nullptr, B, S, H, G, D, stream());
    check_launch();
    return {qmix, rows};
}

static void gate_strides(const c10::optional<Tensor>& gate, const Tensor& like, int B, int S, int C, const void*& p, long& sb, long& st) {
    p = nullptr; sb = st = 0;
    if (!gate) return;
    TORCH_CHECK(gate->dim() == 3 && gate->size(0) == B && gate->size(1) == S && gate->size(2) == C && gate->stride(2) == 1 &&
                    gate->scalar_type() == like.scalar_type(), "gate must be [B,S,H*D] of the queries' dtype");
    p = gate->data_ptr(); sb = gate->stride(0); st = gate->stride(1);
}

// qmix [B,S,H,G*D], krows [B,S,G,D] contiguous, v [B,S,G,D] view, out [B*S, >= H*D] (row stride free)
void headmix_attention_prompt(const Tensor& qmix, const Tensor& krows, const Tensor& v, const c10::optional<Tensor>& sink,
                              const c10::optional<Tensor>& gate, const Tensor& lens, int64_t chunk, int64_t window, Tensor out) {
    TORCH_CHECK(qmix.is_cuda() && qmix.dim() == 4 && qmix.is_contiguous() && krows.dim() == 4 && krows.is_contiguous() && v.dim() == 4 &&
                    v.stride(3) == 1, "bad attention operands");
    const int B = qmix.size(0), S = qmix.size(1), H = qmix.size(2), G = krows.size(2), D = krows.size(3);
    TORCH_CHECK(qmix.size(3) == (long)G * D && krows.size(0) == B && krows.size(1) == S && v.sizes() == krows.sizes() &&
                    (G == 1 || v.stride(2) == D) && H % G == 0, "shape mismatch");
    TORCH_CHECK(qmix.scalar_type() == krows.scalar_type() && qmix.scalar_type() == v.scalar_type() && out.scalar_type() == qmix.scalar_type(), "dtype mismatch");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == (long)B * S && out.size(1) >= (long)H * D && out.stride(1) == 1, "out must be [B*S, >= H*D]");
    const void* gp; long g_sb, g_st;
    gate_strides(gate, qmix, B, S, H * D, gp, g_sb, g_st);
    const float* sk = sink ? f32(*sink) : nullptr;
    if (sink) TORCH_CHECK(sink->numel() == H, "one sink per head");
    if (is_bf(qmix) && seqmix::headmix_prompt_mma_fits(v.data_ptr(), v.stride(0), v.stride(1), G, D, out.data_ptr(), out.stride(0))) {
        seqmix::headmix_prompt_mma(qmix.data_ptr(), krows.data_ptr(), v.data_ptr(), v.stride(0), v.stride(1), sk, gp, g_sb, g_st, i32(lens), B, S,
                                   H, G, D, (int)chunk, (int)window, out.data_ptr(), out.stride(0), stream());
    } else {
        bool ok = seqmix::headmix_attend(qmix.data_ptr(), krows.data_ptr(), (long)S * G * D, v.data_ptr(), v.stride(0), v.stride(1), is_bf(qmix),
                                         sk, gp, g_sb, g_st, nullptr, nullptr, i32(lens), (int)chunk, (int)window, 0, B, S, H, G, D,
                                         out.data_ptr(), out.stride(0), stream());
        TORCH_CHECK(ok, "headmix_attention_prompt: head size ", D, " with ", G, " key heads does not fit");
    }
    check_launch();
}

// qmix [B,1,H,G*D]; kcache / vcache [slots, ring, G, D]; out [B, >= H*D]
void headmix_attention_token(const Tensor& qmix, const Tensor& kcache, const Tensor& vcache, const c10::optional<Tensor>& sink,
                             const c10::optional<Tensor>& gate, const Tensor& slots, const Tensor& pos0, const Tensor& lens, int64_t chunk,
                             int64_t window, Tensor out) {
    TORCH_CHECK(qmix.is_cuda() && qmix.dim() == 4 && qmix.is_contiguous() && qmix.size(1) == 1 && kcache.dim() == 4 && kcache.is_contiguous() &&
                    vcache.is_contiguous() && vcache.sizes() == kcache.sizes(), "bad attention operands");
    const int B = qmix.size(0), H = qmix.size(2), ring = kcache.size(1), G = kcache.size(2), D = kcache.size(3);
    TORCH_CHECK(qmix.size(3) == (long)G * D && H % G == 0, "shape mismatch");
    TORCH_CHECK(qmix.scalar_type() == kcache.scalar_type() && qmix.scalar_type() == vcache.scalar_type() && out.scalar_type() == qmix.scalar_type(),
                "dtype mismatch");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == B && out.size(1) >= (long)H * D && out.stride(1) == 1, "out must be [B, >= H*D]");
    const void* gp; long g_sb, g_st;
    gate_strides(gate, qmix, B, 1, H * D, gp, g_sb, g_st);
    if (sink) TORCH_CHECK(sink->numel() == H, "one sink per head");
    if (seqmix::headmix_token_fits(is_bf(qmix), H, G, D, ring, qmix.data_ptr(), kcache.data_ptr(), vcache.data_ptr())) {
        Tensor part = at::empty({B, seqmix::headmix_token_stretches(ring), H, D + 2}, qmix.options().dtype(at::kFloat));
        seqmix::headmix_token(qmix.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), is_bf(qmix), sink ? f32(*sink) : nullptr, gp, g_sb,
                              i32(slots), i32(pos0), i32(lens), (int)chunk, (int)window, ring, B, H, G, D, part.data_ptr<float>(),
                              out.data_ptr(), out.stride(0), stream());
        check_launch();
        return;
    }
    bool ok = seqmix::headmix_attend(qmix.data_ptr(), kcache.data_ptr(), (long)ring * G * D, vcache.data_ptr(), (long)ring * G * D, (long)G * D,
                                     is_bf(qmix), sink ? f32(*sink) : nullptr, gp, g_sb, g_st, i32(slots), i32(pos0), i32(lens), (int)chunk,
                                     (int)window, ring, B, 1, H, G, D, out.data_ptr(), out.stride(0), stream());
    TORCH_CHECK(ok, "headmix_attention_token: head size ", D, " with ", G, " key heads does not fit");
    check_launch();
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("headmix_qk_prepare", &headmix_qk_prepare);
    m.def("headmix_attention_prompt", &headmix_attention_prompt);
    m.def("headmix_attention_token", &headmix_attention_token);
}
