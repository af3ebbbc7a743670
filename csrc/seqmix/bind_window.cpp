// Python bindings of the grouped-query sliding-window attention kernels.
#include "bind_common.h"

static const float* opt_f32(const c10::optional<Tensor>& t) { return t ? f32(*t) : nullptr; }

// q [B,S,H,D], k [B,S,G,D], v [B,S,G,V] (views; last dim contiguous, heads one after another); caches [slots, ring, G, D|V].
// qw / kw: D numbers (a norm per head) or H*D / G*D numbers (one norm over all heads).  inv_freq: dims/2 rotation frequencies.
// Without k (then also without v and the caches) only the queries are prepared.
void window_qk_prepare(Tensor q, const c10::optional<Tensor>& k, const c10::optional<Tensor>& v, const c10::optional<Tensor>& qw,
                       const c10::optional<Tensor>& kw, bool norm_all, double eps, const c10::optional<Tensor>& inv_freq, int64_t dims,
                       const Tensor& pos0,
                       const Tensor& lens, const Tensor& slots, const c10::optional<Tensor>& kcache, const c10::optional<Tensor>& vcache) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.stride(3) == 1, "bad attention operands");
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3);
    TORCH_CHECK(H == 1 || q.stride(2) == D, "heads must be laid out one after another");
    int G = 1, V = 1, ring = 1;
    if (k) {
        TORCH_CHECK(v && kcache && vcache, "keys come with values and both caches");
        TORCH_CHECK(k->dim() == 4 && v->dim() == 4 && k->stride(3) == 1 && v->stride(3) == 1, "bad attention operands");
        G = k->size(2); V = v->size(3); ring = kcache->size(1);
        TORCH_CHECK(k->size(3) == D && v->size(2) == G && H % G == 0 && (G == 1 || (k->stride(2) == D && v->stride(2) == V)),
                    "heads must be laid out one after another");
        TORCH_CHECK(q.scalar_type() == k->scalar_type() && q.scalar_type() == v->scalar_type() && kcache->scalar_type() == q.scalar_type() &&
                        vcache->scalar_type() == q.scalar_type(), "dtype mismatch");
        TORCH_CHECK(kcache->is_contiguous() && vcache->is_contiguous() && kcache->dim() == 4 && vcache->dim() == 4 &&
                        kcache->size(1) == vcache->size(1) && kcache->size(2) == G && kcache->size(3) == D && vcache->size(2) == G &&
                        vcache->size(3) == V, "caches must be [slots, ring, G, D|V]");
    }
    const bool all = norm_all;
    TORCH_CHECK(!qw || qw->numel() == (all ? (long)H * D : D), "query norm weights must hold D or H*D numbers");
    TORCH_CHECK(!kw || !k || kw->numel() == (all ? (long)G * D : D), "key norm weights must hold D or G*D numbers");
    if (inv_freq) TORCH_CHECK(dims >= 0 && dims % 2 == 0 && dims <= D && inv_freq->numel() == dims / 2, "rotation: dims/2 frequencies, dims <= D");
    seqmix::window_qk_prepare(q.data_ptr(), q.stride(0), q.stride(1), k ? k->data_ptr() : nullptr, k ? k->stride(0) : 0, k ? k->stride(1) : 0,
                              v ? v->data_ptr() : nullptr, v ? v->stride(0) : 0, v ? v->stride(1) : 0, is_bf(q), opt_f32(qw),
                              k ? opt_f32(kw) : nullptr, all, (float)eps, inv_freq ? f32(*inv_freq) : nullptr, inv_freq ? (int)dims : 0, i32(pos0),
                              i32(lens), i32(slots), kcache ? kcache->data_ptr() : nullptr, vcache ? vcache->data_ptr() : nullptr, ring, B, S,
                              H, G, D, V, stream());
    check_launch();
}

static const float* bias_ptr(const c10::optional<Tensor>& b, int H) {
    if (!b) return nullptr;
    TORCH_CHECK(b->numel() == H, "the score bias holds one number per query head");
    return f32(*b);
}

static void check_out(const Tensor& out, long rows, long cols, const Tensor& like) {
    TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == rows && out.size(1) >= cols && out.stride(1) == 1 &&
                    out.scalar_type() == like.scalar_type(), "out must be [rows, >= heads * vdim] of the activations' dtype");
}

void window_attention_prompt(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& gate, const Tensor& lens,
                             int64_t window, double scale, double softcap, const c10::optional<Tensor>& score_bias, Tensor out,
                             double out_scale) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1,
                "bad attention operands");
    const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), G = k.size(2), V = v.size(3);
    TORCH_CHECK(k.size(3) == D && v.size(2) == G && H % G == 0 && (H == 1 || q.stride(2) == D) && (G == 1 || (k.stride(2) == D && v.stride(2) == V)),
                "heads must be laid out one after another");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(), "dtype mismatch");
    check_out(out, (long)B * S, (long)H * V, q);
    const void* gp = nullptr;
    long g_sb = 0, g_st = 0;
    if (gate) {
        TORCH_CHECK(gate->dim() == 3 && gate->size(2) == H && gate->stride(2) == 1 && gate->scalar_type() == q.scalar_type(), "gate must be [B,S,H]");
        gp = gate->data_ptr(); g_sb = gate->stride(0); g_st = gate->stride(1);
    }
    bool ok = seqmix::window_attention_prompt(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(),
                                              v.stride(0), v.stride(1), gp, g_sb, g_st, is_bf(q), i32(lens), B, S, H, G, D, V, (int)window,
                                              (float)scale, (float)softcap, bias_ptr(score_bias, H), out.data_ptr(), out.stride(0),
                                              (float)out_scale, stream());
    TORCH_CHECK(ok, "window_attention_prompt: sizes do not fit the kernel (vdim <= 512)");
    check_launch();
}

void window_attention_token(const Tensor& q, const Tensor& kcache, const Tensor& vcache, const c10::optional<Tensor>& gate, const Tensor& slots,
                            const Tensor& pos0, const Tensor& lens, int64_t window, double scale, double softcap,
                            const c10::optional<Tensor>& score_bias, Tensor out, double out_scale) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.size(1) == 1 && q.stride(3) == 1 && kcache.dim() == 4 && vcache.dim() == 4 &&
                    kcache.is_contiguous() && vcache.is_contiguous(), "bad attention operands");
    const int B = q.size(0), H = q.size(2), D = q.size(3), G = kcache.size(2), V = vcache.size(3), ring = kcache.size(1);
    TORCH_CHECK(kcache.size(3) == D && vcache.size(2) == G && vcache.size(1) == ring && H % G == 0 && (H == 1 || q.stride(2) == D), "shape mismatch");
    TORCH_CHECK(q.scalar_type() == kcache.scalar_type() && q.scalar_type() == vcache.scalar_type(), "dtype mismatch");
    check_out(out, B, (long)H * V, q);
    const void* gp = nullptr;
    long g_sb = 0;
    if (gate) {
        TORCH_CHECK(gate->dim() == 3 && gate->size(2) == H && gate->stride(2) == 1 && gate->scalar_type() == q.scalar_type(), "gate must be [B,1,H]");
        gp = gate->data_ptr(); g_sb = gate->stride(0);
    }
    const int splits = seqmix::window_token_splits(ring, B, H, G);
    const auto f = q.options().dtype(at::kFloat);
    Tensor pm = at::empty({B, H, splits}, f), pl = at::empty({B, H, splits}, f), pa = at::empty({B, H, splits, V}, f);
    bool ok = seqmix::window_attention_token(q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), gp, g_sb, is_bf(q), i32(slots),
                                             i32(pos0), i32(lens), ring, B, H, G, D, V, (int)window, (float)scale, (float)softcap,
                                             bias_ptr(score_bias, H), splits,
                                             pm.data_ptr<float>(), pl.data_ptr<float>(), pa.data_ptr<float>(), out.data_ptr(),
                                             out.stride(0), (float)out_scale, stream());
    TORCH_CHECK(ok, "window_attention_token: sizes do not fit the kernel (vdim <= 512)");
    check_launch();
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("window_qk_prepare", &window_qk_prepare);
    m.def("window_attention_prompt", &window_attention_prompt);
    m.def("window_attention_token", &window_attention_token);
}
