// Python bindings of the matrix-state recurrences with a scalar decay per head (gated delta rule, selective state space).
#include "bind_common.h"

static void same_tokens(const Tensor& a, const Tensor& b, const char* what) {
    TORCH_CHECK((a.size(0) == 1 || a.stride(0) == b.stride(0)) && (a.size(1) == 1 || a.stride(1) == b.stride(1)), what,
                " must share their batch and token strides");
}

// q, k [B,S,G,D], v [B,S,H,V] (views: last dim contiguous, heads one after another), braw / araw float [B,S,H] views of one
// tensor → o float [B,S,H,V]; state [slots,H,D,V] float
Tensor gated_delta_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& braw, const Tensor& araw, const Tensor& a_log,
                        const Tensor& dt_bias, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1,
                "bad recurrence operands");
    const int B = q.size(0), S = q.size(1), G = q.size(2), D = q.size(3), H = v.size(2), V = v.size(3);
    TORCH_CHECK(k.sizes() == q.sizes() && H % G == 0 && (G == 1 || (q.stride(2) == D && k.stride(2) == D)) && (H == 1 || v.stride(2) == V),
                "heads must be laid out one after another");
    same_tokens(q, k, "q and k");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(), "dtype mismatch");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == H && state.size(2) == D && state.size(3) == V,
                "state must be float [slots,H,D,V]");
    Tensor out = at::empty({B, S, H, V}, q.options().dtype(at::kFloat));
    TORCH_CHECK(braw.scalar_type() == at::kFloat && araw.scalar_type() == at::kFloat && braw.dim() == 3 && braw.size(0) == B &&
                    braw.size(1) == S && braw.size(2) == H && braw.stride(2) == 1, "beta pre-activations must be float [B,S,H]");
    if (araw.dim() == 4) {                       // a decay per head and key channel
        TORCH_CHECK(araw.size(0) == B && araw.size(1) == S && araw.size(2) == H && araw.size(3) == D && araw.stride(3) == 1 &&
                        (H == 1 || araw.stride(2) == D) && dt_bias.numel() == (long)H * D && a_log.numel() == H,
                    "decay pre-activations per channel must be float [B,S,H,D], dt_bias [H*D]");
        bool okc = seqmix::gated_delta_channel_scan(q.data_ptr(), k.data_ptr(), q.stride(0), q.stride(1), v.data_ptr(), v.stride(0), v.stride(1),
                                                    is_bf(q), braw.data_ptr<float>(), braw.stride(0), braw.stride(1), araw.data_ptr<float>(),
                                                    araw.stride(0), araw.stride(1), f32(a_log), f32(dt_bias), state.data_ptr<float>(), i32(slots),
                                                    i32(lens), fresh, B, S, H, G, D, V, (float)(1.0 / std::sqrt((double)D)),
                                                    out.data_ptr<float>(), stream());
        TORCH_CHECK(okc, "gated_delta_scan: key size ", D, " does not fit");
        check_launch();
        return out;
    }
    TORCH_CHECK(araw.sizes() == braw.sizes() && araw.stride(2) == 1 && dt_bias.numel() == H, "decay pre-activations must be float [B,S,H]");
    same_tokens(braw, araw, "beta and decay pre-activations");
    bool ok = seqmix::gated_delta_scan(q.data_ptr(), k.data_ptr(), q.stride(0), q.stride(1), v.data_ptr(), v.stride(0), v.stride(1), is_bf(q),
                                       braw.data_ptr<float>(), araw.data_ptr<float>(), braw.stride(0), braw.stride(1), f32(a_log),
                                       f32(dt_bias), state.data_ptr<float>(), i32(slots), i32(lens), fresh, B, S, H, G, D, V,
                                       (float)(1.0 / std::sqrt((double)D)), out.data_ptr<float>(), stream());
    TORCH_CHECK(ok, "gated_delta_scan: key size ", D, " does not fit");
    check_launch();
    return out;
}

// x [B,S,H,V], bm / cm [B,S,G,N] (views), dtraw float [B,S,H] → y float [B,S,H,V]; state [slots,H,N,V] float
Tensor ssd_scan(const Tensor& x, const Tensor& bm, const Tensor& cm, const Tensor& dtraw, const Tensor& a_log, const Tensor& dt_bias,
                const Tensor& dskip, Tensor state, const Tensor& slots, const Tensor& lens, bool fresh) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && bm.dim() == 4 && cm.sizes() == bm.sizes() && x.stride(3) == 1 && bm.stride(3) == 1 &&
                    cm.stride(3) == 1, "bad recurrence operands");
    const int B = x.size(0), S = x.size(1), H = x.size(2), V = x.size(3), G = bm.size(2), N = bm.size(3);
    TORCH_CHECK(H % G == 0 && (H == 1 || x.stride(2) == V) && (G == 1 || (bm.stride(2) == N && cm.stride(2) == N)),
                "heads must be laid out one after another");
    same_tokens(bm, cm, "b and c");
    TORCH_CHECK(x.scalar_type() == bm.scalar_type() && x.scalar_type() == cm.scalar_type(), "dtype mismatch");
    TORCH_CHECK(dtraw.scalar_type() == at::kFloat && dtraw.dim() == 3 && dtraw.size(2) == H && dtraw.stride(2) == 1, "step sizes must be float [B,S,H]");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.size(1) == H && state.size(2) == N && state.size(3) == V,
                "state must be float [slots,H,N,V]");
    Tensor out = at::empty({B, S, H, V}, x.options().dtype(at::kFloat));
    bool ok = seqmix::ssd_scan(x.data_ptr(), x.stride(0), x.stride(1), bm.data_ptr(), cm.data_ptr(), bm.stride(0), bm.stride(1), is_bf(x),
                               dtraw.data_ptr<float>(), dtraw.stride(0), dtraw.stride(1), f32(a_log), f32(dt_bias), f32(dskip),
                               state.data_ptr<float>(), i32(slots), i32(lens), fresh, B, S, H, G, N, V, out.data_ptr<float>(), stream());
    TORCH_CHECK(ok, "ssd_scan: state size ", N, " does not fit");
    check_launch();
    return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("gated_delta_scan", &gated_delta_scan);
    m.def("ssd_scan", &ssd_scan);
}
