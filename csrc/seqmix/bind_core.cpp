// Python bindings of the kernels every sequence-mixer model uses: short convolutions, norms, activations, embedding with sinusoids,
// the small-batch pieces of a routed feed-forward.
#include "bind_common.h"

// x [B,S,C] (last dim contiguous), w [C,taps], state [slots, taps-1, C] of x's dtype → out [B,S,C] of `out_bf16`'s dtype
Tensor short_conv(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, Tensor state, const Tensor& slots,
                  const Tensor& lens, bool fresh, bool residual, bool out_bf16, bool silu) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.stride(2) == 1, "x must be [B,S,C] with a contiguous last dimension");
    const int B = x.size(0), S = x.size(1), C = x.size(2), taps = w.size(1);
    TORCH_CHECK(w.size(0) == C && taps >= 1 && taps <= 16, "taps must be 1..16");
    TORCH_CHECK(state.is_contiguous() && state.scalar_type() == x.scalar_type() && state.size(1) == taps - 1 && state.size(2) == C,
                "history must be [slots, taps-1, C] of the input's dtype");
    Tensor out = at::empty({B, S, C}, x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
    seqmix::short_conv(x.data_ptr(), is_bf(x), x.stride(0), x.stride(1), f32(w), bias ? f32(*bias) : nullptr, state.data_ptr(),
                       i32(slots), i32(lens), B, S, C, taps, fresh, residual, silu, out.data_ptr(), out_bf16, stream());
    check_launch();
    return out;
}

// rows of x ([rows, C], row stride free) → out [rows, C] contiguous; w float [C] or one number
Tensor rms_norm(const Tensor& x, const Tensor& w, double eps, const c10::optional<Tensor>& gate, bool out_bf16, bool center) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "x must be [rows, C] with a contiguous last dimension");
    const int rows = x.size(0), C = x.size(1);
    TORCH_CHECK(w.numel() == 1 || w.numel() == C, "weight must hold 1 or C numbers");
    Tensor out = at::empty({rows, C}, x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
    const void* g = nullptr;
    long gs = 0;
    if (gate) {
        TORCH_CHECK(gate->scalar_type() == out.scalar_type() && gate->dim() == 2 && gate->stride(1) == 1, "gate must match the output");
        g = gate->data_ptr();
        gs = gate->stride(0);
    }
    if (rows)
        seqmix::rms_norm(x.data_ptr(), is_bf(x), x.stride(0), rows, C, f32(w), w.numel() == 1 ? 0 : 1, (float)eps, g, gs, out.data_ptr(),
                         out_bf16, C, nullptr, 0, center, stream());
    check_launch();
    return out;
}

// res [rows, C] float += norm(y) * w
void add_rms_norm_(Tensor res, const Tensor& y, const Tensor& w, double eps, bool center) {
    TORCH_CHECK(y.is_cuda() && y.dim() == 2 && y.stride(1) == 1 && res.dim() == 2 && res.stride(1) == 1 && res.scalar_type() == at::kFloat,
                "res must be float [rows, C], y [rows, C]");
    const int rows = y.size(0), C = y.size(1);
    TORCH_CHECK(res.size(0) == rows && res.size(1) == C && (w.numel() == 1 || w.numel() == C), "shape mismatch");
    if (rows)
        seqmix::rms_norm(y.data_ptr(), is_bf(y), y.stride(0), rows, C, f32(w), w.numel() == 1 ? 0 : 1, (float)eps, nullptr, 0, nullptr, 0, 0,
                         res.data_ptr<float>(), res.stride(0), center, stream());
    check_launch();
}

Tensor xielu(const Tensor& x, double ap, double an) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous");
    Tensor out = at::empty_like(x);
    seqmix::xielu(x.data_ptr(), out.data_ptr(), is_bf(x), x.numel(), (float)ap, (float)an, stream());
    check_launch();
    return out;
}

Tensor gelu_erf(const Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous");
    Tensor out = at::empty_like(x);
    seqmix::gelu_erf(x.data_ptr(), out.data_ptr(), is_bf(x), x.numel(), stream());
    check_launch();
    return out;
}

Tensor relu_sq(const Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous");
    Tensor out = at::empty_like(x);
    seqmix::relu_sq(x.data_ptr(), out.data_ptr(), is_bf(x), x.numel(), stream());
    check_launch();
    return out;
}

// w [E,O,I], sel int [M], x [M,I] → act(w[sel[m]] x[m]): [M,O], or [M,O/2] for the gated kind (act 2)
Tensor indexed_gemv(const Tensor& w, const Tensor& sel, const Tensor& x, int64_t act) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 3 && w.is_contiguous() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == w.scalar_type(), "bad gemv operands");
    const int M = x.size(0), E = w.size(0), O = w.size(1), I = w.size(2);
    TORCH_CHECK(x.size(1) == I && sel.numel() == M && act >= 0 && act <= 3 && (act != 2 || O % 2 == 0), "shape mismatch");
    Tensor out = at::empty({M, act == 2 ? O / 2 : O}, x.options());
    seqmix::indexed_gemv(w.data_ptr(), i32(sel), x.data_ptr(), is_bf(x), x.stride(0), M, E, O, I, (int)act, out.data_ptr(), stream());
    check_launch();
    return out;
}

// gu [M, 2F] contiguous → silu(gu[:, :F]) * gu[:, F:]
Tensor silu_mul(const Tensor& gu) {
    TORCH_CHECK(gu.is_cuda() && gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 2 == 0, "gu must be contiguous [M, 2F]");
    Tensor out = at::empty({gu.size(0), gu.size(1) / 2}, gu.options());
    seqmix::silu_mul(gu.data_ptr(), out.data_ptr(), is_bf(gu), gu.size(0), (int)(gu.size(1) / 2), stream());
    check_launch();
    return out;
}

// rows [M,C], src int [N,top], weight float [N,top], base [N,C] or none (times base_weight float [N] if given) → [N,C]
Tensor moe_combine(const Tensor& rows, const Tensor& src, const Tensor& weight, const c10::optional<Tensor>& base,
                   const c10::optional<Tensor>& base_weight) {
    TORCH_CHECK(rows.is_cuda() && rows.dim() == 2 && rows.is_contiguous() && src.dim() == 2, "bad combine operands");
    const int N = src.size(0), top = src.size(1), C = rows.size(1);
    if (base) TORCH_CHECK(base->is_contiguous() && base->scalar_type() == rows.scalar_type() && base->size(0) == N && base->size(1) == C, "bad base");
    if (base_weight) TORCH_CHECK(base && base_weight->numel() == N, "base_weight needs a base and one number per row");
    Tensor out = at::empty({N, C}, rows.options());
    seqmix::moe_combine(rows.data_ptr(), i32(src), f32(weight), base ? base->data_ptr() : nullptr, base_weight ? f32(*base_weight) : nullptr,
                        is_bf(rows), N, top, C, out.data_ptr(), stream());
    check_launch();
    return out;
}

// tokens int64 [B,S], table [vocab, W] → float [B,S,W]
Tensor embed_sinusoid(const Tensor& tokens, const Tensor& table, double scale, const Tensor& inv_freq, const Tensor& pos0) {
    TORCH_CHECK(tokens.is_cuda() && tokens.dim() == 2 && tokens.is_contiguous() && tokens.scalar_type() == at::kLong && table.dim() == 2 &&
                    table.is_contiguous(), "tokens must be contiguous int64 [B,S], table [vocab, W]");
    const int B = tokens.size(0), S = tokens.size(1), W = table.size(1);
    TORCH_CHECK(inv_freq.numel() == (W + 1) / 2 && pos0.numel() == B, "bad position operands");
    Tensor out = at::empty({B, S, W}, table.options().dtype(at::kFloat));
    seqmix::embed_sinusoid(tokens.data_ptr<int64_t>(), table.data_ptr(), is_bf(table), (float)scale, f32(inv_freq), i32(pos0), B, S, W,
                           (int)table.size(0), out.data_ptr<float>(), stream());
    check_launch();
    return out;
}

// tokens int64 [B,S], table [vocab, W], pairs [buckets + 1, W] (optional), prev int64 [slots] (optional) → float [B,S,W] (+ a copy in
// the table's dtype when `want_lp`)
std::vector<Tensor> embed_bigram(const Tensor& tokens, const Tensor& table, double scale, const c10::optional<Tensor>& pairs, int64_t mul_prev,
                                 int64_t mul_cur, const c10::optional<Tensor>& prev, const Tensor& slots, const Tensor& lens, bool fresh,
                                 bool want_lp) {
    TORCH_CHECK(tokens.is_cuda() && tokens.dim() == 2 && tokens.is_contiguous() && tokens.scalar_type() == at::kLong && table.dim() == 2 &&
                    table.is_contiguous(), "tokens must be contiguous int64 [B,S], table [vocab, W]");
    const int B = tokens.size(0), S = tokens.size(1), W = table.size(1);
    long buckets = 0;
    if (pairs) {
        TORCH_CHECK(pairs->dim() == 2 && pairs->is_contiguous() && pairs->size(1) == W && pairs->size(0) >= 2 &&
                        pairs->scalar_type() == table.scalar_type(), "pairs must be [buckets + 1, W] of the table's dtype");
        buckets = pairs->size(0) - 1;
    }
    if (prev) TORCH_CHECK(prev->is_cuda() && prev->scalar_type() == at::kLong && prev->is_contiguous(), "prev must be int64 [slots]");
    TORCH_CHECK(slots.numel() == B && lens.numel() == B, "one slot and one length per row");
    Tensor out = at::empty({B, S, W}, table.options().dtype(at::kFloat));
    Tensor lp = want_lp ? at::empty({B, S, W}, table.options()) : Tensor();
    seqmix::embed_bigram(tokens.data_ptr<int64_t>(), table.data_ptr(), is_bf(table), (float)scale, pairs ? pairs->data_ptr() : nullptr, buckets,
                         mul_prev, mul_cur, prev ? (long*)prev->data_ptr<int64_t>() : nullptr, i32(slots), i32(lens), fresh, B, S, W,
                         (int)table.size(0), out.data_ptr<float>(), want_lp ? lp.data_ptr() : nullptr, stream());
    check_launch();
    return {out, lp};
}

// x float [rows, C] (in place) <- norm(alpha x + sigmoid(gate) y) * w; y, gate [rows, C] views of one dtype; lp: a copy in that dtype
void postnorm_gated_(Tensor x, const Tensor& y, const c10::optional<Tensor>& gate, const Tensor& w, double alpha, double eps,
                     const c10::optional<Tensor>& lp) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kFloat && y.dim() == 2 && y.stride(1) == 1,
                "x must be float [rows, C], y [rows, C]");
    const int rows = x.size(0), C = x.size(1);
    TORCH_CHECK(y.size(0) == rows && y.size(1) == C && w.numel() == C, "shape mismatch");
    if (gate) TORCH_CHECK(gate->dim() == 2 && gate->stride(1) == 1 && gate->size(0) == rows && gate->size(1) == C &&
                              gate->scalar_type() == y.scalar_type(), "gate must be [rows, C] of y's dtype");
    if (lp) TORCH_CHECK(lp->dim() == 2 && lp->stride(1) == 1 && lp->size(0) == rows && lp->size(1) == C && lp->scalar_type() == y.scalar_type(),
                        "the copy must be [rows, C] of y's dtype");
    seqmix::postnorm_gated(x.data_ptr<float>(), x.stride(0), y.data_ptr(), y.stride(0), gate ? gate->data_ptr() : nullptr,
                           gate ? gate->stride(0) : 0, is_bf(y), f32(w), (float)alpha, (float)eps, rows, C, lp ? lp->data_ptr() : nullptr,
                           lp ? lp->stride(0) : 0, stream());
    check_launch();
}

// x [rows, C], gate [rows, C] (row strides free), w float [C] or [C / groups] → out [rows, C] (row stride free) of the gate's dtype
void group_rms_norm_gated(const Tensor& x, const Tensor& gate, const Tensor& w, int64_t groups, double eps, bool gate_first, Tensor out,
                          double out_scale, bool sigmoid_gate) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && gate.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && gate.stride(1) == 1 && out.stride(1) == 1,
                "x, gate, out must be [rows, C] with contiguous last dimensions");
    const int rows = x.size(0), C = x.size(1);
    TORCH_CHECK(gate.size(0) == rows && gate.size(1) == C && out.size(0) == rows && out.size(1) == C && groups >= 1 && C % groups == 0 &&
                    (w.numel() == C || w.numel() == C / groups) && out.scalar_type() == gate.scalar_type(), "shape mismatch");
    seqmix::group_rms_norm_gated(x.data_ptr(), is_bf(x), x.stride(0), gate.data_ptr(), is_bf(gate), gate.stride(0), f32(w), (int)w.numel(), rows,
                                 C, (int)groups, (float)eps, gate_first, out.data_ptr(), out.stride(0), (float)out_scale, sigmoid_gate, stream());
    check_launch();
}

// logits float [N,E] → (weights float [N,top], expert ids int64 [N,top], identity share float [N]); kind 1: softmax, 0: sigmoid
std::vector<Tensor> route_topk(const Tensor& logits, const c10::optional<Tensor>& correction, int64_t top, int64_t n_real, int64_t kind,
                               double scale) {
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat, "logits must be float [N,E]");
    const int N = logits.size(0), E = logits.size(1);
    TORCH_CHECK(!correction || correction->numel() == E, "the correction holds one number per expert");
    Tensor w = at::empty({N, top}, logits.options()), idx = at::empty({N, top}, logits.options().dtype(at::kLong));
    Tensor ident = at::empty({N}, logits.options());
    bool ok = seqmix::route_topk(logits.data_ptr<float>(), correction ? f32(*correction) : nullptr, N, E, (int)top, (int)n_real, (int)kind,
                                 (float)scale, w.data_ptr<float>(), idx.data_ptr<int64_t>(), ident.data_ptr<float>(), stream());
    TORCH_CHECK(ok, "route_topk: at most 256 experts and top <= experts");
    check_launch();
    return {w, idx, ident};
}

// x [N, I] (row stride free), w [O, I] contiguous → float [N, O]
Tensor small_linear_f32(const Tensor& x, const Tensor& w) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && w.dim() == 2 && w.is_contiguous() && w.size(1) == x.size(1), "bad operands");
    Tensor out = at::empty({x.size(0), w.size(0)}, x.options().dtype(at::kFloat));
    seqmix::small_linear_f32(w.data_ptr(), is_bf(w), x.data_ptr(), is_bf(x), x.stride(0), (int)x.size(0), (int)w.size(0), (int)x.size(1),
                             out.data_ptr<float>(), stream());
    check_launch();
    return out;
}

// gu [M, 2F] contiguous → g sigmoid(slope g) (u + 1) with g = min(gu[:, :F], limit), u = clamp(gu[:, F:], -limit, limit)
Tensor clamped_glu(const Tensor& gu, double limit, double slope) {
    TORCH_CHECK(gu.is_cuda() && gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 2 == 0, "gu must be contiguous [M, 2F]");
    Tensor out = at::empty({gu.size(0), gu.size(1) / 2}, gu.options());
    seqmix::clamped_glu(gu.data_ptr(), out.data_ptr(), is_bf(gu), gu.size(0), (int)(gu.size(1) / 2), (float)limit, (float)slope, stream());
    check_launch();
    return out;
}

// x [N, C] contiguous *= sigmoid(gate [N, Cg]) with C % Cg == 0 (gate: bfloat16 or float, row stride free)
void sigmoid_gate_mul_(Tensor x, const Tensor& gate) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && gate.dim() == 2 && gate.stride(1) == 1 && gate.size(0) == x.size(0) &&
                    gate.size(1) > 0 && x.size(1) % gate.size(1) == 0, "x must be contiguous [N, C], gate [N, Cg] with Cg dividing C");
    seqmix::sigmoid_gate_mul(x.data_ptr(), is_bf(x), gate.data_ptr(), is_bf(gate), gate.stride(0), x.size(0), (int)x.size(1),
                             (int)(x.size(1) / gate.size(1)), stream());
    check_launch();
}

// p [B,S,C] (last dim contiguous): hq query heads and hk key heads of D numbers, then the rest → float [B,S,C]
Tensor rotary_qkv_f32(const Tensor& p, int64_t hq, int64_t hk, int64_t D, int64_t dims, const Tensor& inv_freq, const Tensor& pos0,
                      double q_scale, double k_scale) {
    TORCH_CHECK(p.is_cuda() && p.dim() == 3 && p.stride(2) == 1, "p must be [B,S,C] with a contiguous last dimension");
    const int B = p.size(0), S = p.size(1), C = p.size(2);
    TORCH_CHECK((hq + hk) * D <= C && dims % 2 == 0 && dims <= D && inv_freq.numel() == dims / 2 && pos0.numel() == B, "bad rotary sizes");
    Tensor out = at::empty({B, S, C}, p.options().dtype(at::kFloat));
    seqmix::rotary_qkv_f32(p.data_ptr(), is_bf(p), p.stride(0), p.stride(1), B, S, C, (int)hq, (int)hk, (int)D, (int)dims, f32(inv_freq),
                           i32(pos0), (float)q_scale, (float)k_scale, out.data_ptr<float>(), stream());
    check_launch();
    return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("clamped_glu", &clamped_glu);
    m.def("sigmoid_gate_mul_", &sigmoid_gate_mul_);
    m.def("rotary_qkv_f32", &rotary_qkv_f32);
    m.def("route_topk", &route_topk);
    m.def("small_linear_f32", &small_linear_f32);
    m.def("short_conv", &short_conv);
    m.def("rms_norm", &rms_norm);
    m.def("add_rms_norm_", &add_rms_norm_);
    m.def("xielu", &xielu);
    m.def("gelu_erf", &gelu_erf);
    m.def("relu_sq", &relu_sq);
    m.def("embed_bigram", &embed_bigram);
    m.def("postnorm_gated_", &postnorm_gated_);
    m.def("silu_mul", &silu_mul);
    m.def("indexed_gemv", &indexed_gemv);
    m.def("moe_combine", &moe_combine);
    m.def("embed_sinusoid", &embed_sinusoid);
    m.def("group_rms_norm_gated", &group_rms_norm_gated);
}
