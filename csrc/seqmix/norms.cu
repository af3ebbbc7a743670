// RMS norms of the sequence-mixer models: y = x / sqrt(mean(x^2) + eps) * w with w a vector or ONE number for all coordinates
// (with `center`, x's mean is taken off first: a layer norm with a gain and no bias, two passes over the row for the statistics),
// optionally times silu(gate), written out or accumulated into a float residual stream (x_res += norm(y): the residual sum of a
// layer that normalises the sublayer's OUTPUT).  Statistics in float.
//   postnorm_gated: the closing step of a block whose norm comes AFTER the residual sum, x <- norm(alpha * x + sigmoid(gate) * y) * w,
//   on a float stream in place (gate optional), with an optional copy of the result in the sublayers' dtype.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

// blockDim.x threads share a row (32: a warp per row, many rows; 256: a block per row, few rows such as single-token steps),
// blockDim.y rows per block.  VEC: four consecutive coordinates per thread and access (extents, strides and bases multiples of four
// elements, the gain a vector with stride 1 or one number).
template <typename Tin, typename Tout, bool VEC>
__global__ void rms_norm_kernel(const Tin* __restrict__ x, long x_stride, int rows, int C, const float* __restrict__ w, int w_stride,
                                float eps, const Tout* __restrict__ gate, long gate_stride, Tout* __restrict__ out, long out_stride,
                                float* res, long res_stride, int center) {
    __shared__ float part[8];
    const int row = blockIdx.x * blockDim.y + threadIdx.y, tx = threadIdx.x, TX = blockDim.x;
    const bool on = row < rows;
    const Tin* xr = x + (long)(on ? row : 0) * x_stride;
    auto row_sum = [&](float v) {               // over the threads that share the row
        v = warp_sum(v);
        if (TX > 32) {                          // one row per block: fold the warps' sums
            __syncthreads();
            if ((tx & 31) == 0) part[tx >> 5] = v;
            __syncthreads();
            v = 0.f;
            for (int k = 0; k < TX / 32; ++k) v += part[k];
        }
        return v;
    };
    float mean = 0.f;
    if (center) {
        float sx = 0.f;
        if (on) {
            if (VEC) {
                for (int c = tx * 4; c < C; c += TX * 4) { const float4 v = ld4(xr + c); sx += (v.x + v.y) + (v.z + v.w); }
            } else {
                for (int c = tx; c < C; c += TX) sx += ldf(xr + c);
            }
        }
        mean = row_sum(sx) / (float)C;
    }
    float ss = 0.f;
    if (on) {
        if (VEC) {
            for (int c = tx * 4; c < C; c += TX * 4) {
                float4 v = ld4(xr + c);
                v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
        } else {
            for (int c = tx; c < C; c += TX) { float v = ldf(xr + c) - mean; ss = fmaf(v, v, ss); }
        }
    }
    ss = row_sum(ss);
    if (!on) return;
    const float inv = 1.f / sqrtf(ss / (float)C + eps);
    if (VEC) {
        for (int c = tx * 4; c < C; c += TX * 4) {
            float4 v = ld4(xr + c);
            const float4 g = w_stride ? ld4(w + c) : make_float4(w[0], w[0], w[0], w[0]);
            v = make_float4((v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y, (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w);
            if (gate) {
                const float4 t = ld4(gate + (long)row * gate_stride + c);
                v.x *= t.x * sigmoidf_(t.x); v.y *= t.y * sigmoidf_(t.y); v.z *= t.z * sigmoidf_(t.z); v.w *= t.w * sigmoidf_(t.w);
            }
            if (res) {
                float* r = res + (long)row * res_stride + c;
                const float4 o = ld4(r);
                st4(r, make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w));
            } else st4(out + (long)row * out_stride + c, v);
        }
        return;
    }
    for (int c = tx; c < C; c += TX) {
        float v = (ldf(xr + c) - mean) * inv * w[(long)c * w_stride];
        if (gate) { float g = ldf(gate + (long)row * gate_stride + c); v *= g * sigmoidf_(g); }
        if (res) res[(long)row * res_stride + c] += v;
        else stf(out + (long)row * out_stride + c, v);
    }
}

// Rows in `groups` equal parts, each part divided by its own root mean square.  blockDim.x threads share a (row, part) unit (32: a
// warp per unit; 256: a block per unit, for long parts), blockDim.y units per block.  gate_first: the statistics are those of
// x * silu(gate); otherwise silu(gate) multiplies the normed values.  w holds C numbers or C / groups (wn says which).  VEC: four
// consecutive coordinates per thread and access.
template <typename Tin, typename Tg, bool VEC>
__global__ void group_rms_norm_gated_kernel(const Tin* __restrict__ x, long x_stride, const Tg* __restrict__ gate, long gate_stride,
                                            const float* __restrict__ w, int wn, int rows, int C, int groups, float eps, int gate_first,
                                            Tg* __restrict__ out, long out_stride, float out_scale, int sigmoid_gate) {
    // the gate's factor: silu(z) = z sigmoid(z), or sigmoid(z) alone
    auto gf = [&](float z) { return (sigmoid_gate ? 1.f : z) * sigmoidf_(z); };
    __shared__ float part[8];
    const long unit = (long)blockIdx.x * blockDim.y + threadIdx.y;
    const bool on = unit < (long)rows * groups;
    const int row = on ? (int)(unit / groups) : 0, g = on ? (int)(unit - (long)row * groups) : 0, Cg = C / groups;
    const int tx = threadIdx.x, TX = blockDim.x;
    const Tin* xr = x + (long)row * x_stride + (long)g * Cg;
    const Tg* gr = gate + (long)row * gate_stride + (long)g * Cg;
    float ss = 0.f;
    if (on) {
        if (VEC) {
            for (int c = tx * 4; c < Cg; c += TX * 4) {
                float4 v = ld4(xr + c);
                if (gate_first) {
                    const float4 z = ld4(gr + c);
                    v.x *= gf(z.x); v.y *= gf(z.y); v.z *= gf(z.z); v.w *= gf(z.w);
                }
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
        } else {
            for (int c = tx; c < Cg; c += TX) {
                float v = ldf(xr + c);
                if (gate_first) { const float z = ldf(gr + c); v *= gf(z); }
                ss = fmaf(v, v, ss);
            }
        }
    }
    ss = warp_sum(ss);
    if (TX > 32) {                              // one unit per block: fold the warps' sums
        if ((tx & 31) == 0) part[tx >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int k = 0; k < TX / 32; ++k) ss += part[k];
    }
    if (!on) return;
    const float inv = out_scale / sqrtf(ss / (float)Cg + eps);
    const float* wr = w + (wn == C ? (long)g * Cg : 0);
    Tg* o = out + (long)row * out_stride + (long)g * Cg;
    if (VEC) {
        for (int c = tx * 4; c < Cg; c += TX * 4) {
            const float4 v = ld4(xr + c), z = ld4(gr + c), u = ld4(wr + c);
            st4(o + c, make_float4(v.x * gf(z.x) * inv * u.x, v.y * gf(z.y) * inv * u.y, v.z * gf(z.z) * inv * u.z, v.w * gf(z.w) * inv * u.w));
        }
        return;
    }
    for (int c = tx; c < Cg; c += TX) {
        const float z = ldf(gr + c);
        stf(o + c, ldf(xr + c) * gf(z) * inv * wr[c]);
    }
}

// blockDim.x threads share a row (32: a warp per row, narrow rows; 256: a block per row, rows from 1024 coordinates on and single-token
// steps), blockDim.y rows per block; a thread meets the same coordinates in both passes, so the stream is updated in place.  VEC:
// four consecutive coordinates per thread and access.  NIT > 0 (VEC only): the row has at most NIT * 4 * blockDim.x coordinates and
// a thread keeps its mixed values in registers between the statistics and the scaling, so the stream, the sublayer's result and
// the gate are read once (rows up to 4096 coordinates with a block per row; beyond that the two-pass form).
template <typename T, bool VEC, int NIT>
__global__ void postnorm_gated_kernel(float* x, long x_stride, const T* __restrict__ y, long y_stride, const T* __restrict__ gate,
                                      long gate_stride, const float* __restrict__ w, float alpha, float eps, int rows, int C,
                                      T* __restrict__ lp, long lp_stride) {
    __shared__ float part[8];
    const int row = blockIdx.x * blockDim.y + threadIdx.y, tx = threadIdx.x, TX = blockDim.x;
    const bool on = row < rows;
    float* xr = x + (long)(on ? row : 0) * x_stride;
    const T* yr = y + (long)(on ? row : 0) * y_stride;
    const T* gr = gate ? gate + (long)(on ? row : 0) * gate_stride : nullptr;
    auto mix1 = [&](float xv, float yv, float gv) { return fmaf(alpha, xv, gr ? sigmoidf_(gv) * yv : yv); };
    auto mix4 = [&](int c) {
        const float4 a = ld4(xr + c), b = ld4(yr + c), g = gr ? ld4(gr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        return make_float4(mix1(a.x, b.x, g.x), mix1(a.y, b.y, g.y), mix1(a.z, b.z, g.z), mix1(a.w, b.w, g.w));
    };
    float4 kept[NIT > 0 ? NIT : 1];
    float ss = 0.f;
    if (on) {
        if (NIT > 0) {
#pragma unroll
            for (int i = 0; i < NIT; ++i) {
                const int c = (i * TX + tx) * 4;
                if (c < C) {
                    kept[i] = mix4(c);
                    ss = fmaf(kept[i].x, kept[i].x, fmaf(kept[i].y, kept[i].y, fmaf(kept[i].z, kept[i].z, fmaf(kept[i].w, kept[i].w, ss))));
                }
            }
        } else if (VEC) {
            for (int c = tx * 4; c < C; c += TX * 4) {
                const float4 v = mix4(c);
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
        } else {
            for (int c = tx; c < C; c += TX) { const float v = mix1(xr[c], ldf(yr + c), gr ? ldf(gr + c) : 0.f); ss = fmaf(v, v, ss); }
        }
    }
    ss = warp_sum(ss);
    if (TX > 32) {                              // one row per block: fold the warps' sums
        if ((tx & 31) == 0) part[tx >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int k = 0; k < TX / 32; ++k) ss += part[k];
    }
    if (!on) return;
    const float inv = 1.f / sqrtf(ss / (float)C + eps);
    auto put4 = [&](int c, float4 m) {
        const float4 u = ld4(w + c);
        const float4 v = make_float4(m.x * inv * u.x, m.y * inv * u.y, m.z * inv * u.z, m.w * inv * u.w);
        st4(xr + c, v);
        if (lp) st4(lp + (long)row * lp_stride + c, v);
    };
    if (NIT > 0) {
#pragma unroll
        for (int i = 0; i < NIT; ++i) {
            const int c = (i * TX + tx) * 4;
            if (c < C) put4(c, kept[i]);
        }
        return;
    }
    if (VEC) {
        for (int c = tx * 4; c < C; c += TX * 4) put4(c, mix4(c));
        return;
    }
    for (int c = tx; c < C; c += TX) {
        const float v = mix1(xr[c], ldf(yr + c), gr ? ldf(gr + c) : 0.f) * inv * w[c];
        xr[c] = v;
        if (lp) stf(lp + (long)row * lp_stride + c, v);
    }
}

void postnorm_gated(float* x, long x_stride, const void* y, long y_stride, const void* gate, long gate_stride, int bf, const float* w,
                    float alpha, float eps, int rows, int C, void* lp, long lp_stride, cudaStream_t s) {
    if (rows == 0) return;
    const bool few = C >= 1024 || (rows < 148 * 8 && C >= 512);      // a block per row: wide rows stay in registers that way
    dim3 block(few ? 256 : 32, few ? 1 : 8), grid(few ? rows : (rows + 7) / 8);
    const size_t e = bf ? 2 : 4;
    auto al = [](const void* p, size_t b) { return p == nullptr || (uintptr_t)p % b == 0; };
    const bool vec = C % 4 == 0 && x_stride % 4 == 0 && y_stride % 4 == 0 && (!gate || gate_stride % 4 == 0) && (!lp || lp_stride % 4 == 0) &&
                     al(x, 16) && al(w, 16) && al(y, 4 * e) && al(gate, 4 * e) && al(lp, 4 * e);
    const int per = vec ? (C / 4 + (int)block.x - 1) / (int)block.x : 0;   // 16-byte groups per thread
#define SEQMIX_PN(T, V, N)                                                                                                           \
    postnorm_gated_kernel<T, V, N><<<grid, block, 0, s>>>(x, x_stride, (const T*)y, y_stride, (const T*)gate, gate_stride, w, alpha, eps,   \
                                                          rows, C, (T*)lp, lp_stride)
#define SEQMIX_PN_T(T)                                                                                                               \
    do {                                                                                                                             \
        if (!vec) SEQMIX_PN(T, false, 0);                                                                                            \
        else if (per <= 4) SEQMIX_PN(T, true, 4);                                                                                    \
        else SEQMIX_PN(T, true, 0);                                                                                                  \
    } while (0)
    if (bf) SEQMIX_PN_T(bf16); else SEQMIX_PN_T(float);
#undef SEQMIX_PN_T
#undef SEQMIX_PN
}

void group_rms_norm_gated(const void* x, int in_bf16, long x_stride, const void* gate, int gate_bf16, long gate_stride, const float* w,
                          int wn, int rows, int C, int groups, float eps, int gate_first, void* out, long out_stride, float out_scale,
                          int sigmoid_gate, cudaStream_t s) {
    const long units = (long)rows * groups;
    if (units == 0) return;
    const int Cg = C / groups;
    const bool wide = Cg >= 1024;
    dim3 block(wide ? 256 : 32, wide ? 1 : 8), grid((unsigned)(wide ? units : (units + 7) / 8));
    const size_t ei = in_bf16 ? 2 : 4, eg = gate_bf16 ? 2 : 4;
    const bool vec = Cg % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 && (uintptr_t)x % (4 * ei) == 0 &&
                     (uintptr_t)gate % (4 * eg) == 0 && (uintptr_t)out % (4 * eg) == 0 && (uintptr_t)w % 16 == 0;
#define SEQMIX_GN_V(TI, TG, V)                                                                                                        \
    group_rms_norm_gated_kernel<TI, TG, V><<<grid, block, 0, s>>>((const TI*)x, x_stride, (const TG*)gate, gate_stride, w, wn, rows, C,  \
                                                                  groups, eps, gate_first, (TG*)out, out_stride, out_scale, sigmoid_gate)
#define SEQMIX_GN(TI, TG) do { if (vec) SEQMIX_GN_V(TI, TG, true); else SEQMIX_GN_V(TI, TG, false); } while (0)
    if (in_bf16 && gate_bf16) SEQMIX_GN(bf16, bf16);
    else if (!in_bf16 && gate_bf16) SEQMIX_GN(float, bf16);
    else if (!in_bf16 && !gate_bf16) SEQMIX_GN(float, float);
    else SEQMIX_GN(bf16, float);
#undef SEQMIX_GN_V
#undef SEQMIX_GN
}

void rms_norm(const void* x, int in_bf16, long x_stride, int rows, int C, const float* w, int w_stride, float eps, const void* gate,
              long gate_stride, void* out, int out_bf16, long out_stride, float* res, long res_stride, int center, cudaStream_t s) {
    const bool few = rows < 148 * 8 && C >= 512;
    dim3 block(few ? 256 : 32, few ? 1 : 8), grid(few ? rows : (rows + 7) / 8);
    const size_t ei = in_bf16 ? 2 : 4, eo = out_bf16 ? 2 : 4;
    auto al = [](const void* p, size_t e) { return p == nullptr || (uintptr_t)p % (4 * e) == 0; };
    const bool vec = C % 4 == 0 && x_stride % 4 == 0 && (w_stride == 0 || w_stride == 1) && al(x, ei) && al(w, 4) && al(gate, eo) &&
                     (!gate || gate_stride % 4 == 0) && al(out, eo) && (res || out_stride % 4 == 0) && al(res, 4) && (!res || res_stride % 4 == 0);
#define SEQMIX_NORM_V(TI, TO, V)                                                                                                    \
    rms_norm_kernel<TI, TO, V><<<grid, block, 0, s>>>((const TI*)x, x_stride, rows, C, w, w_stride, eps, (const TO*)gate, gate_stride, \
                                                      (TO*)out, out_stride, res, res_stride, center)
#define SEQMIX_NORM(TI, TO) do { if (vec) SEQMIX_NORM_V(TI, TO, true); else SEQMIX_NORM_V(TI, TO, false); } while (0)
    if (in_bf16 && out_bf16) SEQMIX_NORM(bf16, bf16);
    else if (!in_bf16 && out_bf16) SEQMIX_NORM(float, bf16);
    else if (!in_bf16 && !out_bf16) SEQMIX_NORM(float, float);
    else SEQMIX_NORM(bf16, float);
#undef SEQMIX_NORM_V
#undef SEQMIX_NORM
}

}  // namespace seqmix
