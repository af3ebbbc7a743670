// Elementwise activations and the small-batch pieces of a routed feed-forward.
//   xielu        : z > 0: ap z^2 + z/2;  z <= 0: an (exp(z) - 1 - z) + z/2   (ap, an are positive numbers prepared by the caller)
//   gelu_erf     : 0.5 z (1 + erf(z / sqrt 2))
//   relu_sq      : max(z, 0)^2
//   silu_mul     : silu(gate) * up for rows [gate | up]
//   clamped_glu  : g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(slope g) (u + 1) for rows [gate | up]
//   sigmoid_gate_mul : x *= sigmoid(gate), one gate number per `rep` consecutive coordinates (a head, or one coordinate)
//   indexed_gemv : out[m,:] = act(W[sel[m]] x[m,:]) for a few rows m, each with its own matrix out of a stack [E, O, I]
//                  (token generation: the chosen experts' matrices are streamed once, a warp per output row); act 0: none,
//                  1: gelu_erf, 2: the matrix stacks gate rows over up rows and out = silu(gate row . x) * (up row . x), O/2 columns;
//                  3: the square of relu; rows whose sel names no matrix give zeros
//   moe_combine  : y[n,:] = base_weight[n] * base[n,:] + sum_k weight[n,k] * rows[src[n,k],:], summed in float
//   route_topk   : scores, choice with a correction, top-k, weights and the identity experts' share in one launch
//   small_linear_f32 : a few rows times a matrix with float results (router logits, per-head scalars of the recurrences)
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

__device__ __forceinline__ float gelu_erf_(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752f)); }

__device__ __forceinline__ float xielu_(float z, float ap, float an) {
    return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
}

__device__ __forceinline__ float relu_sq_(float z) { const float r = fmaxf(z, 0.f); return r * r; }

template <int ACT>
__device__ __forceinline__ float act_value(float z, float ap, float an) {
    return ACT == 0 ? xielu_(z, ap, an) : (ACT == 1 ? gelu_erf_(z) : relu_sq_(z));
}

// 16 bytes per thread and access (8 bfloat16 / 4 float); `n16` counts whole 16-byte groups, the tail goes one by one
template <typename T, int ACT>
__global__ void act_kernel(const T* __restrict__ x, T* __restrict__ out, long n, long n16, float ap, float an) {
    constexpr int VEC = 16 / sizeof(T);
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n16) {
        uint4 raw = reinterpret_cast<const uint4*>(x)[i];
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float z = ldf(e + k);
            stf(e + k, act_value<ACT>(z, ap, an));
        }
        reinterpret_cast<uint4*>(out)[i] = raw;
    } else {
        const long j = n16 * VEC + (i - n16);
        if (j < n) stf(out + j, act_value<ACT>(ldf(x + j), ap, an));
    }
}

template <typename T, int ACT>
static void act_launch(const void* x, void* out, long n, float ap, float an, cudaStream_t s) {
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const long n16 = aligned ? n / VEC : 0, total = n16 + (n - n16 * VEC);
    act_kernel<T, ACT><<<(unsigned)((total + 255) / 256), 256, 0, s>>>((const T*)x, (T*)out, n, n16, ap, an);
}

template <typename T, bool VEC>
__device__ __forceinline__ float row_dot(const T* __restrict__ wr, const T* __restrict__ xr, int I, int lane) {
    float acc = 0.f;
    if (VEC) {                                   // four weights per lane and access, two accesses in flight
        float acc2 = 0.f;
        int i = lane * 4;
        for (; i + 128 < I; i += 256) {
            const float4 a = ld4(wr + i), b = ld4(wr + i + 128), xa = ld4(xr + i), xb = ld4(xr + i + 128);
            acc = fmaf(a.x, xa.x, fmaf(a.y, xa.y, fmaf(a.z, xa.z, fmaf(a.w, xa.w, acc))));
            acc2 = fmaf(b.x, xb.x, fmaf(b.y, xb.y, fmaf(b.z, xb.z, fmaf(b.w, xb.w, acc2))));
        }
        if (i < I) {
            const float4 a = ld4(wr + i), xa = ld4(xr + i);
            acc = fmaf(a.x, xa.x, fmaf(a.y, xa.y, fmaf(a.z, xa.z, fmaf(a.w, xa.w, acc))));
        }
        acc += acc2;
    } else {
        for (int i = lane; i < I; i += 32) acc = fmaf(ldf(wr + i), ldf(xr + i), acc);
    }
    return warp_sum(acc);
}

template <typename T, bool VEC>
__global__ void indexed_gemv_kernel(const T* __restrict__ w, const int* __restrict__ sel, const T* __restrict__ x, long x_stride,
                                    int M, int E, int O, int I, int act, T* __restrict__ out) {
    const int On = act == 2 ? O / 2 : O;
    const int o = blockIdx.x * blockDim.y + threadIdx.y, m = blockIdx.y, lane = threadIdx.x;
    if (o >= On) return;
    const int e = sel[m];
    if (e < 0 || e >= E) {
        if (lane == 0) stf(out + (long)m * On + o, 0.f);
        return;
    }
    const T* wr = w + ((long)e * O + o) * I;
    const T* xr = x + (long)m * x_stride;
    float acc = row_dot<T, VEC>(wr, xr, I, lane);
    if (act == 1) acc = gelu_erf_(acc);
    else if (act == 3) acc = relu_sq_(acc);
    else if (act == 2) acc = acc * sigmoidf_(acc) * row_dot<T, VEC>(wr + (long)On * I, xr, I, lane);
    if (lane == 0) stf(out + (long)m * On + o, acc);
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, long rows, int F, T* __restrict__ out) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * F) return;
    const long r = i / F;
    const int c = (int)(i - r * F);
    const float g = ldf(gu + r * 2 * F + c), u = ldf(gu + r * 2 * F + F + c);
    stf(out + i, g * sigmoidf_(g) * u);
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ src, const float* __restrict__ weight,
                                   const T* __restrict__ base, const float* __restrict__ base_weight, int N, int top, int C,
                                   T* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, n = blockIdx.y;
    if (c >= C) return;
    float acc = base ? ldf(base + (long)n * C + c) * (base_weight ? base_weight[n] : 1.f) : 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weight[(long)n * top + k], ldf(rows + (long)src[(long)n * top + k] * C + c), acc);
    stf(out + (long)n * C + c, acc);
}

// Router: a warp per row.  scores = softmax (kind 1) or sigmoid (kind 0) of the row's logits; the `top` largest of scores + correction
// are chosen (ties: the lower index), in descending order; a chosen real expert (index < n_real) gets weight score * scale, a chosen
// identity expert weight 0 while its score is added to ident[row].  Kind 2: the scores are the logits themselves and the weights
// are the softmax over the CHOSEN logits only (times scale).  PL: logits per lane (E <= 32 PL).
template <int PL>
__global__ void route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int N, int E, int top, int n_real,
                                  int kind, float scale, float* __restrict__ w, long* __restrict__ idx, float* __restrict__ ident) {
    const int row = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (row >= N) return;
    const float* z = logits + (long)row * E;
    float sc[PL], ch[PL];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        sc[i] = e < E ? z[e] : -INFINITY;
        mx = fmaxf(mx, sc[i]);
    }
    if (kind == 1) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PL; ++i) { sc[i] = lane + 32 * i < E ? expf(sc[i] - mx) : 0.f; sum += sc[i]; }
        sum = warp_sum(sum);
#pragma unroll
        for (int i = 0; i < PL; ++i) sc[i] = sc[i] / sum;
    } else if (kind == 0) {
#pragma unroll
        for (int i = 0; i < PL; ++i) sc[i] = lane + 32 * i < E ? sigmoidf_(sc[i]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        ch[i] = e < E ? sc[i] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    float idw = 0.f, first = 0.f, total = 0.f, keep = 0.f;
    for (int t = 0; t < top; ++t) {
        float bv = -INFINITY, bs = 0.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PL; ++i)
            if (ch[i] > bv) { bv = ch[i]; bs = sc[i]; be = lane + 32 * i; }      // ascending e within a lane: ties keep the lower index
        float v = bv;
        int e = be;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oe = __shfl_xor_sync(0xffffffffu, e, o);
            if (ov > v || (ov == v && oe < e)) { v = ov; e = oe; }
        }
        const float s_e = __shfl_sync(0xffffffffu, bs, e & 31);                  // the owner's best is the winner
        if ((e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PL; ++i)
                if (lane + 32 * i == e) ch[i] = -INFINITY;
        }
        if (kind == 2) {                                                         // every lane follows the sum; lane t keeps the t-th
            if (t == 0) first = s_e;                                             // exponential (the first chosen logit is the largest)
            const float x = expf(s_e - first);
            total += x;
            if (t == lane) keep = x;
            if (t >= 32 && lane == 0) w[(long)row * top + t] = x;                // beyond a warp's worth: through memory
        }
        if (lane == 0) {
            idx[(long)row * top + t] = e;
            if (kind != 2) {
                w[(long)row * top + t] = e < n_real ? s_e * scale : 0.f;
                if (e >= n_real) idw += s_e;
            }
        }
    }
    if (kind == 2) {
        if (lane < top) w[(long)row * top + lane] = keep / total * scale;
        if (top > 32 && lane == 0)
            for (int t = 32; t < top; ++t) w[(long)row * top + t] = w[(long)row * top + t] / total * scale;
    }
    if (lane == 0 && ident) ident[row] = idw;
}

bool route_topk(const float* logits, const float* correction, int N, int E, int top, int n_real, int kind, float scale, float* w, long* idx,
                float* ident, cudaStream_t s) {
    if (E > 256 || top > E) return false;
    if (N == 0) return true;
    dim3 block(32, 4), grid((N + 3) / 4);
    const int pl = (E + 31) / 32;
#define SEQMIX_ROUTE(P) route_topk_kernel<P><<<grid, block, 0, s>>>(logits, correction, N, E, top, n_real, kind, scale, w, idx, ident)
    if (pl <= 1) SEQMIX_ROUTE(1); else if (pl <= 2) SEQMIX_ROUTE(2); else if (pl <= 4) SEQMIX_ROUTE(4); else SEQMIX_ROUTE(8);
#undef SEQMIX_ROUTE
    return true;
}

// out[n, o] = w[o, :] . x[n, :] in float for a few rows n (a warp per output; w float or bfloat16, x float or bfloat16)
template <typename Tw, typename Tx>
__global__ void small_linear_f32_kernel(const Tw* __restrict__ w, const Tx* __restrict__ x, long x_stride, int N, int O, int I,
                                        float* __restrict__ out) {
    const int o = blockIdx.x * blockDim.y + threadIdx.y, n = blockIdx.y, lane = threadIdx.x;
    if (o >= O) return;
    const Tw* wr = w + (long)o * I;
    const Tx* xr = x + (long)n * x_stride;
    float acc = 0.f;
    for (int i = lane; i < I; i += 32) acc = fmaf(ldf(wr + i), ldf(xr + i), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[(long)n * O + o] = acc;
}

void small_linear_f32(const void* w, int w_bf, const void* x, int x_bf, long x_stride, int N, int O, int I, float* out, cudaStream_t s) {
    if (N * O == 0) return;
    dim3 block(32, 8), grid((O + 7) / 8, N);
    if (w_bf && x_bf) small_linear_f32_kernel<bf16, bf16><<<grid, block, 0, s>>>((const bf16*)w, (const bf16*)x, x_stride, N, O, I, out);
    else if (!w_bf && x_bf) small_linear_f32_kernel<float, bf16><<<grid, block, 0, s>>>((const float*)w, (const bf16*)x, x_stride, N, O, I, out);
    else if (w_bf && !x_bf) small_linear_f32_kernel<bf16, float><<<grid, block, 0, s>>>((const bf16*)w, (const float*)x, x_stride, N, O, I, out);
    else small_linear_f32_kernel<float, float><<<grid, block, 0, s>>>((const float*)w, (const float*)x, x_stride, N, O, I, out);
}

void xielu(const void* x, void* out, int bf, long n, float ap, float an, cudaStream_t s) {
    if (n == 0) return;
    if (bf) act_launch<bf16, 0>(x, out, n, ap, an, s); else act_launch<float, 0>(x, out, n, ap, an, s);
}

void gelu_erf(const void* x, void* out, int bf, long n, cudaStream_t s) {
    if (n == 0) return;
    if (bf) act_launch<bf16, 1>(x, out, n, 0.f, 0.f, s); else act_launch<float, 1>(x, out, n, 0.f, 0.f, s);
}

void relu_sq(const void* x, void* out, int bf, long n, cudaStream_t s) {
    if (n == 0) return;
    if (bf) act_launch<bf16, 2>(x, out, n, 0.f, 0.f, s); else act_launch<float, 2>(x, out, n, 0.f, 0.f, s);
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, long rows, int F, T* __restrict__ out) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= rows * F) return;
    const long r = i / F;
    const int c = (int)(i - r * F);
    const float4 g = ld4(gu + r * 2 * F + c), u = ld4(gu + r * 2 * F + F + c);
    st4(out + i, make_float4(g.x * sigmoidf_(g.x) * u.x, g.y * sigmoidf_(g.y) * u.y, g.z * sigmoidf_(g.z) * u.z, g.w * sigmoidf_(g.w) * u.w));
}

void silu_mul(const void* gu, void* out, int bf, long rows, int F, cudaStream_t s) {
    if (rows * F == 0) return;
    const size_t a4 = bf ? 8 : 16;
    if (F % 4 == 0 && (uintptr_t)gu % a4 == 0 && (uintptr_t)out % a4 == 0) {
        const unsigned vblocks = (unsigned)((rows * F / 4 + 255) / 256);
        if (bf) silu_mul_vec_kernel<bf16><<<vblocks, 256, 0, s>>>((const bf16*)gu, rows, F, (bf16*)out);
        else silu_mul_vec_kernel<float><<<vblocks, 256, 0, s>>>((const float*)gu, rows, F, (float*)out);
        return;
    }
    const unsigned blocks = (unsigned)((rows * F + 255) / 256);
    if (bf) silu_mul_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)gu, rows, F, (bf16*)out);
    else silu_mul_kernel<float><<<blocks, 256, 0, s>>>((const float*)gu, rows, F, (float*)out);
}

__device__ __forceinline__ float clamped_glu_f(float g, float u, float limit, float slope) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(slope * g) * (u + 1.f);
}

template <typename T, bool VEC>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, long rows, int F, float limit, float slope, T* __restrict__ out) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
    if (i >= rows * F) return;
    const long r = i / F;
    const int c = (int)(i - r * F);
    if (VEC) {
        const float4 g = ld4(gu + r * 2 * F + c), u = ld4(gu + r * 2 * F + F + c);
        st4(out + i, make_float4(clamped_glu_f(g.x, u.x, limit, slope), clamped_glu_f(g.y, u.y, limit, slope),
                                 clamped_glu_f(g.z, u.z, limit, slope), clamped_glu_f(g.w, u.w, limit, slope)));
    } else {
        stf(out + i, clamped_glu_f(ldf(gu + r * 2 * F + c), ldf(gu + r * 2 * F + F + c), limit, slope));
    }
}

void clamped_glu(const void* gu, void* out, int bf, long rows, int F, float limit, float slope, cudaStream_t s) {
    if (rows * F == 0) return;
    const size_t a4 = bf ? 8 : 16;
    if (F % 4 == 0 && (uintptr_t)gu % a4 == 0 && (uintptr_t)out % a4 == 0) {
        const unsigned vblocks = (unsigned)((rows * F / 4 + 255) / 256);
        if (bf) clamped_glu_kernel<bf16, true><<<vblocks, 256, 0, s>>>((const bf16*)gu, rows, F, limit, slope, (bf16*)out);
        else clamped_glu_kernel<float, true><<<vblocks, 256, 0, s>>>((const float*)gu, rows, F, limit, slope, (float*)out);
        return;
    }
    const unsigned blocks = (unsigned)((rows * F + 255) / 256);
    if (bf) clamped_glu_kernel<bf16, false><<<blocks, 256, 0, s>>>((const bf16*)gu, rows, F, limit, slope, (bf16*)out);
    else clamped_glu_kernel<float, false><<<blocks, 256, 0, s>>>((const float*)gu, rows, F, limit, slope, (float*)out);
}

// x [rows, C] contiguous, gate [rows, C / rep] with its own row stride
template <typename T, typename TG>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ x, const TG* __restrict__ gate, long gate_stride, long rows, int C, int rep) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const long r = i / C;
    const int c = (int)(i - r * C);
    stf(x + i, ldf(x + i) * sigmoidf_(ldf(gate + r * gate_stride + c / rep)));
}

// four consecutive coordinates per thread (C in whole fours); GV: the four have their own gates (rep == 1), else they share one
template <typename T, typename TG, bool GV>
__global__ void sigmoid_gate_mul_vec_kernel(T* __restrict__ x, const TG* __restrict__ gate, long gate_stride, long rows, int C, int rep) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= rows * C) return;
    const long r = i / C;
    const int c = (int)(i - r * C);
    float4 v = ld4(x + i);
    if (GV) {
        const float4 g = ld4(gate + r * gate_stride + c);
        v.x *= sigmoidf_(g.x); v.y *= sigmoidf_(g.y); v.z *= sigmoidf_(g.z); v.w *= sigmoidf_(g.w);
    } else {
        const float g = sigmoidf_(ldf(gate + r * gate_stride + c / rep));
        v.x *= g; v.y *= g; v.z *= g; v.w *= g;
    }
    st4(x + i, v);
}

void sigmoid_gate_mul(void* x, int bf, const void* gate, int gate_bf, long gate_stride, long rows, int C, int rep, cudaStream_t s) {
    if (rows * C == 0) return;
    const bool x_ok = C % 4 == 0 && (uintptr_t)x % 16 == 0;
    const bool shared = x_ok && rep % 4 == 0;
    const bool own = x_ok && rep == 1 && gate_stride % 4 == 0 && (uintptr_t)gate % 16 == 0;
    if (shared || own) {
        const unsigned blocks = (unsigned)((rows * C / 4 + 255) / 256);
#define SEQMIX_SGM(T, TG)                                                                                                       \
    do {                                                                                                                        \
        if (own) sigmoid_gate_mul_vec_kernel<T, TG, true><<<blocks, 256, 0, s>>>((T*)x, (const TG*)gate, gate_stride, rows, C, rep);   \
        else sigmoid_gate_mul_vec_kernel<T, TG, false><<<blocks, 256, 0, s>>>((T*)x, (const TG*)gate, gate_stride, rows, C, rep);      \
    } while (0)
        if (bf && gate_bf) SEQMIX_SGM(bf16, bf16);
        else if (bf) SEQMIX_SGM(bf16, float);
        else if (gate_bf) SEQMIX_SGM(float, bf16);
        else SEQMIX_SGM(float, float);
#undef SEQMIX_SGM
        return;
    }
    const unsigned blocks = (unsigned)((rows * C + 255) / 256);
    if (bf && gate_bf) sigmoid_gate_mul_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((bf16*)x, (const bf16*)gate, gate_stride, rows, C, rep);
    else if (bf) sigmoid_gate_mul_kernel<bf16, float><<<blocks, 256, 0, s>>>((bf16*)x, (const float*)gate, gate_stride, rows, C, rep);
    else if (gate_bf) sigmoid_gate_mul_kernel<float, bf16><<<blocks, 256, 0, s>>>((float*)x, (const bf16*)gate, gate_stride, rows, C, rep);
    else sigmoid_gate_mul_kernel<float, float><<<blocks, 256, 0, s>>>((float*)x, (const float*)gate, gate_stride, rows, C, rep);
}

void indexed_gemv(const void* w, const int* sel, const void* x, int bf, long x_stride, int M, int E, int O, int I, int act, void* out,
                  cudaStream_t s) {
    if (M == 0) return;
    const int On = act == 2 ? O / 2 : O;
    dim3 block(32, 8), grid((On + 7) / 8, M);
    const size_t a4 = bf ? 8 : 16;
    const bool vec = I % 4 == 0 && x_stride % 4 == 0 && (uintptr_t)w % a4 == 0 && (uintptr_t)x % a4 == 0;
#define SEQMIX_IGEMV(T, V) indexed_gemv_kernel<T, V><<<grid, block, 0, s>>>((const T*)w, sel, (const T*)x, x_stride, M, E, O, I, act, (T*)out)
    if (bf) { if (vec) SEQMIX_IGEMV(bf16, true); else SEQMIX_IGEMV(bf16, false); }
    else { if (vec) SEQMIX_IGEMV(float, true); else SEQMIX_IGEMV(float, false); }
#undef SEQMIX_IGEMV
}

// four columns per thread (C and the bases in whole fours)
template <typename T>
__global__ void moe_combine_vec_kernel(const T* __restrict__ rows, const int* __restrict__ src, const float* __restrict__ weight,
                                       const T* __restrict__ base, const float* __restrict__ base_weight, int N, int top, int C,
                                       T* __restrict__ out) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4, n = blockIdx.y;
    if (c >= C) return;
    float4 acc = base ? ld4(base + (long)n * C + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (base && base_weight) { const float bw = base_weight[n]; acc.x *= bw; acc.y *= bw; acc.z *= bw; acc.w *= bw; }
    for (int k = 0; k < top; ++k) {
        const float w = weight[(long)n * top + k];
        const float4 r = ld4(rows + (long)src[(long)n * top + k] * C + c);
        acc.x = fmaf(w, r.x, acc.x); acc.y = fmaf(w, r.y, acc.y); acc.z = fmaf(w, r.z, acc.z); acc.w = fmaf(w, r.w, acc.w);
    }
    st4(out + (long)n * C + c, acc);
}

void moe_combine(const void* rows, const int* src, const float* weight, const void* base, const float* base_weight, int bf, int N, int top,
                 int C, void* out, cudaStream_t s) {
    if (N == 0) return;
    const size_t a4 = bf ? 8 : 16;
    if (C % 4 == 0 && (uintptr_t)rows % a4 == 0 && (uintptr_t)out % a4 == 0 && (base == nullptr || (uintptr_t)base % a4 == 0)) {
        dim3 vblock(128), vgrid((C / 4 + 127) / 128, N);
        if (bf) moe_combine_vec_kernel<bf16><<<vgrid, vblock, 0, s>>>((const bf16*)rows, src, weight, (const bf16*)base, base_weight, N, top, C, (bf16*)out);
        else moe_combine_vec_kernel<float><<<vgrid, vblock, 0, s>>>((const float*)rows, src, weight, (const float*)base, base_weight, N, top, C, (float*)out);
        return;
    }
    dim3 block(128), grid((C + 127) / 128, N);
    if (bf) moe_combine_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)rows, src, weight, (const bf16*)base, base_weight, N, top, C, (bf16*)out);
    else moe_combine_kernel<float><<<grid, block, 0, s>>>((const float*)rows, src, weight, (const float*)base, base_weight, N, top, C, (float*)out);
}

}  // namespace seqmix
