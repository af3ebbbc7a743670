// Grouped-query sliding-window attention over a prompt as one fused tensor-core kernel (bfloat16 operands): scores, score cap, window
// mask, softmax and the weighted sum of values never leave the chip.  A block owns 64 consecutive queries of one (sequence, query
// head); its four warps own 16 queries each; the query heads of a group read the same key / value head (through L2).  Key / value
// tiles of 64 positions are staged in shared memory by asynchronous copies, one tile ahead of the arithmetic.  Scores come from
// mma.sync m16n8k16 products with float accumulation; they are scaled, capped (cap * tanh(s / cap), the tanh formed from one base-2
// exponential), masked and exponentiated in float with a running maximum and sum per query; the weights are rounded to bfloat16
// only as operands of the value product, whose accumulator is float.  The result is multiplied by sigmoid(gate) and a constant and
// written with a free row stride.  Position i sees j with 0 <= i - j < window.  Queries at or past lens[b] give zeros.
// SIG: every visible key's weight is sigmoid(score + bias[h]) by itself (no running maximum, no sum, no division at the end).
// Sizes: key and value sizes are multiples of 16 up to 16 * DK16 / 16 * VD16 (template bounds; the real sizes are arguments).
#include "mma_tiles.cuh"
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kQT = 64, kKT = 64, kPad = 8;     // queries / keys per tile; row padding (elements) against bank conflicts

template <int DK16, int VD16, bool SIG>
__global__ void __launch_bounds__(128)
window_prompt_mma_kernel(const bf16* __restrict__ q, long q_sb, long q_st, const bf16* __restrict__ k, long k_sb, long k_st,
                         const bf16* __restrict__ v, long v_sb, long v_st, const bf16* __restrict__ gate, long g_sb, long g_st,
                         const int* __restrict__ lens, int S, int H, int G, int DK, int VD, int window, float scale, float softcap,
                         const float* __restrict__ score_bias, bf16* __restrict__ out, long out_stride, float out_scale) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk16 = DK / 16, vd16 = VD / 16, ldk = DK + kPad, ldv = VD + kPad;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [kQT][ldk] queries, then key stage 1 (same size)
    auto Kst = [&](int st) { return st ? Qs : Qs + kQT * ldk; };                               // [kKT][ldk] each
    auto Vst = [&](int st) { return Qs + (kQT + kKT) * ldk + (st ? kKT * ldv : 0); };          // [kKT][ldv] each
    const int q0 = blockIdx.x * kQT, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = h / (H / G);
    const int len = min(lens[b], S);
    bf16* ob = out + ((long)b * S) * out_stride + (long)h * VD;
    if (q0 >= len) {                                       // nothing but padding: zeros
        for (int i = tid; i < min(kQT, S - q0) * (VD / 2); i += 128) {
            const int r = i / (VD / 2), c = (i % (VD / 2)) * 2;
            *reinterpret_cast<unsigned*>(ob + (long)(q0 + r) * out_stride + c) = 0u;
        }
        return;
    }
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    for (int i = tid; i < kQT * (DK / 8); i += 128) {
        const int r = i / (DK / 8), c = (i % (DK / 8)) * 8, t = q0 + r;
        *reinterpret_cast<uint4*>(Qs + r * ldk + c) =
            t < S ? *reinterpret_cast<const uint4*>(q + (long)b * q_sb + (long)t * q_st + (long)h * DK + c) : zero4;
    }
    __syncthreads();
    const int r0 = warp * 16, g = lane >> 2, tq = lane & 3;
    unsigned qa[DK16][4];
#pragma unroll
    for (int kk = 0; kk < DK16; ++kk)
        if (kk < dk16) ldsm4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], Qs + (r0 + (lane & 15)) * ldk + kk * 16 + (lane >> 4) * 8);
    float oacc[2 * VD16][4];
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int i0 = q0 + r0 + g, i1 = i0 + 8;               // this thread's two queries
    const float log2e = 1.4426950408889634f;
    const float scale2 = scale * log2e;                    // uncapped scores go straight to base 2
    const float cap_in = softcap > 0.f ? 2.f * log2e * scale / softcap : 0.f, cap_out = softcap * log2e;
    const float sbias2 = SIG ? score_bias[h] * log2e : 0.f;
    const int jlo = max(0, q0 - window + 1), jhi = min(q0 + kQT - 1, len - 1);
    const bf16* kb = k + (long)b * k_sb + (long)hk * DK;
    const bf16* vb = v + (long)b * v_sb + (long)hk * VD;
    auto fetch = [&](int kt, int st) {
        const int j0 = kt * kKT;
        bf16 *Kd = Kst(st), *Vd = Vst(st);
        for (int c = lane * 8; c < DK; c += 256) {
#pragma unroll 4
            for (int r = warp; r < kKT; r += 4) {
                const int j = j0 + r;
                cp16(Kd + r * ldk + c, kb + (long)min(j, len - 1) * k_st + c, j < len);
            }
        }
        for (int c = lane * 8; c < VD; c += 256) {
#pragma unroll 4
            for (int r = warp; r < kKT; r += 4) {
                const int j = j0 + r;
                cp16(Vd + r * ldv + c, vb + (long)min(j, len - 1) * v_st + c, j < len);
            }
        }
        cp_commit();
    };
    const int kt0 = jlo / kKT, kt1 = jhi / kKT;
    __syncthreads();                                       // every warp holds its queries: their room becomes key stage 1
    fetch(kt0, 0);
    for (int kt = kt0; kt <= kt1; ++kt) {
        const int j0 = kt * kKT, st = (kt - kt0) & 1;
        if (kt < kt1) { fetch(kt + 1, st ^ 1); cp_wait<1>(); } else cp_wait<0>();
        __syncthreads();                                   // tile kt has landed for everyone
        const bf16 *Ks = Kst(st), *Vs = Vst(st);
        float sacc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DK16; ++kk) {
            if (kk < dk16) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {           // two 8-key groups per ldmatrix
                    unsigned b0, b1, b2, b3;
                    ldsm4(b0, b1, b2, b3, Ks + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(sacc[2 * np], qa[kk], b0, b1);
                    mma16816(sacc[2 * np + 1], qa[kk], b2, b3);
                }
            }
        }
        // scale, cap, mask, running softmax (float, in base 2); a thread holds 16 scores of query i0 and 16 of i1.  A tile that every
        // query of the warp sees in full needs no mask.
        const int wlo = q0 + r0, whi = wlo + 15;
        const bool full = j0 + kKT - 1 <= wlo && j0 > whi - window && j0 + kKT - 1 < len;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                bool vis = true;
                if (!full) {
                    const int j = j0 + n * 8 + tq * 2 + (e & 1), i = (e < 2) ? i0 : i1;
                    vis = j <= i && j > i - window && j < len;
                }
                float sc;
                if (softcap > 0.f) {                       // cap tanh(x) = cap (1 - 2 / (1 + e^(2x))), already times log2(e)
                    const float t = exp2f(fminf(sacc[n][e] * cap_in, 126.f));
                    sc = cap_out * (1.f - __fdividef(2.f, 1.f + t));
                } else {
                    sc = sacc[n][e] * scale2;
                }
                if (SIG) {                                 // sigmoid(x) = 1 / (1 + 2^(-x log2 e)); sc already holds x log2 e
                    sacc[n][e] = vis ? __fdividef(1.f, 1.f + exp2f(fminf(-(sc + sbias2), 126.f))) : 0.f;
                } else {
                    sacc[n][e] = vis ? sc : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sacc[n][e]);
                }
            }
        float corr[2], base[2];
        if (!SIG) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(mrow[r], mx[r]);
            base[r] = mn == -INFINITY ? 0.f : mn;          // nothing visible so far: every weight is exp(-inf) = 0
            corr[r] = exp2f(mrow[r] - base[r]);
            mrow[r] = mn;
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sacc[n][e] = exp2f(sacc[n][e] - base[e >> 1]);
                ls[e >> 1] += sacc[n][e];
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + ls[r];
#pragma unroll
        for (int n = 0; n < 2 * VD16; ++n) { oacc[n][0] *= corr[0]; oacc[n][1] *= corr[0]; oacc[n][2] *= corr[1]; oacc[n][3] *= corr[1]; }
        }
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
            unsigned pa[4];
            pa[0] = pack2(sacc[2 * kp][0], sacc[2 * kp][1]);
            pa[1] = pack2(sacc[2 * kp][2], sacc[2 * kp][3]);
            pa[2] = pack2(sacc[2 * kp + 1][0], sacc[2 * kp + 1][1]);
            pa[3] = pack2(sacc[2 * kp + 1][2], sacc[2 * kp + 1][3]);
#pragma unroll
            for (int nv = 0; nv < VD16; ++nv) {
                if (nv < vd16) {
                    unsigned b0, b1, b2, b3;
                    ldsm4t(b0, b1, b2, b3, Vs + (kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + nv * 16 + (lane >> 4) * 8);
                    mma16816(oacc[2 * nv], pa, b0, b1);
                    mma16816(oacc[2 * nv + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();                                   // the stage may be refilled
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    if (SIG) lrow[0] = lrow[1] = 1.f;
    float inv0 = (i0 < len && lrow[0] > 0.f) ? out_scale / lrow[0] : 0.f, inv1 = (i1 < len && lrow[1] > 0.f) ? out_scale / lrow[1] : 0.f;
    if (gate) {
        if (i0 < len) inv0 *= sigmoidf_(__bfloat162float(gate[(long)b * g_sb + (long)i0 * g_st + h]));
        if (i1 < len) inv1 *= sigmoidf_(__bfloat162float(gate[(long)b * g_sb + (long)i1 * g_st + h]));
    }
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) {
        if (n < 2 * vd16) {
            const int c = n * 8 + tq * 2;
            if (i0 < S) *reinterpret_cast<unsigned*>(ob + (long)i0 * out_stride + c) = pack2(oacc[n][0] * inv0, oacc[n][1] * inv0);
            if (i1 < S) *reinterpret_cast<unsigned*>(ob + (long)i1 * out_stride + c) = pack2(oacc[n][2] * inv1, oacc[n][3] * inv1);
        }
    }
}

// The fused kernel takes bfloat16 with key and value sizes in whole 16s up to 256 and 16-byte aligned rows.
bool window_prompt_mma_fits(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                            int D, int V, const void* out, long out_stride) {
    auto a16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
    return D % 16 == 0 && V % 16 == 0 && D <= 256 && V <= 256 && a16(q) && a16(k) && a16(v) && (uintptr_t)out % 4 == 0 && q_sb % 8 == 0 &&
           q_st % 8 == 0 && k_sb % 8 == 0 && k_st % 8 == 0 && v_sb % 8 == 0 && v_st % 8 == 0 && out_stride % 2 == 0;
}

void window_prompt_mma(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                       const void* gate, long g_sb, long g_st, const int* lens, int B, int S, int H, int G, int D, int V, int window,
                       float scale, float softcap, const float* score_bias, void* out, long out_stride, float out_scale, cudaStream_t s) {
    const size_t smem = (size_t)((kQT + kKT) * (D + kPad) + 2 * kKT * (V + kPad)) * sizeof(bf16);
    dim3 grid((S + kQT - 1) / kQT, H, B);
#define SEQMIX_WPM_S(A, Bv, SG)                                                                                                       \
    do {                                                                                                                              \
        cudaFuncSetAttribute(window_prompt_mma_kernel<A, Bv, SG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);           \
        window_prompt_mma_kernel<A, Bv, SG><<<grid, 128, smem, s>>>((const bf16*)q, q_sb, q_st, (const bf16*)k, k_sb, k_st,             \
                                                                   (const bf16*)v, v_sb, v_st, (const bf16*)gate, g_sb, g_st, lens, S,  \
                                                                   H, G, D, V, window, scale, softcap, score_bias, (bf16*)out,         \
                                                                   out_stride, out_scale);                                            \
    } while (0)
#define SEQMIX_WPM(A, Bv) do { if (score_bias) SEQMIX_WPM_S(A, Bv, true); else SEQMIX_WPM_S(A, Bv, false); } while (0)
    if (D <= 64 && V <= 64) SEQMIX_WPM(4, 4);
    else if (D <= 128 && V <= 128) SEQMIX_WPM(8, 8);
    else SEQMIX_WPM(16, 16);
#undef SEQMIX_WPM
#undef SEQMIX_WPM_S
}

}  // namespace seqmix
