// Head-mixing attention over a prompt as one fused tensor-core kernel (bfloat16 operands): the queries arrive already mixed
// (Q' [B,S,H,DK] with DK = G*D, see headmix_attention.cu), so scores are one product of Q' rows with the positions' key rows (all
// key heads side by side); mask (aligned chunks and / or a sliding window), softmax with a sink term and the weighted sum of values
// never leave the chip.  A block owns 64 consecutive queries of one (sequence, head); its four warps own 16 queries each.  Key rows
// (DK wide, the same for every head) and the value rows of the head's key/value head (D wide, the keys before rotation) are staged
// in shared memory by asynchronous copies, one tile ahead of the arithmetic; the query tile stays in shared memory and its
// fragments are fetched per 16 coordinates, so DK may be several hundred.  Scores come from mma.sync m16n8k16 products with float
// accumulation; mask, running maximum / sum and exponentials are float; the weights are rounded to bfloat16 only as operands of the
// value product, whose accumulator is float.  exp(sink_h) joins the denominator after the last tile.  The result is multiplied
// coordinate by coordinate with sigmoid(gate) and written with a free row stride.  Queries at or past lens[b] give zeros.
#include "mma_tiles.cuh"
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kHQ = 64, kHPad = 8;              // queries per block; row padding (elements) against bank conflicts

template <int KT, int VD16>
__global__ void __launch_bounds__(128)
headmix_prompt_mma_kernel(const bf16* __restrict__ qmix, const bf16* __restrict__ keys, const bf16* __restrict__ v, long v_sb, long v_st,
                          const float* __restrict__ sink, const bf16* __restrict__ gate, long g_sb, long g_st,
                          const int* __restrict__ lens, int S, int H, int G, int D, int chunk, int window, bf16* __restrict__ out,
                          long out_stride) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DK = G * D, dk16 = DK / 16, vd16 = D / 16, ldk = DK + kHPad, ldv = D + kHPad;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                                              // [kHQ][ldk]
    auto Kst = [&](int st) { return Qs + kHQ * ldk + st * KT * ldk; };                         // [KT][ldk] each
    auto Vst = [&](int st) { return Qs + (kHQ + 2 * KT) * ldk + st * KT * ldv; };              // [KT][ldv] each
    const int q0 = blockIdx.x * kHQ, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = h / (H / G);
    const int len = min(lens[b], S);
    bf16* ob = out + ((long)b * S) * out_stride + (long)h * D;
    if (q0 >= len) {                                       // nothing but padding: zeros
        for (int i = tid; i < min(kHQ, S - q0) * (D / 2); i += 128) {
            const int r = i / (D / 2), c = (i % (D / 2)) * 2;
            *reinterpret_cast<unsigned*>(ob + (long)(q0 + r) * out_stride + c) = 0u;
        }
        return;
    }
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    for (int i = tid; i < kHQ * (DK / 8); i += 128) {
        const int r = i / (DK / 8), c = (i % (DK / 8)) * 8, t = q0 + r;
        *reinterpret_cast<uint4*>(Qs + r * ldk + c) =
            t < len ? *reinterpret_cast<const uint4*>(qmix + (((long)b * S + t) * H + h) * DK + c) : zero4;
    }
    const int r0 = warp * 16, g = lane >> 2, tq = lane & 3;
    float oacc[2 * VD16][4];
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int i0 = q0 + r0 + g, i1 = i0 + 8;               // this thread's two queries
    auto lower = [&](int i) {                              // the first position query i sees
        int lo = 0;
        if (chunk > 0) lo = (i / chunk) * chunk;
        if (window > 0) lo = max(lo, i - window + 1);
        return lo;
    };
    const int lo0 = lower(i0), lo1 = lower(i1);
    const float log2e = 1.4426950408889634f;
    const int jlo = lower(q0), jhi = min(q0 + kHQ - 1, len - 1);
    const bf16* kb = keys + (long)b * S * DK;
    const bf16* vb = v + (long)b * v_sb + (long)hk * D;
    auto fetch = [&](int kt, int st) {
        const int j0 = kt * KT;
        bf16 *Kd = Kst(st), *Vd = Vst(st);
        for (int c = lane * 8; c < DK; c += 256) {
#pragma unroll 4
            for (int r = warp; r < KT; r += 4) {
                const int j = j0 + r;
                cp16(Kd + r * ldk + c, kb + (long)min(j, len - 1) * DK + c, j < len);
            }
        }
        for (int c = lane * 8; c < D; c += 256) {
#pragma unroll 4
            for (int r = warp; r < KT; r += 4) {
                const int j = j0 + r;
                cp16(Vd + r * ldv + c, vb + (long)min(j, len - 1) * v_st + c, j < len);
            }
        }
        cp_commit();
    };
    const int kt0 = jlo / KT, kt1 = jhi / KT;
    fetch(kt0, 0);
    __syncthreads();                                       // the query tile is in place
    for (int kt = kt0; kt <= kt1; ++kt) {
        const int j0 = kt * KT, st = (kt - kt0) & 1;
        if (kt < kt1) { fetch(kt + 1, st ^ 1); cp_wait<1>(); } else cp_wait<0>();
        __syncthreads();                                   // tile kt has landed for everyone
        const int wlo = q0 + r0, whi = wlo + 15;
        // a warp whose queries see nothing of this tile skips it (tiles before its chunk / window, or after its last query)
        if (j0 <= whi && j0 + KT - 1 >= lower(wlo)) {
            const bf16 *Ks = Kst(st), *Vs = Vst(st);
            float sacc[KT / 8][4];
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
            for (int kk = 0; kk < dk16; ++kk) {
                unsigned qa[4];
                ldsm4(qa[0], qa[1], qa[2], qa[3], Qs + (r0 + (lane & 15)) * ldk + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < KT / 16; ++np) {     // two 8-key groups per ldmatrix
                    unsigned b0, b1, b2, b3;
                    ldsm4(b0, b1, b2, b3, Ks + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * ldk + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(sacc[2 * np], qa, b0, b1);
                    mma16816(sacc[2 * np + 1], qa, b2, b3);
                }
            }
            // mask and running softmax (float, in base 2); a thread holds KT/4 scores of query i0 and as many of i1.  A tile that
            // every query of the warp sees in full needs no mask.
            const bool full = j0 + KT - 1 <= wlo && j0 >= lower(whi) && j0 + KT - 1 < len;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < KT / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    bool vis = true;
                    if (!full) {
                        const int j = j0 + n * 8 + tq * 2 + (e & 1);
                        vis = (e < 2) ? (j <= i0 && j >= lo0 && j < len) : (j <= i1 && j >= lo1 && j < len);
                    }
                    sacc[n][e] = vis ? sacc[n][e] * log2e : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sacc[n][e]);
                }
            float corr[2], base[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float mn = fmaxf(mrow[r], mx[r]);
                base[r] = mn == -INFINITY ? 0.f : mn;      // nothing visible so far: every weight is exp(-inf) = 0
                corr[r] = exp2f(mrow[r] - base[r]);
                mrow[r] = mn;
            }
            float ls[2] = {0.f, 0.f};
#pragma unroll
            for (int n = 0; n < KT / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    sacc[n][e] = exp2f(sacc[n][e] - base[e >> 1]);
                    ls[e >> 1] += sacc[n][e];
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * corr[r] + ls[r];
#pragma unroll
            for (int n = 0; n < 2 * VD16; ++n) { oacc[n][0] *= corr[0]; oacc[n][1] *= corr[0]; oacc[n][2] *= corr[1]; oacc[n][3] *= corr[1]; }
#pragma unroll
            for (int kp = 0; kp < KT / 16; ++kp) {
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
        }
        __syncthreads();                                   // the stage may be refilled
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    float fac[2] = {1.f, 1.f};
    if (sink) {                                            // exp(sink) joins the denominator; the larger of the two maxima is the base
        const float s2 = sink[h] * log2e;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float mn = fmaxf(mrow[r], s2);
            fac[r] = exp2f(mrow[r] - mn);                  // 0 when the row saw no key
            lrow[r] = lrow[r] * fac[r] + exp2f(s2 - mn);
        }
    }
    const float inv0 = (i0 < len && lrow[0] > 0.f) ? fac[0] / lrow[0] : 0.f, inv1 = (i1 < len && lrow[1] > 0.f) ? fac[1] / lrow[1] : 0.f;
#pragma unroll
    for (int n = 0; n < 2 * VD16; ++n) {
        if (n < 2 * vd16) {
            const int c = n * 8 + tq * 2;
            float a0 = oacc[n][0] * inv0, a1 = oacc[n][1] * inv0, c0 = oacc[n][2] * inv1, c1 = oacc[n][3] * inv1;
            if (gate) {
                if (i0 < len) {
                    const bf16* gp = gate + (long)b * g_sb + (long)i0 * g_st + (long)h * D + c;
                    a0 *= sigmoidf_(__bfloat162float(gp[0])); a1 *= sigmoidf_(__bfloat162float(gp[1]));
                }
                if (i1 < len) {
                    const bf16* gp = gate + (long)b * g_sb + (long)i1 * g_st + (long)h * D + c;
                    c0 *= sigmoidf_(__bfloat162float(gp[0])); c1 *= sigmoidf_(__bfloat162float(gp[1]));
                }
            }
            if (i0 < S) *reinterpret_cast<unsigned*>(ob + (long)i0 * out_stride + c) = pack2(a0, a1);
            if (i1 < S) *reinterpret_cast<unsigned*>(ob + (long)i1 * out_stride + c) = pack2(c0, c1);
        }
    }
}

static size_t headmix_prompt_smem(int DK, int D, int KT) {
    return (size_t)((kHQ + 2 * KT) * (DK + kHPad) + 2 * KT * (D + kHPad)) * sizeof(bf16);
}

// The fused kernel takes bfloat16 with the head size in whole 16s up to 256, 16-byte aligned rows and a key row that fits on chip.
bool headmix_prompt_mma_fits(const void* v, long v_sb, long v_st, int G, int D, const void* out, long out_stride) {
    auto a16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
    return D % 16 == 0 && D <= 256 && a16(v) && v_sb % 8 == 0 && v_st % 8 == 0 && (uintptr_t)out % 4 == 0 && out_stride % 2 == 0 &&
           headmix_prompt_smem(G * D, D, 16) <= 200 * 1024;
}

void headmix_prompt_mma(const void* qmix, const void* keys, const void* v, long v_sb, long v_st, const float* sink, const void* gate,
                        long g_sb, long g_st, const int* lens, int B, int S, int H, int G, int D, int chunk, int window, void* out,
                        long out_stride, cudaStream_t s) {
    // keys per tile: the most that leaves room for two blocks per SM (each block has only four warps, and a second block hides the
    // first one's waits on its staged tiles); if none does, the most that fits at all
    int kt = 0;
    for (int c : {64, 32, 16}) if (!kt && headmix_prompt_smem(G * D, D, c) <= 112 * 1024) kt = c;
    for (int c : {64, 32, 16}) if (!kt && headmix_prompt_smem(G * D, D, c) <= 200 * 1024) kt = c;
    const size_t smem = headmix_prompt_smem(G * D, D, kt);
    dim3 grid((S + kHQ - 1) / kHQ, H, B);
#define SEQMIX_HPM(KT, Bv)                                                                                                            \
    do {                                                                                                                              \
        cudaFuncSetAttribute(headmix_prompt_mma_kernel<KT, Bv>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);             \
        headmix_prompt_mma_kernel<KT, Bv><<<grid, 128, smem, s>>>((const bf16*)qmix, (const bf16*)keys, (const bf16*)v, v_sb, v_st, sink,   \
                                                                  (const bf16*)gate, g_sb, g_st, lens, S, H, G, D, chunk, window,       \
                                                                  (bf16*)out, out_stride);                                            \
    } while (0)
#define SEQMIX_HPM_V(KT) do { if (D <= 64) SEQMIX_HPM(KT, 4); else if (D <= 128) SEQMIX_HPM(KT, 8); else SEQMIX_HPM(KT, 16); } while (0)
    if (kt == 64) SEQMIX_HPM_V(64); else if (kt == 32) SEQMIX_HPM_V(32); else SEQMIX_HPM_V(16);
#undef SEQMIX_HPM_V
#undef SEQMIX_HPM
}

}  // namespace seqmix
