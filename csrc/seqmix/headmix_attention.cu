// Softmax attention whose heads' scores are mixed before the softmax ("talking heads"), with keys that double as values, a sink term
// in the denominator, aligned chunks and / or a sliding window.
//
// The mixing is linear in the queries, so it is moved onto them: with score_g(i,j) = c_g q_g(i) . k_kv(g)(j) and the mixed score
// s_h = sum_g T[h,g] score_g, head h's mixed query against key/value head c is  Q'[h,c,:] = sum_{g in group c} T[h,g] c_g q_g  and
// s_h(i,j) = sum_c Q'[h,c,:] . k_c(j): ONE dot product of length G*D between head h's mixed query row and the position's key row
// with all key heads side by side.  After that the attention is an ordinary one with key size G*D (all heads read the same key
// rows) and value size D (head h reads value head kv(h)).
//   headmix_qk_prepare : rotation of the queries (float, rotate-half pairs), the mixing into Q' [B,S,H,G*D]; rotation of the keys into
//                        the key rows / the key ring; the keys as they come into the value ring
//   headmix_attend     : a (query, head) per block, its warps split the visible keys, partial softmaxes meet in shared memory; the
//                        sink joins the denominator there; the result times sigmoid(gate) is written.  Used for single tokens against
//                        the ring (any dtype) and for prompts in float or with sizes the tensor-core kernel does not take.
// Everything between the loads and the store is float.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

// grid (S, B), 128 threads.  q [B,S,H,D] and k [B,S,G,D] are views (strides in elements); mixw [H,H] float = T[h,g] * c_g.
template <typename T>
__global__ void __launch_bounds__(128) headmix_qk_prepare_kernel(
    const T* __restrict__ q, long q_sb, long q_st, const T* __restrict__ k, long k_sb, long k_st, const float* __restrict__ mixw,
    int dims, const float* __restrict__ inv_freq, const int* __restrict__ pos0, const int* __restrict__ lens,
    const int* __restrict__ slots, T* __restrict__ kcache, T* __restrict__ vcache, int ring, T* __restrict__ qmix, T* __restrict__ rows,
    int S, int H, int G, int D) {
    extern __shared__ __align__(16) float qs[];   // [H][D] rotated queries
    const int t = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int len = min(lens[b], S);
    if (t >= len) return;                          // padding: nothing is read from these rows later
    const int p = pos0[b] + t, half = dims / 2, rest = D - dims;
    const T* qr = q + (long)b * q_sb + (long)t * q_st;
    const T* kr = k + (long)b * k_sb + (long)t * k_st;
    const bool keep = t >= len - ring;             // the last `ring` tokens go to the rings
    const long crow = ((long)slots[b] * ring + (p % ring)) * G * D;
    T* rrow = rows ? rows + ((long)b * S + t) * G * D : nullptr;
    // rotated pairs: the angle of pair i is the same for every query and key head, so sin / cos are formed once per pair and the
    // thread walks the heads (the threads split into groups over the heads when the pairs are few)
    if (half > 0) {
        const int nh = H + G, groups = max(1, min(nh, 128 / half));
        for (int u = tid; u < half * groups; u += 128) {
            const int g = u / half, i = u - g * half;
            float sn, cs;
            sincosf((float)p * inv_freq[i], &sn, &cs);
            for (int h = g; h < nh; h += groups) {
                if (h < H) {
                    const float a = ldf(qr + h * D + i), c = ldf(qr + h * D + i + half);
                    qs[h * D + i] = a * cs - c * sn;
                    qs[h * D + i + half] = c * cs + a * sn;
                } else {
                    const int c0 = (h - H) * D + i;
                    const T ka = kr[c0], kb = kr[c0 + half];
                    const float a = ldf(&ka), cc = ldf(&kb);
                    const float x = a * cs - cc * sn, y = cc * cs + a * sn;
                    if (rrow) { stf(rrow + c0, x); stf(rrow + c0 + half, y); }
                    if (keep) {
                        stf(kcache + crow + c0, x); stf(kcache + crow + c0 + half, y);
                        vcache[crow + c0] = ka; vcache[crow + c0 + half] = kb;
                    }
                }
            }
        }
    }
    for (int u = tid; u < H * rest; u += 128) {    // coordinates past the rotated ones pass unchanged
        const int h = u / rest, d = h * D + dims + (u - h * rest);
        qs[d] = ldf(qr + d);
    }
    for (int u = tid; u < G * rest; u += 128) {
        const int c = u / rest, d = c * D + dims + (u - c * rest);
        const T kv = kr[d];
        if (rrow) rrow[d] = kv;
        if (keep) { kcache[crow + d] = kv; vcache[crow + d] = kv; }
    }
    __syncthreads();
    const int hpg = H / G;
    T* qm = qmix + ((long)b * S + t) * H * G * D;
    if (D % 4 == 0) {                              // four coordinates per thread
        const int d4 = D / 4;
        for (int o = tid; o < H * G * d4; o += 128) {
            const int h = o / (G * d4), r = o - h * G * d4, c = r / d4, d = (r - c * d4) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int g = c * hpg; g < (c + 1) * hpg; ++g) {
                const float m = mixw[h * H + g];
                const float4 v = *reinterpret_cast<const float4*>(qs + g * D + d);
                acc.x = fmaf(m, v.x, acc.x); acc.y = fmaf(m, v.y, acc.y); acc.z = fmaf(m, v.z, acc.z); acc.w = fmaf(m, v.w, acc.w);
            }
            st4(qm + ((long)h * G + c) * D + d, acc);
        }
        return;
    }
    for (int o = tid; o < H * G * D; o += 128) {
        const int h = o / (G * D), r = o - h * G * D, c = r / D, d = r - c * D;
        float acc = 0.f;
        for (int g = c * hpg; g < (c + 1) * hpg; ++g) acc = fmaf(mixw[h * H + g], qs[g * D + d], acc);
        stf(qm + o, acc);
    }
}

void headmix_qk_prepare(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, int bf, const float* mixw, int dims,
                        const float* inv_freq, const int* pos0, const int* lens, const int* slots, void* kcache, void* vcache, int ring,
                        void* qmix, void* rows, int B, int S, int H, int G, int D, cudaStream_t s) {
    if (B == 0 || S == 0) return;
    dim3 grid(S, B);
    const size_t smem = (size_t)H * D * sizeof(float);
    if (bf) {
        cudaFuncSetAttribute(headmix_qk_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        headmix_qk_prepare_kernel<bf16><<<grid, 128, smem, s>>>((const bf16*)q, q_sb, q_st, (const bf16*)k, k_sb, k_st, mixw, dims, inv_freq, pos0,
                                                               lens, slots, (bf16*)kcache, (bf16*)vcache, ring, (bf16*)qmix, (bf16*)rows, S, H, G, D);
    } else {
        cudaFuncSetAttribute(headmix_qk_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        headmix_qk_prepare_kernel<float><<<grid, 128, smem, s>>>((const float*)q, q_sb, q_st, (const float*)k, k_sb, k_st, mixw, dims, inv_freq,
                                                                pos0, lens, slots, (float*)kcache, (float*)vcache, ring, (float*)qmix,
                                                                (float*)rows, S, H, G, D);
    }
}

constexpr int kAttWarps = 4, kValPerLane = 8;      // value size up to 32 * kValPerLane

// grid (S, H, B), 128 threads: block = one (query, head).  Keys are rows of `keys` [*, DK] (DK = G*D), values rows of `vals` with
// row stride v_stride, head kv(h)'s D numbers at offset kv(h) * D.  ring > 0: single tokens (S = 1) at position pos0[b]; position j
// sits in row j % ring of block slots[b].  ring == 0: a prompt from position 0; position j is row j of sequence b.
template <typename T>
__global__ void __launch_bounds__(32 * kAttWarps) headmix_attend_kernel(
    const T* __restrict__ qmix, const T* __restrict__ keys, long key_sb, const T* __restrict__ vals, long v_sb, long v_stride,
    const float* __restrict__ sink, const T* __restrict__ gate, long g_sb, long g_st, const int* __restrict__ slots,
    const int* __restrict__ pos0, const int* __restrict__ lens, int chunk, int window, int ring, int S, int H, int G, int D,
    T* __restrict__ out, long out_stride) {
    extern __shared__ float sm[];
    const int DK = G * D;
    float* qv = sm;                                // [DK]
    float* pm = qv + DK;                           // [warps] running maxima
    float* pl = pm + kAttWarps;                    // [warps] running sums
    float* pacc = pl + kAttWarps;                  // [warps][D]
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int len = min(lens[b], S);
    T* o = out + ((long)b * S + t) * out_stride + (long)h * D;
    if (t >= len) {
        for (int d = tid; d < D; d += 32 * kAttWarps) stf(o + d, 0.f);
        return;
    }
    const int i = ring > 0 ? pos0[b] : t;          // the query's position
    int lo = 0;
    if (chunk > 0) lo = (i / chunk) * chunk;
    if (window > 0) lo = max(lo, i - window + 1);
    const T* qr = qmix + (((long)b * S + t) * H + h) * DK;
    for (int d = tid; d < DK; d += 32 * kAttWarps) qv[d] = ldf(qr + d);
    __syncthreads();
    const T* kb = keys + (ring > 0 ? (long)slots[b] * key_sb : (long)b * key_sb);
    const T* vb = vals + (ring > 0 ? (long)slots[b] * v_sb : (long)b * v_sb) + (long)(h / (H / G)) * D;
    float m = -INFINITY, l = 0.f, acc[kValPerLane];
#pragma unroll
    for (int x = 0; x < kValPerLane; ++x) acc[x] = 0.f;
    for (int j = lo + w; j <= i; j += kAttWarps) {
        const long row = ring > 0 ? j % ring : j;
        const T* kr = kb + row * DK;
        float s = 0.f;
        for (int d = lane; d < DK; d += 32) s = fmaf(qv[d], ldf(kr + d), s);
        s = warp_sum(s);
        const float mn = fmaxf(m, s), corr = expf(m - mn), pj = expf(s - mn);
        l = l * corr + pj;
        const T* vr = vb + row * v_stride;
#pragma unroll
        for (int x = 0; x < kValPerLane; ++x) {
            const int d = lane + 32 * x;
            if (d < D) acc[x] = fmaf(pj, ldf(vr + d), acc[x] * corr);
        }
        m = mn;
    }
    if (lane == 0) { pm[w] = m; pl[w] = l; }
#pragma unroll
    for (int x = 0; x < kValPerLane; ++x) {
        const int d = lane + 32 * x;
        if (d < D) pacc[w * D + d] = acc[x];
    }
    __syncthreads();
    float M = sink ? sink[h] : -INFINITY;
#pragma unroll
    for (int x = 0; x < kAttWarps; ++x) M = fmaxf(M, pm[x]);
    float L = sink ? expf(sink[h] - M) : 0.f, f[kAttWarps];
#pragma unroll
    for (int x = 0; x < kAttWarps; ++x) { f[x] = pm[x] == -INFINITY ? 0.f : expf(pm[x] - M); L = fmaf(pl[x], f[x], L); }
    const T* gr = gate ? gate + (long)b * g_sb + (long)t * g_st + (long)h * D : nullptr;
    for (int d = tid; d < D; d += 32 * kAttWarps) {
        float v = 0.f;
#pragma unroll
        for (int x = 0; x < kAttWarps; ++x) v = fmaf(pacc[x * D + d], f[x], v);
        v /= L;
        if (gr) v *= sigmoidf_(ldf(gr + d));
        stf(o + d, v);
    }
}

bool headmix_attend(const void* qmix, const void* keys, long key_sb, const void* vals, long v_sb, long v_stride, int bf, const float* sink,
                    const void* gate, long g_sb, long g_st, const int* slots, const int* pos0, const int* lens, int chunk, int window,
                    int ring, int B, int S, int H, int G, int D, void* out, long out_stride, cudaStream_t s) {
    if (D > 32 * kValPerLane) return false;
    const size_t smem = sizeof(float) * ((size_t)G * D + 2 * kAttWarps + (size_t)kAttWarps * D);
    if (smem > 96 * 1024) return false;
    if (B == 0 || S == 0) return true;
    dim3 grid(S, H, B);
#define SEQMIX_HMA(T)                                                                                                                 \
    do {                                                                                                                              \
        cudaFuncSetAttribute(headmix_attend_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);                       \
        headmix_attend_kernel<T><<<grid, 32 * kAttWarps, smem, s>>>((const T*)qmix, (const T*)keys, key_sb, (const T*)vals, v_sb, v_stride, \
                                                                    sink, (const T*)gate, g_sb, g_st, slots, pos0, lens, chunk, window,   \
                                                                    ring, S, H, G, D, (T*)out, out_stride);                           \
    } while (0)
    if (bf) SEQMIX_HMA(bf16); else SEQMIX_HMA(float);
#undef SEQMIX_HMA
    return true;
}

}  // namespace seqmix
