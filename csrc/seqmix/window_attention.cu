// Grouped-query attention over a sliding window: query position i sees i - window < j <= i; query head h reads key/value head
// h / (H/G).  Scores are q.k * scale, capped as softcap * tanh(score / softcap) when softcap > 0; scores, weights and sums are
// float.  The weights are a softmax over the visible keys, or — when a score bias per head is given — sigmoid(score + bias[h]) of
// each visible key by itself, not normalised over the keys.  Each head's result may be multiplied by sigmoid(gate[b,t,h]) and a
// constant before it is written (row stride free: several mixers write side by side into one buffer).
//   window_qk_prepare      : RMS norm of queries and keys in place, per head (one weight vector of D numbers each) or over the whole
//                            projection at once (weights of H*D and G*D numbers); then, when frequencies are given, rotation of the
//                            first `dims` coordinates of every head at the token's position (pairs i, i + dims/2; angles in float);
//                            and the last `ring` real tokens' keys and values to the sequence's ring rows (position mod ring);
//                            with no keys given only the queries are prepared (a layer that reads another layer's ring)
//   window_attention_prompt: prompts starting at position 0, keys and values of the call itself.  A block owns 16 consecutive
//                            queries of one head (4 warps x 4 queries); key / value rows come through shared memory 32 at a time;
//                            in the score pass a lane owns one key (4 queries per shared-memory read), in the value pass a lane
//                            owns value columns lane, lane + 32, ...  (float, and bfloat16 of sizes the fused tensor-core kernel
//                            of window_prefill.cu does not take)
//   window_attention_token : one query per (sequence, head) against the ring.  A block owns up to 4 query heads of one key/value
//                            group (a warp each) over one stretch of ring rows, staged 32 rows at a time for all of them; a
//                            second kernel folds the stretches' partial softmaxes.
#include <math.h>

#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

template <typename T>
__global__ void window_qk_prepare_kernel(T* q, long q_sb, long q_st, T* k, long k_sb, long k_st, const T* __restrict__ v, long v_sb,
                                         long v_st, const float* __restrict__ qw, const float* __restrict__ kw, int norm_all, float eps,
                                         const float* __restrict__ inv_freq, int dims, const int* __restrict__ pos0,
                                         const int* __restrict__ lens, const int* __restrict__ slots, T* kcache, T* vcache, int ring, int S,
                                         int H, int G, int D, int V) {
    __shared__ float red[2][8];
    const int row = blockIdx.x, b = row / S, t = row - b * S, lane = threadIdx.x;
    const int len = min(lens[b], S);
    if (t >= len) return;
    const bool keep = k != nullptr && t >= len - ring;
    const int pos = pos0[b] + t, half = inv_freq ? dims / 2 : 0, rot = 2 * half;
    const long cr = k ? ((long)slots[b] * ring + pos % ring) * G : 0;
    T* qrow = q + (long)b * q_sb + (long)t * q_st;
    T* krow = k ? k + (long)b * k_sb + (long)t * k_st : nullptr;
    float inv_all[2] = {1.f, 1.f};
    if (norm_all) {                                          // one statistic over all heads of the queries, one over all of the keys
        const int tid = threadIdx.y * 32 + lane, nthr = blockDim.y * 32;
        float sq = 0.f, sk = 0.f;
        if (qw) for (int x = tid; x < H * D; x += nthr) { const float e = ldf(qrow + x); sq = fmaf(e, e, sq); }
        if (kw && krow) for (int x = tid; x < G * D; x += nthr) { const float e = ldf(krow + x); sk = fmaf(e, e, sk); }
        sq = warp_sum(sq); sk = warp_sum(sk);
        if (lane == 0) { red[0][threadIdx.y] = sq; red[1][threadIdx.y] = sk; }
        __syncthreads();
        sq = sk = 0.f;
        for (int x = 0; x < (int)blockDim.y; ++x) { sq += red[0][x]; sk += red[1][x]; }
        inv_all[0] = 1.f / sqrtf(sq / (float)(H * D) + eps);
        inv_all[1] = 1.f / sqrtf(sk / (float)(G * D) + eps);
    }
    const int units = krow ? H + 2 * G : H;
    for (int u = threadIdx.y; u < units; u += blockDim.y) {
        if (u < H + G) {
            const bool isq = u < H;
            const int hh = isq ? u : u - H;
            T* p = (isq ? qrow : krow) + (long)hh * D;
            const float* w = isq ? qw : kw;
            T* dst = (!isq && keep) ? kcache + (cr + hh) * D : nullptr;
            float inv = 1.f;
            if (w && norm_all) {
                inv = inv_all[isq ? 0 : 1];
                w += (long)hh * D;
            } else if (w) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) { const float x = ldf(p + d); ss = fmaf(x, x, ss); }
                inv = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
            }
            if (!(w || dst || rot)) continue;
            for (int i = lane; i < half; i += 32) {          // a lane reads both members of a pair before it writes them
                float x0 = ldf(p + i), x1 = ldf(p + i + half);
                if (w) { x0 *= inv * w[i]; x1 *= inv * w[i + half]; }
                float sn, cs;
                sincosf((float)pos * inv_freq[i], &sn, &cs);
                const float y0 = x0 * cs - x1 * sn, y1 = x1 * cs + x0 * sn;
                stf(p + i, y0); stf(p + i + half, y1);
                if (dst) { stf(dst + i, y0); stf(dst + i + half, y1); }
            }
            for (int d = rot + lane; d < D; d += 32) {
                const float x = w ? ldf(p + d) * inv * w[d] : ldf(p + d);
                if (w) stf(p + d, x);
                if (dst) stf(dst + d, x);
            }
        } else if (keep) {
            const int hh = u - H - G;
            const T* p = v + (long)b * v_sb + (long)t * v_st + (long)hh * V;
            T* dst = vcache + (cr + hh) * V;
            for (int d = lane; d < V; d += 32) dst[d] = p[d];
        }
    }
}

__device__ __forceinline__ float cap_score(float s, float softcap, float inv_cap) { return softcap > 0.f ? softcap * tanhf(s * inv_cap) : s; }

constexpr int kKeys = 32;       // keys per shared-memory chunk
constexpr int kQW = 4;          // queries per warp (prompts)
constexpr int kWarps = 4;

// shared: Ks [kKeys][D+1], Vs [kKeys][V], Qs [kWarps][D][kQW], Ps [kWarps][kKeys][kQW]
template <typename T, int VPL>
__global__ void __launch_bounds__(128) window_prompt_kernel(
    const T* __restrict__ q, long q_sb, long q_st, const T* __restrict__ k, long k_sb, long k_st, const T* __restrict__ v, long v_sb,
    long v_st, const T* __restrict__ gate, long g_sb, long g_st, const int* __restrict__ lens, int S, int H, int G, int D, int V,
    int window, float scale, float softcap, const float* __restrict__ score_bias, T* __restrict__ out, long out_stride, float out_scale) {
    extern __shared__ float sm[];
    const int DP = D + 1;
    float* Ks = sm;
    float* Vs = Ks + kKeys * DP;
    float* Qs = Vs + kKeys * V;
    float* Ps = Qs + kWarps * D * kQW;
    const int i0 = blockIdx.x * (kWarps * kQW), h = blockIdx.y, b = blockIdx.z, g = h / (H / G);
    const bool sig = score_bias != nullptr;                          // independent sigmoid weights instead of a softmax
    const float sbias = sig ? score_bias[h] : 0.f;
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int len = min(lens[b], S);
    const int iq0 = i0 + wp * kQW;                                   // this warp's first query position
    float* Qw = Qs + wp * D * kQW;
    float* Pw = Ps + wp * kKeys * kQW;
    for (int x = lane; x < D * kQW; x += 32) {
        const int d = x / kQW, rq = x - d * kQW, i = iq0 + rq;
        Qw[x] = i < len ? ldf(q + (long)b * q_sb + (long)i * q_st + (long)h * D + d) : 0.f;
    }
    float m[kQW], l[kQW], acc[kQW][VPL];
#pragma unroll
    for (int rq = 0; rq < kQW; ++rq) {
        m[rq] = -INFINITY; l[rq] = 0.f;
#pragma unroll
        for (int c = 0; c < VPL; ++c) acc[rq][c] = 0.f;
    }
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
    const int last = min(i0 + kWarps * kQW, len) - 1;                // last key any query of the block sees
    const int first = max(0, i0 - window + 1);
    const T* kb = k + (long)b * k_sb + (long)g * D;
    const T* vb = v + (long)b * v_sb + (long)g * V;
    for (int c0 = first; c0 <= last; c0 += kKeys) {
        __syncthreads();
        for (int x = tid; x < kKeys * D; x += 128) {
            const int jj = x / D, d = x - jj * D, j = c0 + jj;
            Ks[jj * DP + d] = j <= last ? ldf(kb + (long)j * k_st + d) : 0.f;
        }
        for (int x = tid; x < kKeys * V; x += 128) {
            const int jj = x / V, d = x - jj * V, j = c0 + jj;
            Vs[x] = j <= last ? ldf(vb + (long)j * v_st + d) : 0.f;
        }
        __syncthreads();
        // is any of this warp's queries inside the chunk's reach?
        if (c0 > iq0 + kQW - 1 || c0 + kKeys - 1 <= iq0 - window || iq0 >= len) continue;
        float s[kQW];
#pragma unroll
        for (int rq = 0; rq < kQW; ++rq) s[rq] = 0.f;
        const float* kr = Ks + lane * DP;
        for (int d = 0; d < D; ++d) {
            const float kv = kr[d];
            const float4 qv = *reinterpret_cast<const float4*>(Qw + d * kQW);
            s[0] = fmaf(qv.x, kv, s[0]); s[1] = fmaf(qv.y, kv, s[1]); s[2] = fmaf(qv.z, kv, s[2]); s[3] = fmaf(qv.w, kv, s[3]);
        }
        const int j = c0 + lane;
        float corr[kQW];
#pragma unroll
        for (int rq = 0; rq < kQW; ++rq) {
            const int i = iq0 + rq;
            const bool ok = i < len && j <= i && j > i - window;
            const float sc = ok ? cap_score(s[rq] * scale, softcap, inv_cap) : -INFINITY;
            if (sig) {
                corr[rq] = 1.f;
                Pw[lane * kQW + rq] = ok ? sigmoidf_(sc + sbias) : 0.f;
                continue;
            }
            float mx = sc;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mn = fmaxf(m[rq], mx);
            const float p = (ok && mn > -INFINITY) ? expf(sc - mn) : 0.f;
            corr[rq] = (m[rq] > -INFINITY) ? expf(m[rq] - mn) : 0.f;
            m[rq] = mn;
            l[rq] = fmaf(l[rq], corr[rq], p);                        // per-lane part of the sum; folded at the end
            Pw[lane * kQW + rq] = p;
        }
#pragma unroll
        for (int rq = 0; rq < kQW; ++rq)
#pragma unroll
            for (int c = 0; c < VPL; ++c) acc[rq][c] *= corr[rq];
        __syncwarp();
        for (int jj = 0; jj < kKeys; ++jj) {
            const float4 p = *reinterpret_cast<const float4*>(Pw + jj * kQW);
#pragma unroll
            for (int c = 0; c < VPL; ++c) {
                const int col = lane + 32 * c;
                const float vv = col < V ? Vs[jj * V + col] : 0.f;
                acc[0][c] = fmaf(p.x, vv, acc[0][c]); acc[1][c] = fmaf(p.y, vv, acc[1][c]);
                acc[2][c] = fmaf(p.z, vv, acc[2][c]); acc[3][c] = fmaf(p.w, vv, acc[3][c]);
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int rq = 0; rq < kQW; ++rq) {
        const int i = iq0 + rq;
        if (i >= S) continue;
        const float lt = sig ? 1.f : warp_sum(l[rq]);
        float f = 0.f;
        if (i < len && lt > 0.f) {
            f = out_scale / lt;
            if (gate) f *= sigmoidf_(ldf(gate + (long)b * g_sb + (long)i * g_st + h));
        }
        T* o = out + ((long)b * S + i) * out_stride + (long)h * V;
#pragma unroll
        for (int c = 0; c < VPL; ++c) {
            const int col = lane + 32 * c;
            if (col < V) stf(o + col, acc[rq][c] * f);
        }
    }
}

// 16 bytes at a time when the row allows it (VEC), else element by element; rows at or past `valid` become zeros
template <typename T, bool VEC>
__device__ __forceinline__ void stage_rows(float* dst, int ld, const T* __restrict__ src, long row_stride, int valid, int cols, int tid,
                                           int nthr) {
    if (VEC) {
        constexpr int E = 16 / sizeof(T);
        const int per = cols / E;
        for (int x = tid; x < kKeys * per; x += nthr) {
            const int jj = x / per, c = (x - jj * per) * E;
            float* d = dst + jj * ld + c;
            if (jj < valid) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src + (long)jj * row_stride + c);
                const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int u = 0; u < E; ++u) d[u] = ldf(e + u);
            } else {
#pragma unroll
                for (int u = 0; u < E; ++u) d[u] = 0.f;
            }
        }
    } else {
        for (int x = tid; x < kKeys * cols; x += nthr) {
            const int jj = x / cols, c = x - jj * cols;
            dst[jj * ld + c] = jj < valid ? ldf(src + (long)jj * row_stride + c) : 0.f;
        }
    }
}

// Single tokens against their rings.  grid (ring splits, head quads, sequences): a block takes up to 4 query heads of one key/value
// group (a warp each) over one stretch of ring rows, staged 32 rows at a time for all of them, and leaves a partial softmax per
// head: part_m / part_l [B, H, splits], part_acc [B, H, splits, V].  shared: Ks [kKeys][D+1], Vs [kKeys][V], Qs [4][D], Ps [4][kKeys]
template <typename T, int VPL, bool VEC>
__global__ void __launch_bounds__(128) window_token_kernel(
    const T* __restrict__ q, long q_sb, const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ slots,
    const int* __restrict__ pos0, const int* __restrict__ lens, int ring, int H, int G, int D, int V, int window, float scale,
    float softcap, const float* __restrict__ score_bias, int splits, float* __restrict__ part_m, float* __restrict__ part_l,
    float* __restrict__ part_acc) {
    extern __shared__ float sm[];
    const int DP = D + 1;
    float* Ks = sm;
    float* Vs = Ks + kKeys * DP;
    float* Qs = Vs + kKeys * V;
    float* Ps = Qs + kWarps * D;
    const int split = blockIdx.x, b = blockIdx.z, HG = H / G, qpg = (HG + kWarps - 1) / kWarps;
    const int g = blockIdx.y / qpg, hq = (blockIdx.y - g * qpg) * kWarps;
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const bool has = hq + wp < HG;                                   // this warp has a head
    const int h = g * HG + hq + wp;
    const bool sig = score_bias != nullptr;                          // independent sigmoid weights: the partial results are plain sums
    const float sbias = (sig && has) ? score_bias[h] : 0.f;
    const int p = pos0[b];
    const int rows = lens[b] > 0 ? min(ring, p + 1) : 0;             // ring rows that hold a position (rows 0..p before the ring wraps)
    int per = (rows + splits - 1) / splits;
    per = (per + kKeys - 1) / kKeys * kKeys;
    const int r0 = split * per, r1 = min(rows, r0 + per);
    float* Qw = Qs + wp * D;
    float* Pw = Ps + wp * kKeys;
    if (has)
        for (int d = lane; d < D; d += 32) Qw[d] = ldf(q + (long)b * q_sb + (long)h * D + d);
    float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) acc[c] = 0.f;
    const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
    const T* kb = kcache + (long)slots[b] * ring * G * D + (long)g * D;
    const T* vb = vcache + (long)slots[b] * ring * G * V + (long)g * V;
    for (int c0 = r0; c0 < r1; c0 += kKeys) {
        __syncthreads();
        stage_rows<T, VEC>(Ks, DP, kb + (long)c0 * G * D, (long)G * D, r1 - c0, D, tid, 128);
        stage_rows<T, VEC>(Vs, V, vb + (long)c0 * G * V, (long)G * V, r1 - c0, V, tid, 128);
        __syncthreads();
        if (!has) continue;
        float s = 0.f;
        const float* kr = Ks + lane * DP;
        for (int d = 0; d < D; ++d) s = fmaf(Qw[d], kr[d], s);
        const int rr = c0 + lane;
        int back = (p - rr) % ring;                                  // how far back the position of ring row rr lies
        if (back < 0) back += ring;
        const bool ok = rr < r1 && back < window && p - back >= 0;
        const float sc = ok ? cap_score(s * scale, softcap, inv_cap) : -INFINITY;
        float pr, corr;
        if (sig) {
            pr = ok ? sigmoidf_(sc + sbias) : 0.f;
            corr = 1.f;
        } else {
            float mx = sc;
#pragma unroll
            for (int w = 16; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
            const float mn = fmaxf(m, mx);
            pr = (ok && mn > -INFINITY) ? expf(sc - mn) : 0.f;
            corr = (m > -INFINITY) ? expf(m - mn) : 0.f;
            m = mn;
            l = fmaf(l, corr, pr);
        }
        Pw[lane] = pr;
#pragma unroll
        for (int c = 0; c < VPL; ++c) acc[c] *= corr;
        __syncwarp();
        for (int jj = 0; jj < kKeys; ++jj) {
            const float pj = Pw[jj];
#pragma unroll
            for (int c = 0; c < VPL; ++c) {
                const int col = lane + 32 * c;
                acc[c] = fmaf(pj, col < V ? Vs[jj * V + col] : 0.f, acc[c]);
            }
        }
        __syncwarp();
    }
    if (!has) return;
    l = warp_sum(l);
    if (sig) { m = 0.f; l = split == 0 ? 1.f : 0.f; }              // the merge then adds the stretches' sums and divides by one
    const long o = ((long)b * H + h) * splits + split;
    if (lane == 0) { part_m[o] = m; part_l[o] = l; }
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
        const int col = lane + 32 * c;
        if (col < V) part_acc[o * V + col] = acc[c];
    }
}

// grid (H, B): the splits' partial softmaxes of one (sequence, head) folded, gated, scaled and written
template <typename T>
__global__ void window_token_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                          const float* __restrict__ part_acc, const T* __restrict__ gate, long g_sb, int H, int V,
                                          int splits, T* __restrict__ out, long out_stride, float out_scale) {
    const int h = blockIdx.x, b = blockIdx.y;
    const long o = ((long)b * H + h) * splits;
    float mt = -INFINITY;
    for (int s = 0; s < splits; ++s) mt = fmaxf(mt, part_m[o + s]);
    float lt = 0.f;
    for (int s = 0; s < splits; ++s)
        if (part_m[o + s] > -INFINITY) lt = fmaf(part_l[o + s], expf(part_m[o + s] - mt), lt);
    float f = lt > 0.f ? out_scale / lt : 0.f;
    if (gate) f *= sigmoidf_(ldf(gate + (long)b * g_sb + h));
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < splits; ++s)
            if (part_m[o + s] > -INFINITY) a = fmaf(part_acc[(o + s) * V + c], expf(part_m[o + s] - mt), a);
        stf(out + (long)b * out_stride + (long)h * V + c, a * f);
    }
}

void window_qk_prepare(void* q, long q_sb, long q_st, void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st, int bf,
                       const float* qw, const float* kw, int norm_all, float eps, const float* inv_freq, int dims, const int* pos0,
                       const int* lens, const int* slots, void* kcache, void* vcache, int ring, int B, int S, int H, int G, int D, int V,
                       cudaStream_t s) {
    if (B * S == 0) return;
    dim3 grid(B * S), block(32, 8);
    if (bf)
        window_qk_prepare_kernel<bf16><<<grid, block, 0, s>>>((bf16*)q, q_sb, q_st, (bf16*)k, k_sb, k_st, (const bf16*)v, v_sb, v_st, qw, kw,
                                                             norm_all, eps, inv_freq, dims, pos0, lens, slots, (bf16*)kcache, (bf16*)vcache,
                                                             ring, S, H, G, D, V);
    else
        window_qk_prepare_kernel<float><<<grid, block, 0, s>>>((float*)q, q_sb, q_st, (float*)k, k_sb, k_st, (const float*)v, v_sb, v_st, qw, kw,
                                                              norm_all, eps, inv_freq, dims, pos0, lens, slots, (float*)kcache,
                                                              (float*)vcache, ring, S, H, G, D, V);
}

static int value_cols_per_lane(int V) { return V <= 64 ? 2 : (V <= 128 ? 4 : (V <= 256 ? 8 : (V <= 512 ? 16 : 0))); }

template <typename K>
static bool raise_smem(K kernel, size_t smem) {
    if (smem <= 48 * 1024) return true;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
}

bool window_attention_prompt(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                             const void* gate, long g_sb, long g_st, int bf, const int* lens, int B, int S, int H, int G, int D, int V,
                             int window, float scale, float softcap, const float* score_bias, void* out, long out_stride, float out_scale,
                             cudaStream_t s) {
    const int vpl = value_cols_per_lane(V);
    if (!vpl) return false;
    if (B * S == 0) return true;
    if (bf && window_prompt_mma_fits(q, q_sb, q_st, k, k_sb, k_st, v, v_sb, v_st, D, V, out, out_stride)) {
        window_prompt_mma(q, q_sb, q_st, k, k_sb, k_st, v, v_sb, v_st, gate, g_sb, g_st, lens, B, S, H, G, D, V, window, scale, softcap,
                          score_bias, out, out_stride, out_scale, s);
        return true;
    }
    const size_t smem = sizeof(float) * ((size_t)kKeys * (D + 1) + (size_t)kKeys * V + (size_t)kWarps * D * kQW + kWarps * kKeys * kQW);
    dim3 grid((S + kWarps * kQW - 1) / (kWarps * kQW), H, B), block(128);
#define SEQMIX_WP(T, P)                                                                                                               \
    do {                                                                                                                              \
        if (!raise_smem(window_prompt_kernel<T, P>, smem)) return false;                                                              \
        window_prompt_kernel<T, P><<<grid, block, smem, s>>>((const T*)q, q_sb, q_st, (const T*)k, k_sb, k_st, (const T*)v, v_sb, v_st,   \
                                                             (const T*)gate, g_sb, g_st, lens, S, H, G, D, V, window, scale, softcap,   \
                                                             score_bias, (T*)out, out_stride, out_scale);                             \
    } while (0)
#define SEQMIX_WP_T(P) do { if (bf) SEQMIX_WP(bf16, P); else SEQMIX_WP(float, P); } while (0)
    if (vpl == 2) SEQMIX_WP_T(2); else if (vpl == 4) SEQMIX_WP_T(4); else if (vpl == 8) SEQMIX_WP_T(8); else SEQMIX_WP_T(16);
#undef SEQMIX_WP_T
#undef SEQMIX_WP
    return true;
}

int window_token_splits(int ring, int B, int H, int G) {
    const int quads = G * ((H / G + kWarps - 1) / kWarps);
    const int want = (2 * 148 + B * quads - 1) / (B * quads);       // two blocks per SM's worth of work items
    const int most = (ring + 4 * kKeys - 1) / (4 * kKeys);          // a split has at least 4 chunks
    return max(1, min(min(want, most), 64));
}

bool window_attention_token(const void* q, long q_sb, const void* kcache, const void* vcache, const void* gate, long g_sb, int bf,
                            const int* slots, const int* pos0, const int* lens, int ring, int B, int H, int G, int D, int V, int window,
                            float scale, float softcap, const float* score_bias, int splits, float* part_m, float* part_l, float* part_acc,
                            void* out, long out_stride, float out_scale, cudaStream_t s) {
    const int vpl = value_cols_per_lane(V);
    if (!vpl) return false;
    if (B == 0) return true;
    const size_t smem = sizeof(float) * ((size_t)kKeys * (D + 1) + (size_t)kKeys * V + (size_t)kWarps * D + kWarps * kKeys);
    const int quads = G * ((H / G + kWarps - 1) / kWarps), per16 = bf ? 8 : 4;
    const bool vec = D % per16 == 0 && V % per16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0;
    dim3 grid(splits, quads, B), block(128);
#define SEQMIX_WT(T, P, VC)                                                                                                           \
    do {                                                                                                                              \
        if (!raise_smem(window_token_kernel<T, P, VC>, smem)) return false;                                                           \
        window_token_kernel<T, P, VC><<<grid, block, smem, s>>>((const T*)q, q_sb, (const T*)kcache, (const T*)vcache, slots, pos0, lens, \
                                                                ring, H, G, D, V, window, scale, softcap, score_bias, splits, part_m,  \
                                                                part_l, part_acc);                                                    \
    } while (0)
#define SEQMIX_WT_V(T, P) do { if (vec) SEQMIX_WT(T, P, true); else SEQMIX_WT(T, P, false); } while (0)
#define SEQMIX_WT_T(P) do { if (bf) SEQMIX_WT_V(bf16, P); else SEQMIX_WT_V(float, P); } while (0)
    if (vpl == 2) SEQMIX_WT_T(2); else if (vpl == 4) SEQMIX_WT_T(4); else if (vpl == 8) SEQMIX_WT_T(8); else SEQMIX_WT_T(16);
#undef SEQMIX_WT_T
#undef SEQMIX_WT_V
#undef SEQMIX_WT
    dim3 mgrid(H, B);
    if (bf) window_token_merge_kernel<bf16><<<mgrid, 128, 0, s>>>(part_m, part_l, part_acc, (const bf16*)gate, g_sb, H, V, splits, (bf16*)out, out_stride, out_scale);
    else window_token_merge_kernel<float><<<mgrid, 128, 0, s>>>(part_m, part_l, part_acc, (const float*)gate, g_sb, H, V, splits, (float*)out, out_stride, out_scale);
    return true;
}

}  // namespace seqmix
