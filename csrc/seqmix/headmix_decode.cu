// Head-mixing attention for single tokens against the key / value rings (see headmix_attention.cu for the formulation: the queries
// arrive mixed, Q' [B,1,H,DK] with DK = G*D, and every head reads the SAME key rows, all key heads side by side).
//
// Two kernels.  headmix_token_kernel: a block per (stretch of 32 visible positions, sequence) serves ALL heads, so a key row is
// read from memory once and not once per head.  A warp holds one key row in registers (lane = 4 consecutive numbers per 128) and
// forms its dot product with every head's mixed query from shared memory; the stretch's scores [H][32] stay in shared memory, a warp
// per head turns them into weights exp(s - m) with the stretch's maximum m and sum l, and the threads then spread over (head, value
// coordinate) for the weighted sum of the stretch's value rows.  Each stretch leaves (m, l, sum) per head.
// headmix_token_merge_kernel: a block per (head, sequence) joins the stretches; exp(sink_h) enters the denominator here; the result
// times sigmoid(gate) is written.  Everything between the loads and the store is float.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kTokKeys = 32, kTokWarps = 8;

__device__ __forceinline__ int visible_from(int i, int chunk, int window) {
    int lo = 0;
    if (chunk > 0) lo = (i / chunk) * chunk;
    if (window > 0) lo = max(lo, i - window + 1);
    return lo;
}

// grid (stretches, B), 256 threads.  part [B, stretches, H, D + 2]: D sums, then m, then l.
template <typename T, int NCH>
__global__ void __launch_bounds__(32 * kTokWarps) headmix_token_kernel(
    const T* __restrict__ qmix, const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ slots,
    const int* __restrict__ pos0, const int* __restrict__ lens, int chunk, int window, int ring, int H, int G, int D,
    float* __restrict__ part) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int DK = G * D, b = blockIdx.y, st = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    if (lens[b] <= 0) return;
    const int i = pos0[b], lo = visible_from(i, chunk, window);
    const int j0 = lo + st * kTokKeys;
    if (j0 > i) return;                                    // past the query: no such stretch for this row
    const int nk = min(kTokKeys, i - j0 + 1);
    T* qs = reinterpret_cast<T*>(smem_raw);                                                 // [H][DK]
    float* sc = reinterpret_cast<float*>(smem_raw + (((size_t)H * DK * sizeof(T) + 15) / 16) * 16);   // [H][kTokKeys]
    long* rowoff = reinterpret_cast<long*>(sc + H * kTokKeys);                              // [kTokKeys] element offsets of the ring rows
    const T* qr = qmix + (long)b * H * DK;
    for (int x = tid * 4; x < H * DK; x += 32 * kTokWarps * 4) st4(qs + x, ld4(qr + x));
    __syncthreads();
    const long base = (long)slots[b] * ring;
    if (tid < kTokKeys) rowoff[tid] = (base + (j0 + min(tid, nk - 1)) % ring) * DK;
    __syncthreads();
    // scores: a key row per warp at a time, the next row fetched while this one meets the heads
    float4 kv[NCH], kn[NCH];
    auto fetch = [&](int j, float4* dst) {
        const T* kr = kcache + rowoff[j];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int x = (c * 32 + lane) * 4;
            dst[c] = x < DK ? ld4(kr + x) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    if (w < nk) fetch(w, kn);
    for (int j = w; j < nk; j += kTokWarps) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) kv[c] = kn[c];
        if (j + kTokWarps < nk) fetch(j + kTokWarps, kn);
        for (int h = 0; h < H; ++h) {
            const T* qh = qs + h * DK;
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int x = (c * 32 + lane) * 4;
                if (x < DK) {
                    const float4 qv = ld4(qh + x);
                    s = fmaf(qv.x, kv[c].x, s); s = fmaf(qv.y, kv[c].y, s); s = fmaf(qv.z, kv[c].z, s); s = fmaf(qv.w, kv[c].w, s);
                }
            }
            s = warp_sum(s);
            if (lane == 0) sc[h * kTokKeys + j] = s;
        }
    }
    __syncthreads();
    // weights: a head per warp at a time, a key per lane
    float* pb = part + ((long)b * gridDim.x + st) * H * (D + 2);
    for (int h = w; h < H; h += kTokWarps) {
        const float s = lane < nk ? sc[h * kTokKeys + lane] : -INFINITY;
        float m = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float p = lane < nk ? expf(s - m) : 0.f;
        const float l = warp_sum(p);
        sc[h * kTokKeys + lane] = p;
        if (lane == 0) { pb[h * (D + 2) + D] = m; pb[h * (D + 2) + D + 1] = l; }
    }
    __syncthreads();
    // weighted sums of the value rows: threads over (head, four coordinates) when the head size is in whole fours
    const int hpg = H / G;
    if (D % 4 == 0) {
        const int d4 = D / 4;
        for (int x = tid; x < H * d4; x += 32 * kTokWarps) {
            const int h = x / d4, d = (x - h * d4) * 4;
            const T* vb = vcache + (long)(h / hpg) * D + d;
            const float* ph = sc + h * kTokKeys;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int j = 0; j < nk; ++j) {
                const float4 v = ld4(vb + rowoff[j]);
                const float pj = ph[j];
                acc.x = fmaf(pj, v.x, acc.x); acc.y = fmaf(pj, v.y, acc.y); acc.z = fmaf(pj, v.z, acc.z); acc.w = fmaf(pj, v.w, acc.w);
            }
            float* po = pb + h * (D + 2) + d;
            po[0] = acc.x; po[1] = acc.y; po[2] = acc.z; po[3] = acc.w;
        }
        return;
    }
    for (int x = tid; x < H * D; x += 32 * kTokWarps) {
        const int h = x / D, d = x - h * D;
        const T* vb = vcache + (long)(h / hpg) * D + d;
        const float* ph = sc + h * kTokKeys;
        float acc = 0.f;
        for (int j = 0; j < nk; ++j) acc = fmaf(ph[j], ldf(vb + rowoff[j]), acc);
        pb[h * (D + 2) + d] = acc;
    }
}

// grid (H, B), 128 threads
template <typename T>
__global__ void __launch_bounds__(128) headmix_token_merge_kernel(
    const float* __restrict__ part, int stretches, const float* __restrict__ sink, const T* __restrict__ gate, long g_sb,
    const int* __restrict__ pos0, const int* __restrict__ lens, int chunk, int window, int H, int D, T* __restrict__ out, long out_stride) {
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    T* o = out + (long)b * out_stride + (long)h * D;
    if (lens[b] <= 0) {
        for (int d = tid; d < D; d += 128) stf(o + d, 0.f);
        return;
    }
    const int i = pos0[b], lo = visible_from(i, chunk, window);
    const int nst = min(stretches, (i - lo) / kTokKeys + 1);
    const float* pb = part + ((long)b * stretches * H + h) * (D + 2);
    const long step = (long)H * (D + 2);
    extern __shared__ float fs[];                  // [stretches] exp(m_s - M), then [1] the denominator
    float M = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < nst; ++s) M = fmaxf(M, pb[s * step + D]);
    for (int s = tid; s < nst; s += 128) fs[s] = expf(pb[s * step + D] - M);
    __syncthreads();
    if (tid == 0) {
        float L = sink ? expf(sink[h] - M) : 0.f;
        for (int s = 0; s < nst; ++s) L = fmaf(pb[s * step + D + 1], fs[s], L);
        fs[stretches] = L;
    }
    __syncthreads();
    const float L = fs[stretches];
    const T* gr = gate ? gate + (long)b * g_sb + (long)h * D : nullptr;
    for (int d = tid; d < D; d += 128) {
        float v = 0.f;
        for (int s = 0; s < nst; ++s) v = fmaf(pb[s * step + d], fs[s], v);
        v /= L;
        if (gr) v *= sigmoidf_(ldf(gr + d));
        stf(o + d, v);
    }
}

int headmix_token_stretches(int ring) { return (ring + kTokKeys - 1) / kTokKeys; }

static size_t token_smem(int H, int DK, size_t elem) {
    return (((size_t)H * DK * elem + 15) / 16) * 16 + (size_t)H * kTokKeys * sizeof(float) + kTokKeys * sizeof(long);
}

bool headmix_token_fits(int bf, int H, int G, int D, int ring, const void* qmix, const void* kcache, const void* vcache) {
    const int DK = G * D;
    auto a16 = [](const void* p) { return (uintptr_t)p % 16 == 0; };
    return DK % 4 == 0 && DK <= 16 * 128 && headmix_token_stretches(ring) <= 4096 && a16(qmix) && a16(kcache) && a16(vcache) && token_smem(H, DK, bf ? 2 : 4) <= 200 * 1024;
}

template <typename T>
static void token_launch(const void* qmix, const void* kcache, const void* vcache, const float* sink, const void* gate, long g_sb,
                         const int* slots, const int* pos0, const int* lens, int chunk, int window, int ring, int B, int H, int G, int D,
                         float* part, void* out, long out_stride, cudaStream_t s) {
    const int DK = G * D, nst = headmix_token_stretches(ring);
    const size_t smem = token_smem(H, DK, sizeof(T));
    dim3 grid(nst, B);
#define SEQMIX_HTK(NCH)                                                                                                              \
    do {                                                                                                                             \
        cudaFuncSetAttribute(headmix_token_kernel<T, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);                 \
        headmix_token_kernel<T, NCH><<<grid, 32 * kTokWarps, smem, s>>>((const T*)qmix, (const T*)kcache, (const T*)vcache, slots, pos0, \
                                                                        lens, chunk, window, ring, H, G, D, part);                   \
    } while (0)
    if (DK <= 128) SEQMIX_HTK(1);
    else if (DK <= 256) SEQMIX_HTK(2);
    else if (DK <= 512) SEQMIX_HTK(4);
    else if (DK <= 1024) SEQMIX_HTK(8);
    else SEQMIX_HTK(16);
#undef SEQMIX_HTK
    headmix_token_merge_kernel<T><<<dim3(H, B), 128, (nst + 1) * sizeof(float), s>>>(part, nst, sink, (const T*)gate, g_sb, pos0, lens, chunk, window, H, D, (T*)out,
                                                             out_stride);
}

void headmix_token(const void* qmix, const void* kcache, const void* vcache, int bf, const float* sink, const void* gate, long g_sb,
                   const int* slots, const int* pos0, const int* lens, int chunk, int window, int ring, int B, int H, int G, int D,
                   float* part, void* out, long out_stride, cudaStream_t s) {
    if (B == 0) return;
    if (bf) token_launch<bf16>(qmix, kcache, vcache, sink, gate, g_sb, slots, pos0, lens, chunk, window, ring, B, H, G, D, part, out, out_stride, s);
    else token_launch<float>(qmix, kcache, vcache, sink, gate, g_sb, slots, pos0, lens, chunk, window, ring, B, H, G, D, part, out, out_stride, s);
}

}  // namespace seqmix
