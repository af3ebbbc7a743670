// Gated linear attention over a long run of tokens, in chunks of kC tokens, so that the work is matrix products instead of a token by
// token scan.  With b_t[d] = sum of log2(alpha_s[d]) over the chunk's tokens s <= t (all <= 0), and S_in the state before the chunk,
//   o_t   = (q_t * 2^b_t)^T S_in  +  sum_{s <= t} A[t,s] v_s,     A[t,s] = sum_d q_t[d] k_s[d] 2^(b_t[d] - b_s[d]),
//   S_out = diag(2^b_last) S_in   +  sum_s (k_s * 2^(b_last - b_s)) v_s^T.
// Every exponent is <= 0, so nothing overflows whatever the decays are.  Three kernels here; the matrix products between them are
// float library products issued by the binding:
//   gla_chunk_prep : cumulative log-decays per chunk, the scaled queries / keys, the chunk's total decay, the values as float
//   gla_intra      : A, pair by pair (the decay couples t, s and d, so this part is not a matrix product)
//   gla_carry      : the chunks' local state sums are turned, in sequence, into the state before each chunk; the last one is the
//                    sequence's new state
// Tokens at or past lens[b] neither change the state nor produce output (their rows of the scaled queries, keys and A are zero).
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kC = 64;                                // tokens per chunk (gla_chunk_tokens() tells the binding)
constexpr float kLog2e = 1.4426950408889634f;

int gla_chunk_tokens() { return kC; }

// grid (chunks, H, B).  Qe, Ke, Bc [blk, kC, D]; G [blk, D]; Vf [blk, kC, V] with blk = (b * H + h) * chunks + c.
template <typename T>
__global__ void gla_chunk_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long sb, long st,
                                      const T* __restrict__ z, long z_sb, long z_st, const float* __restrict__ zbias, float inv_tau2,
                                      float qscale, const float* __restrict__ decay, const int* __restrict__ lens, int S, int H, int D, int V,
                                      float* __restrict__ Qe, float* __restrict__ Ke, float* __restrict__ Bc, float* __restrict__ G,
                                      float* __restrict__ Vf) {
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, nC = gridDim.x;
    const int len = min(lens[b], S), t0 = c * kC, n = max(0, min(kC, len - t0));
    const long blk = ((long)b * H + h) * nC + c;
    float* qe = Qe + blk * kC * D;
    float* ke = Ke + blk * kC * D;
    float* bc = Bc + blk * kC * D;
    const float fixed = decay ? log2f(decay[h]) : 0.f;     // a fixed decay per head: the same log-decay for every token and channel
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float zb = decay ? 0.f : zbias[h * D + d];
        const T* zp = z + (long)b * z_sb + (long)t0 * z_st + h * D + d;
        const T* qp = q + (long)b * sb + (long)t0 * st + h * D + d;
        const T* kp = k + (long)b * sb + (long)t0 * st + h * D + d;
        float cum = 0.f;
#pragma unroll 8
        for (int t = 0; t < kC; ++t) {
            float qv = 0.f;
            if (t < n) {
                cum += decay ? fixed : log_sigmoidf_(ldf(zp + (long)t * z_st) + zb) * inv_tau2;
                qv = ldf(qp + (long)t * st) * qscale * exp2f(cum);
            }
            bc[t * D + d] = cum;
            qe[t * D + d] = qv;
        }
        G[blk * D + d] = exp2f(cum);
#pragma unroll 8
        for (int t = 0; t < kC; ++t) ke[t * D + d] = t < n ? ldf(kp + (long)t * st) * exp2f(cum - bc[t * D + d]) : 0.f;
    }
    float* vf = Vf + blk * kC * V;
    const T* vp = v + (long)b * sb + (long)t0 * st + (long)h * V;
    for (int i = threadIdx.x; i < kC * V; i += blockDim.x) {
        const int t = i / V, j = i - t * V;
        vf[i] = t < n ? ldf(vp + (long)t * st + j) : 0.f;
    }
}

// grid (chunks, H, B), 256 threads: thread (t = tid / 4, g = tid % 4) owns A[t, 4 i + g], i < 16.  q, k and the cumulative log-decays
// pass through shared memory 32 key channels at a time.
template <typename T>
__global__ void gla_intra_kernel(const T* __restrict__ q, const T* __restrict__ k, long sb, long st, const float* __restrict__ Bc,
                                 float qscale, const int* __restrict__ lens, int S, int H, int D, float* __restrict__ A) {
    __shared__ float qs[kC][33], ks[kC][33], bs[kC][33];
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, nC = gridDim.x, tid = threadIdx.x;
    const int len = min(lens[b], S), t0 = c * kC, n = max(0, min(kC, len - t0));
    const long blk = ((long)b * H + h) * nC + c;
    const float* bc = Bc + blk * kC * D;
    const int t = tid >> 2, g = tid & 3;
    const int imax = min(16, (((tid >> 5) * 8 + 7) >> 2) + 1);        // same for the whole warp: keys past its last row are skipped
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int d0 = 0; d0 < D; d0 += 32) {
        for (int i = tid; i < kC * 32; i += blockDim.x) {
            const int tt = i >> 5, dd = i & 31, d = d0 + dd;
            const bool ok = d < D && tt < n;
            const long tok = (long)b * sb + (long)(t0 + tt) * st + h * D + d;
            qs[tt][dd] = ok ? ldf(q + tok) * qscale : 0.f;
            ks[tt][dd] = ok ? ldf(k + tok) : 0.f;
            bs[tt][dd] = d < D ? bc[tt * D + d] : 0.f;
        }
        __syncthreads();
        const int dn = min(32, D - d0);
        for (int dd = 0; dd < dn; ++dd) {
            const float qt = qs[t][dd], bt = bs[t][dd];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (i < imax) {
                    const int s = 4 * i + g;
                    if (s <= t) acc[i] = fmaf(qt * ks[s][dd], exp2f(bt - bs[s][dd]), acc[i]);
                }
            }
        }
        __syncthreads();
    }
    float* a = A + (blk * kC + t) * kC;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int s = 4 * i + g;
        a[s] = (s <= t && t < n) ? acc[i] : 0.f;
    }
}

// grid (ceil(D V / 256), H, B).  Sl [blk, D, V] holds each chunk's own sum of k v^T on entry and the state BEFORE the chunk on exit.
__global__ void gla_carry_kernel(float* __restrict__ Sl, const float* __restrict__ G, float* __restrict__ state,
                                 const int* __restrict__ slots, int fresh, int nC, int H, int D, int V) {
    const long e = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (long)D * V) return;
    const int h = blockIdx.y, b = blockIdx.z, d = (int)(e / V);
    const long bh = (long)b * H + h;
    float* sp = state + ((long)slots[b] * H + h) * D * V + e;
    float run = fresh ? 0.f : *sp;
    constexpr int kU = 8;                                      // chunks whose loads are in flight together
    for (int c0 = 0; c0 < nC; c0 += kU) {
        float loc[kU], gg[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int c = min(c0 + u, nC - 1);
            loc[u] = __ldcs(Sl + (bh * nC + c) * D * V + e);
            gg[u] = G[(bh * nC + c) * D + d];
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            if (c0 + u < nC) {
                __stcs(Sl + (bh * nC + c0 + u) * D * V + e, run);
                run = fmaf(gg[u], run, loc[u]);
            }
        }
    }
    *sp = run;
}

void gla_chunk_prep(const void* q, const void* k, const void* v, int bf, long sb, long st, const void* z, long z_sb, long z_st,
                    const float* zbias, float inv_tau, float qscale, const float* decay, const int* lens, int B, int S, int H, int D, int V,
                    int chunks, float* Qe, float* Ke, float* Bc, float* G, float* Vf, float* A, cudaStream_t s) {
    dim3 grid(chunks, H, B);
    const int threads = D >= 256 ? 256 : (D > 64 ? 128 : 64);
    const float inv_tau2 = inv_tau * kLog2e;
    if (bf) {
        gla_chunk_prep_kernel<bf16><<<grid, threads, 0, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, sb, st, (const bf16*)z, z_sb,
                                                            z_st, zbias, inv_tau2, qscale, decay, lens, S, H, D, V, Qe, Ke, Bc, G, Vf);
        gla_intra_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)q, (const bf16*)k, sb, st, Bc, qscale, lens, S, H, D, A);
    } else {
        gla_chunk_prep_kernel<float><<<grid, threads, 0, s>>>((const float*)q, (const float*)k, (const float*)v, sb, st, (const float*)z,
                                                             z_sb, z_st, zbias, inv_tau2, qscale, decay, lens, S, H, D, V, Qe, Ke, Bc, G, Vf);
        gla_intra_kernel<float><<<grid, 256, 0, s>>>((const float*)q, (const float*)k, sb, st, Bc, qscale, lens, S, H, D, A);
    }
}

void gla_carry(float* Sl, const float* G, float* state, const int* slots, int fresh, int B, int chunks, int H, int D, int V,
               cudaStream_t s) {
    dim3 grid((unsigned)(((long)D * V + 255) / 256), H, B);
    gla_carry_kernel<<<grid, 256, 0, s>>>(Sl, G, state, slots, fresh, chunks, H, D, V);
}

}  // namespace seqmix
