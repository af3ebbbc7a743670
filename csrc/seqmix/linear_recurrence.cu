// Gated linear recurrences carried from token to token, states in float.
//   gla_scan  : per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, with a decay per KEY channel
//               alpha = sigmoid(z + bias)^(1/tau) = exp(log_sigmoid(z + bias) / tau), formed here in float from the projected z;
//               with `decay` given (one number per head) alpha is that number for every token and channel (retention) and z is
//               not read.
//               A block owns one (sequence, head, slice of value columns); a thread owns DPT rows of one state column in registers;
//               the step's alpha / k / q / v are staged through shared memory (double buffered: one barrier per token).
//   rglru_scan: per channel  a = exp(-8 r softplus(lam)),  h_t = a h_(t-1) + sqrt(1 - a^2) i u_t,  out = h_t * gelu_tanh(y)
//               with r, i = sigmoid(gate pre-activations + bias); sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)).
// Tokens at or past lens[b] are padding: they write zeros and do not touch the state.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kStage = 28;  // staged loads per thread and barrier
constexpr int kSteps = 8;   // tokens staged per barrier

// Shared-memory image of one token: float4 {alpha, k, q, -} per key channel, then the slice's Vb values.
template <typename T, int DPT>
__global__ void gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long sb, long st,
                                const T* __restrict__ z, long z_sb, long z_st, const float* __restrict__ zbias, float inv_tau,
                                float qscale, const float* __restrict__ decay, float* state, const int* __restrict__ slots,
                                const int* __restrict__ lens, int fresh, int S, int H, int D, int V, int R, int Vb, int TB,
                                float* __restrict__ out) {
    extern __shared__ float4 sm4[];
    float* sm = reinterpret_cast<float*>(sm4);
    const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * Vb;
    const int tid = threadIdx.x, nthr = blockDim.x, r = tid % R, jl = tid / R, j = j0 + jl;
    const int len = min(lens[b], S), per = 4 * D + ((Vb + 3) & ~3), chunk = TB * per;
    const bool live = jl < Vb && j < V;
    float s[DPT];
    float* sp = state + (((long)slots[b] * H + h) * D) * V;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r + i * R;
        s[i] = (!fresh && live && d < D) ? sp[(long)d * V + j] : 0.f;
    }
    const long hq = (long)h * D, hv = (long)h * V + j0;
    // A chunk of TB tokens is fetched plane by plane (z, k, q: TB*D numbers each; v: TB*Vb), every load independent of the others and
    // free of branches, so that all of a thread's loads are in flight together; tokens past the end read the last real token's
    // numbers (never used).  The decays are formed when the chunk is written to shared memory.
    const int nD = (TB * D + nthr - 1) / nthr, nV = (TB * Vb + nthr - 1) / nthr;     // loads per thread and plane (host keeps 3 nD + nV <= kStage)
    const T* zp = z + (long)b * z_sb + hq;
    const T* kp = k + (long)b * sb + hq;
    const T* qp = q + (long)b * sb + hq;
    const T* vp = v + (long)b * sb + hv;
    float stage[kStage];
    auto load_chunk = [&](int t0) {
#pragma unroll
        for (int x = 0; x < kStage; ++x) {
            stage[x] = 0.f;
            if (x < 3 * nD) {
                const int pl = x / nD, idx = tid + (x - pl * nD) * nthr;
                const int u = idx / D, d = idx - u * D, t = min(t0 + u, len - 1);
                if (u < TB) stage[x] = pl == 0 ? (decay ? 0.f : ldf(zp + (long)t * z_st + d)) : ldf((pl == 1 ? kp : qp) + (long)t * st + d);
            } else if (x < 3 * nD + nV) {
                const int idx = tid + (x - 3 * nD) * nthr;
                const int u = idx / Vb, jj = idx - u * Vb, t = min(t0 + u, len - 1);
                if (u < TB && j0 + jj < V) stage[x] = ldf(vp + (long)t * st + jj);
            }
        }
    };
    auto store_chunk = [&](float* dst) {
#pragma unroll
        for (int x = 0; x < kStage; ++x) {
            if (x < 3 * nD) {
                const int pl = x / nD, idx = tid + (x - pl * nD) * nthr;
                const int u = idx / D, d = idx - u * D;
                if (u < TB) {
                    float val = stage[x];
                    if (pl == 0) val = decay ? decay[h] : 1.f + expm1f(log_sigmoidf_(val + zbias[hq + d]) * inv_tau);   // one rounding of an accurate value
                    else if (pl == 2) val *= qscale;
                    dst[u * per + 4 * d + pl] = val;
                }
            } else if (x < 3 * nD + nV) {
                const int idx = tid + (x - 3 * nD) * nthr;
                const int u = idx / Vb, jj = idx - u * Vb;
                if (u < TB) dst[u * per + 4 * D + jj] = stage[x];
            }
        }
    };
    const int nchunks = (len + TB - 1) / TB;
    if (nchunks > 0) { load_chunk(0); store_chunk(sm); }
    for (int c = 0; c < nchunks; ++c) {
        const float* cur = sm + (c & 1) * chunk;
        float* nxt = sm + ((c + 1) & 1) * chunk;
        __syncthreads();
        const bool more = c + 1 < nchunks;
        if (more) load_chunk((c + 1) * TB);
        const int steps = min(TB, len - c * TB);
        for (int u = 0; u < steps; ++u) {
            const float* tokp = cur + u * per;
            const float4* akq = reinterpret_cast<const float4*>(tokp);
            const float vj = live ? tokp[4 * D + jl] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int d = r + i * R;
                if (d < D) {
                    const float4 a = akq[d];
                    s[i] = fmaf(a.x, s[i], a.y * vj);
                    acc = fmaf(s[i], a.z, acc);
                }
            }
            for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (r == 0 && live) out[(((long)b * S + c * TB + u) * H + h) * V + j] = acc;
        }
        if (more) store_chunk(nxt);
    }
    if (r == 0 && live)
        for (int t = len; t < S; ++t) out[(((long)b * S + t) * H + h) * V + j] = 0.f;
    if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r + i * R;
            if (d < D) sp[(long)d * V + j] = s[i];
        }
    }
}

static int pow2ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

template <typename T>
static bool gla_launch(const void* q, const void* k, const void* v, long sb, long st, const void* z, long z_sb, long z_st,
                       const float* zbias, float inv_tau, float qscale, const float* decay, float* state, const int* slots,
                       const int* lens, int fresh, int B, int S, int H, int D, int V, float* out, cudaStream_t s) {
    // fewer, fatter blocks (more state rows per thread) as long as the grid still fills the GPU: the step's alpha / k / q are
    // prepared once per block, so every extra slice of value columns repeats that work
    const int dpts[3] = {32, 16, 8};
    int pick = -1, pR = 0, pVb = 0;
    for (int a = 0; a < 3; ++a) {
        const int DPT = dpts[a], R = pow2ceil((D + DPT - 1) / DPT);
        if (R > 32) continue;
        int Vb = 256 / R; if (Vb < 1) Vb = 1; if (Vb > V) Vb = V;
        const long blocks = (long)H * B * ((V + Vb - 1) / Vb);
        if (pick < 0 || blocks >= 148) { pick = DPT; pR = R; pVb = Vb; }
        if (blocks >= 148) break;
    }
    if (pick < 0) return false;
    const int R = pR, Vb = pVb;
    int threads = ((R * Vb + 31) / 32) * 32;
    const int per = 4 * D + ((Vb + 3) & ~3);
    int TB = S < kSteps ? (S < 1 ? 1 : S) : kSteps;
    auto fits = [&](int tb) {
        return 3 * ((tb * D + threads - 1) / threads) + (tb * Vb + threads - 1) / threads <= kStage && 2L * tb * per * 4 <= 96 * 1024;
    };
    while (TB > 1 && !fits(TB)) --TB;
    if (!fits(TB)) return false;
    dim3 grid(H, B, (V + Vb - 1) / Vb);
    const size_t smem = 2 * (size_t)TB * per * sizeof(float);
#define SEQMIX_GLA(P)                                                                                                             \
    do {                                                                                                                          \
        cudaFuncSetAttribute(gla_scan_kernel<T, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);                      \
        gla_scan_kernel<T, P><<<grid, threads, smem, s>>>((const T*)q, (const T*)k, (const T*)v, sb, st, (const T*)z, z_sb, z_st,    \
                                                          zbias, inv_tau, qscale, decay, state, slots, lens, fresh, S, H, D, V, R, Vb, TB, out); \
    } while (0)
    if (pick == 8) SEQMIX_GLA(8); else if (pick == 16) SEQMIX_GLA(16); else SEQMIX_GLA(32);
#undef SEQMIX_GLA
    return true;
}

bool gla_scan(const void* q, const void* k, const void* v, int bf, long sb, long st, const void* z, long z_sb, long z_st,
              const float* zbias, float inv_tau, float qscale, const float* decay, float* state, const int* slots, const int* lens,
              int fresh, int B, int S, int H, int D, int V, float* out, cudaStream_t s) {
    return bf ? gla_launch<bf16>(q, k, v, sb, st, z, z_sb, z_st, zbias, inv_tau, qscale, decay, state, slots, lens, fresh, B, S, H, D, V, out, s)
              : gla_launch<float>(q, k, v, sb, st, z, z_sb, z_st, zbias, inv_tau, qscale, decay, state, slots, lens, fresh, B, S, H, D, V, out, s);
}

// One new token per sequence (token generation): the step is bound by reading and writing the state once, so a block owns 64
// consecutive value columns of one (sequence, head) and all key channels; thread (column, group g of 4) walks the rows d = g, g+4, ...
// with whole 256-byte rows per access and eight independent rows in flight; the four groups' sums meet in shared memory.
constexpr int kStepCols = 64, kStepGroups = 4, kStepUnroll = 8;

template <typename T>
__global__ void __launch_bounds__(kStepCols* kStepGroups)
gla_step_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long sb, const T* __restrict__ z, long z_sb,
                const float* __restrict__ zbias, float inv_tau, float qscale, const float* __restrict__ decay, float* state,
                const int* __restrict__ slots, const int* __restrict__ lens, int fresh, int H, int D, int V, float* __restrict__ out) {
    extern __shared__ float sm[];              // alpha [D], k [D], q [D], sums [groups][cols]
    float *sa = sm, *sk = sm + D, *sq = sm + 2 * D, *red = sm + 3 * D;
    const int h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, jl = tid % kStepCols, g = tid / kStepCols;
    const int j = blockIdx.x * kStepCols + jl;
    const bool live = j < V;
    float* o = out + ((long)b * H + h) * V + j;
    if (lens[b] < 1) {                          // a padded row: zeros out, state untouched
        if (g == 0 && live) *o = 0.f;
        return;
    }
    const long hq = (long)h * D;
    for (int d = tid; d < D; d += kStepCols * kStepGroups) {
        sa[d] = decay ? decay[h] : 1.f + expm1f(log_sigmoidf_(ldf(z + (long)b * z_sb + hq + d) + zbias[hq + d]) * inv_tau);
        sk[d] = ldf(k + (long)b * sb + hq + d);
        sq[d] = ldf(q + (long)b * sb + hq + d) * qscale;
    }
    __syncthreads();
    const float vj = live ? ldf(v + (long)b * sb + (long)h * V + j) : 0.f;
    float* sp = state + (((long)slots[b] * H + h) * D) * V + j;
    float acc = 0.f;
    for (int d0 = g; d0 < D; d0 += kStepGroups * kStepUnroll) {
        float s[kStepUnroll];
#pragma unroll
        for (int u = 0; u < kStepUnroll; ++u) {
            const int d = d0 + u * kStepGroups;
            s[u] = (!fresh && live && d < D) ? sp[(long)d * V] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < kStepUnroll; ++u) {
            const int d = d0 + u * kStepGroups;
            if (d < D) {
                s[u] = fmaf(sa[d], s[u], sk[d] * vj);
                acc = fmaf(s[u], sq[d], acc);
                if (live) sp[(long)d * V] = s[u];
            }
        }
    }
    red[g * kStepCols + jl] = acc;
    __syncthreads();
    if (g == 0 && live) {
        float t = 0.f;
#pragma unroll
        for (int x = 0; x < kStepGroups; ++x) t += red[x * kStepCols + jl];
        *o = t;
    }
}

template <typename T>
static void gla_step_launch(const void* q, const void* k, const void* v, long sb, const void* z, long z_sb, const float* zbias,
                            float inv_tau, float qscale, const float* decay, float* state, const int* slots, const int* lens, int fresh, int B, int H, int D,
                            int V, float* out, cudaStream_t s) {
    dim3 grid((V + kStepCols - 1) / kStepCols, H, B);
    const size_t smem = (size_t)(3 * D + kStepGroups * kStepCols) * sizeof(float);
    gla_step_kernel<T><<<grid, kStepCols * kStepGroups, smem, s>>>((const T*)q, (const T*)k, (const T*)v, sb, (const T*)z, z_sb, zbias, inv_tau,
                                                                  qscale, decay, state, slots, lens, fresh, H, D, V, out);
}

bool gla_step(const void* q, const void* k, const void* v, int bf, long sb, const void* z, long z_sb, const float* zbias, float inv_tau,
              float qscale, const float* decay, float* state, const int* slots, const int* lens, int fresh, int B, int H, int D, int V, float* out,
              cudaStream_t s) {
    if ((size_t)(3 * D + kStepGroups * kStepCols) * sizeof(float) > 48 * 1024) return false;
    if (bf) gla_step_launch<bf16>(q, k, v, sb, z, z_sb, zbias, inv_tau, qscale, decay, state, slots, lens, fresh, B, H, D, V, out, s);
    else gla_step_launch<float>(q, k, v, sb, z, z_sb, zbias, inv_tau, qscale, decay, state, slots, lens, fresh, B, H, D, V, out, s);
    return true;
}

// One block = 32 channels of one sequence x TY time lanes.  Each lane scans its slice of the tokens from zero keeping the product of
// its decays; the carries are folded through shared memory; the lanes scan again from their true carry and write the outputs.
template <typename T>
__global__ void rglru_scan_kernel(const T* __restrict__ u, const float* __restrict__ gr, const float* __restrict__ gi, int wb,
                                  const float* __restrict__ rbias, const float* __restrict__ ibias, const float* __restrict__ lam_sp,
                                  const T* __restrict__ y, long y_sb, long y_st, float* state, const int* __restrict__ slots,
                                  const int* __restrict__ lens, int fresh, int B, int S, int W, T* __restrict__ out) {
    __shared__ float sA[32][33], sH[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x, b = blockIdx.y, ty = threadIdx.y, TY = blockDim.y;
    const int len = min(lens[b], S);
    const int L = (len + TY - 1) / TY, t0 = min(len, ty * L), t1 = min(len, t0 + L);
    const bool on = c < W;
    const long N = (long)B * S;
    const long gbase = on ? ((long)(c / wb) * N + (long)b * S) * wb + c % wb : 0;   // gates: [block, token, channel in block]
    const float rb = on ? rbias[c] : 0.f, ib = on ? ibias[c] : 0.f, sp = on ? lam_sp[c] : 0.f;
    float A = 1.f, h = 0.f;
    if (on && TY > 1) {
#pragma unroll 4
        for (int t = t0; t < t1; ++t) {
            const float r = sigmoidf_(gr[gbase + (long)t * wb] + rb), g = sigmoidf_(gi[gbase + (long)t * wb] + ib);
            const float la = -8.f * r * sp, a = 1.f + expm1f(la), mult = sqrtf(-expm1f(2.f * la));
            h = fmaf(a, h, mult * g * ldf(u + ((long)b * S + t) * W + c));
            A *= a;
        }
    }
    sA[ty][threadIdx.x] = A;
    sH[ty][threadIdx.x] = h;
    __syncthreads();
    if (!on) return;
    float* hs = state + (long)slots[b] * W + c;
    h = fresh ? 0.f : *hs;
    for (int k = 0; k < ty; ++k) h = fmaf(sA[k][threadIdx.x], h, sH[k][threadIdx.x]);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const float r = sigmoidf_(gr[gbase + (long)t * wb] + rb), g = sigmoidf_(gi[gbase + (long)t * wb] + ib);
        const float uu = ldf(u + ((long)b * S + t) * W + c), yy = ldf(y + (long)b * y_sb + (long)t * y_st + c);
        const float la = -8.f * r * sp, a = 1.f + expm1f(la), mult = sqrtf(-expm1f(2.f * la));
        h = fmaf(a, h, mult * g * uu);
        const float gl = 0.5f * yy * (1.f + tanhf(0.7978845608028654f * (yy + 0.044715f * yy * yy * yy)));
        stf(out + ((long)b * S + t) * W + c, h * gl);
    }
    for (int t = len + ty; t < S; t += TY) stf(out + ((long)b * S + t) * W + c, 0.f);
    if (ty == TY - 1) *hs = h;      // the last lane's slice ends at the sequence's last token (an empty slice passes the carry on)
}

void rglru_scan(const void* u, int bf, const float* gr, const float* gi, int wb, const float* rbias, const float* ibias,
                const float* lam_sp, const void* y, long y_sb, long y_st, float* state, const int* slots, const int* lens, int fresh,
                int B, int S, int W, void* out, cudaStream_t s) {
    int ty = 1;
    while (ty < 32 && ty * 16 < S) ty <<= 1;
    dim3 block(32, ty), grid((W + 31) / 32, B);
    if (bf) rglru_scan_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)u, gr, gi, wb, rbias, ibias, lam_sp, (const bf16*)y, y_sb, y_st,
                                                          state, slots, lens, fresh, B, S, W, (bf16*)out);
    else rglru_scan_kernel<float><<<grid, block, 0, s>>>((const float*)u, gr, gi, wb, rbias, ibias, lam_sp, (const float*)y, y_sb, y_st,
                                                         state, slots, lens, fresh, B, S, W, (float*)out);
}

}  // namespace seqmix
