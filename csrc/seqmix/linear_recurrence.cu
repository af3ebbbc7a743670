// Gated linear recurrences carried from token to token, states in float.
//   gla_scan  : per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, with a decay per KEY channel
//               alpha = sigmoid(z + bias)^(1/tau) = exp(log_sigmoid(z + bias) / tau), formed here in float from the projected z;
//               with `decay` given (one number per head) alpha is that number for every token and channel (retention) and z is
//               not read.
//               A block owns one (sequence, head, slice of value columns); a thread owns DPT rows of one state column in registers;
//               the step's alpha / k / q / v are staged through shared memory (double buffered: one barrier per token).
//   rglru_scan: per channel  a = exp(-8 r softplus(lam)),  h_t = a h_(t-1) + sqrt(1 - a^2) i u_t,  out = h_t * gelu_tanh(y)
//               with r, i = sigmoid(gate pre-activations + bias); sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)).
//   mingru_scan: per channel h_t = (1 - z) h_(t-1) + z c with z = sigmoid(zraw) and the candidate c = uraw + 1/2 (uraw >= 0) or
//               sigmoid(uraw) (below), out = h_t * silu(graw)
// Tokens at or past lens[b] are padding: they write zeros and do not touch the state.
#include <cooperative_groups.h>

#include "seq_common.cuh"
#include "seqmix.h"

namespace cg = cooperative_groups;

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

// minGRU: per channel h_t = (1 - z_t) h_(t-1) + z_t c_t with z = sigmoid(zraw), c = uraw + 1/2 where uraw >= 0 and sigmoid(uraw) below,
// out_t = h_t * silu(graw_t); the gates read only the current token, so the same two-pass scan as the real-gated LRU applies: each
// time lane scans its slice from zero keeping the product of its (1 - z), the carries are folded through shared memory, the lanes
// scan again from their true carry.  One block = 32 * CPT channels of one sequence x TY time lanes; gates, candidate and state in
// float.  sigmoid(z) and 1 - sigmoid(z) = sigmoid(-z) come from ONE exponential of -|z| and one reciprocal, both exact to rounding.
// FAST (the bfloat16 instantiation, whose inputs carry 8 bits): the exponential and the reciprocal are the hardware approximations
// (relative error about 1e-6, far below the inputs' rounding); the float instantiation uses the exact-rounded library functions.
// CPT = 2: a thread owns two neighbouring channels and reads them as one 4-byte pair.
template <bool FAST> __device__ __forceinline__ float exp_neg_(float x) { return FAST ? __expf(x) : expf(x); }
template <bool FAST> __device__ __forceinline__ float rcp1p_(float e) { return FAST ? __fdividef(1.f, 1.f + e) : 1.f / (1.f + e); }
template <bool FAST> __device__ __forceinline__ void sigmoid_pair_(float z, float& s, float& a) {       // s = sigmoid(z), a = sigmoid(-z)
    const float e = exp_neg_<FAST>(-fabsf(z)), r = rcp1p_<FAST>(e), er = e * r;
    s = z >= 0.f ? r : er;
    a = z >= 0.f ? er : r;
}
template <bool FAST> __device__ __forceinline__ float mingru_candidate_(float u) {
    const float e = exp_neg_<FAST>(fminf(u, 0.f));
    return u >= 0.f ? u + 0.5f : e * rcp1p_<FAST>(e);
}
template <int CPT, typename T> __device__ __forceinline__ void ld_ch(const T* p, float (&v)[CPT]) {
    if (CPT == 1) v[0] = ldf(p);
    else {
        const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p);      // CPT == 2 is only instantiated for bfloat16
        v[0] = __low2float(t); v[CPT - 1] = __high2float(t);
    }
}
template <int CPT, typename T> __device__ __forceinline__ void st_ch(T* p, const float (&v)[CPT]) {
    if (CPT == 1) stf(p, v[0]);
    else *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[CPT - 1]);
}

// CL: the time lanes of a sequence's channels are blockDim.y lanes in each of gridDim.z blocks that form ONE thread-block cluster
// (so that a long prompt of few sequences still fills the GPU): every block folds its lanes' carries into one pair per channel, the
// blocks read the pairs of the blocks before them through distributed shared memory.  Every thread reaches both cluster barriers.
template <typename T, int CPT, bool FAST, bool CL>
__global__ void __launch_bounds__(1024, 2) mingru_scan_kernel(const T* __restrict__ z, const T* __restrict__ u, const T* __restrict__ g, long sb, long st,
                                   float* state, const int* __restrict__ slots, const int* __restrict__ lens, int fresh, int S, int W,
                                   T* __restrict__ out) {
    __shared__ float sA[CPT][32][33], sH[CPT][32][33], cA[CPT][32], cH[CPT][32];
    const int c = (blockIdx.x * 32 + threadIdx.x) * CPT, b = blockIdx.y, ty = threadIdx.y, TY = blockDim.y;
    const int cz = CL ? blockIdx.z : 0, lanes = CL ? TY * gridDim.z : TY, gl = cz * TY + ty;   // the cluster spans the grid's z extent
    const int len = min(lens[b], S);
    const int L = (len + lanes - 1) / lanes, t0 = min(len, gl * L), t1 = min(len, t0 + L);
    const bool on = c < W;                                   // W is a multiple of CPT: a thread's channels are all in or all out
    const long base = (long)b * sb + c;
    float A[CPT], h[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k) { A[k] = 1.f; h[k] = 0.f; }
    if (on && lanes > 1) {
#pragma unroll 4
        for (int t = t0; t < t1; ++t) {
            float zr[CPT], ur[CPT];
            ld_ch<CPT>(z + base + (long)t * st, zr);
            ld_ch<CPT>(u + base + (long)t * st, ur);
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                float sg, a;
                sigmoid_pair_<FAST>(zr[k], sg, a);
                h[k] = fmaf(a, h[k], sg * mingru_candidate_<FAST>(ur[k]));
                A[k] *= a;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CPT; ++k) { sA[k][ty][threadIdx.x] = A[k]; sH[k][ty][threadIdx.x] = h[k]; }
    __syncthreads();
    if (CL && ty == TY - 1) {                                // this block's lanes as one pair per channel
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            float a = 1.f, x = 0.f;
            for (int j = 0; j < TY; ++j) { x = fmaf(sA[k][j][threadIdx.x], x, sH[k][j][threadIdx.x]); a *= sA[k][j][threadIdx.x]; }
            cA[k][threadIdx.x] = a; cH[k][threadIdx.x] = x;
        }
    }
    if (CL) cg::this_cluster().sync();
    float* hs = state + (long)(on ? slots[b] : 0) * W + (on ? c : 0);
    if (on) {
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            h[k] = fresh ? 0.f : hs[k];
            if (CL) {
                cg::cluster_group cluster = cg::this_cluster();
                for (int r = 0; r < cz; ++r) {
                    const float* ra = cluster.map_shared_rank(&cA[k][threadIdx.x], r);
                    const float* rh = cluster.map_shared_rank(&cH[k][threadIdx.x], r);
                    h[k] = fmaf(*ra, h[k], *rh);
                }
            }
            for (int j = 0; j < ty; ++j) h[k] = fmaf(sA[k][j][threadIdx.x], h[k], sH[k][j][threadIdx.x]);
        }
#pragma unroll 4
        for (int t = t0; t < t1; ++t) {
            float zr[CPT], ur[CPT], gr[CPT], o[CPT];
            ld_ch<CPT>(z + base + (long)t * st, zr);
            ld_ch<CPT>(u + base + (long)t * st, ur);
            ld_ch<CPT>(g + base + (long)t * st, gr);
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                float sg, a, gs, gn;
                sigmoid_pair_<FAST>(zr[k], sg, a);
                h[k] = fmaf(a, h[k], sg * mingru_candidate_<FAST>(ur[k]));
                sigmoid_pair_<FAST>(gr[k], gs, gn);
                o[k] = h[k] * gr[k] * gs;
            }
            st_ch<CPT>(out + ((long)b * S + t) * W + c, o);
        }
        float zero[CPT];
#pragma unroll
        for (int k = 0; k < CPT; ++k) zero[k] = 0.f;
        for (int t = len + gl; t < S; t += lanes) st_ch<CPT>(out + ((long)b * S + t) * W + c, zero);
    }
    if (CL) cg::this_cluster().sync();   // no block leaves while another may still read its pairs; the state's old value has been read
    if (on && gl == lanes - 1)       // the last lane's slice ends at the sequence's last token (an empty slice passes the carry on)
#pragma unroll
        for (int k = 0; k < CPT; ++k) hs[k] = h[k];
}

template <typename T, int CPT, bool FAST>
static void mingru_launch(dim3 grid, dim3 block, const void* z, const void* u, const void* g, long sb, long st, float* state, const int* slots,
                          const int* lens, int fresh, int S, int W, void* out, cudaStream_t s) {
    if (grid.z == 1) {
        mingru_scan_kernel<T, CPT, FAST, false><<<grid, block, 0, s>>>((const T*)z, (const T*)u, (const T*)g, sb, st, state, slots, lens, fresh,
                                                                       S, W, (T*)out);
        return;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = grid.z;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, mingru_scan_kernel<T, CPT, FAST, true>, (const T*)z, (const T*)u, (const T*)g, sb, st, state, slots, lens, fresh, S, W,
                       (T*)out);
}

void mingru_scan(const void* z, const void* u, const void* g, int bf, long sb, long st, float* state, const int* slots, const int* lens,
                 int fresh, int B, int S, int W, void* out, cudaStream_t s) {
    if (B * S * W == 0) return;
    int ty = 1;
    while (ty < 32 && ty * 16 < S) ty <<= 1;
    int cz_most = 1;                                         // blocks per cluster: a lane keeps at least 16 tokens; 8 is the portable limit
    while (cz_most < 8 && ty * cz_most * 2 * 16 <= S) cz_most <<= 1;
    auto shape = [&](int cpt, int& cz) {                     // blocks of the launch with cpt channels per thread
        const int base = (W + 32 * cpt - 1) / (32 * cpt) * B;
        cz = 1;
        while (cz < cz_most && base * cz < 148) cz <<= 1;    // clusters only while a block per SM is not reached
        return base * cz;
    };
    auto a4 = [](const void* p) { return (uintptr_t)p % 4 == 0; };
    int cz2 = 1, cz1 = 1;
    const bool can_pair = bf && W % 2 == 0 && sb % 2 == 0 && st % 2 == 0 && a4(z) && a4(u) && a4(g) && a4(out);
    const bool pairs = can_pair && shape(2, cz2) >= 148;     // two channels per thread where that still fills the GPU
    shape(1, cz1);
    const int cz = pairs ? cz2 : cz1;
    dim3 block(32, ty), grid((W + (pairs ? 63 : 31)) / (pairs ? 64 : 32), B, cz);
    if (pairs) mingru_launch<bf16, 2, true>(grid, block, z, u, g, sb, st, state, slots, lens, fresh, S, W, out, s);
    else if (bf) mingru_launch<bf16, 1, true>(grid, block, z, u, g, sb, st, state, slots, lens, fresh, S, W, out, s);
    else mingru_launch<float, 1, false>(grid, block, z, u, g, sb, st, state, slots, lens, fresh, S, W, out, s);
}

}  // namespace seqmix
