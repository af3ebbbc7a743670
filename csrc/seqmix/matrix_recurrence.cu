// Recurrences with a matrix state per head and ONE decay per head and token, states in float.
//   gated_delta_scan : M <- g M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q      (M [D, V]; the read-out sees the write)
//                      q and k are made unit vectors here (x / sqrt(sum x^2 + 1e-6), q also times D^-1/2); beta = sigmoid(braw),
//                      g = exp(-exp(a_log) softplus(araw + dt_bias)).  With A = M_old^T k and Bq = M_old^T q one pass over the old
//                      state gives u = beta (v - g A) and o = g Bq + (k.q) u, and the update M = g M_old + k u^T follows in registers.
//   gated_delta_scan with a decay per KEY CHANNEL (araw / dt_bias hold D numbers per head): g is a vector that scales the rows of M.
//                      With gk = g * k and gq = g * q (coordinate by coordinate), A = M_old^T gk and Bq = M_old^T gq give
//                      u = beta (v - A), o = Bq + (k.q) u and M = diag(g) M_old + k u^T: four staged vectors per token instead of two.
//   ssd_scan         : dt = softplus(dtraw + dt_bias);  M <- exp(-exp(a_log) dt) M + dt b x^T;  y = M^T c + dskip x   (M [N, V])
// A block owns 32 value columns of one (sequence, head): lane = column, warp = one of 8 row groups, a thread keeps DPT consecutive
// rows of its column in registers (rows past the state's size are zeros that never change), so state loads and stores are whole
// 128-byte rows and a token's per-row numbers come from shared memory four at a time.  Tokens are staged through shared
// memory 8 at a time (a warp prepares one token: norms, decays, gates, from numbers fetched one chunk ahead); the per-token sums over
// rows are folded across the warps
// through a shared array: one barrier per token in the delta rule (its write needs the sum), one per 8 tokens in the state space scan
// (its read-out does not feed back).  Tokens at or past lens[b] write zeros and leave the state alone.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

constexpr int kCols = 32, kRowGroups = 8, kTok = 8;

template <typename T, int DPT>
__global__ void __launch_bounds__(256) gated_delta_kernel(
    const T* __restrict__ q, const T* __restrict__ k, long qk_sb, long qk_st, const T* __restrict__ v, long v_sb, long v_st,
    const float* __restrict__ braw, const float* __restrict__ araw, long ba_sb, long ba_st, const float* __restrict__ a_log,
    const float* __restrict__ dt_bias, float* state, const int* __restrict__ slots, const int* __restrict__ lens, int fresh, int S,
    int H, int G, int D, int V, float qscale, float* __restrict__ out) {
    extern __shared__ float sm[];
    constexpr int Dp = DPT * kRowGroups;         // padded row count (>= D); rows past D hold zeros
    float* sk = sm;                              // [kTok][Dp] unit keys
    float* sq = sk + kTok * Dp;                  // [kTok][Dp] unit queries times qscale
    float* sv = sq + kTok * Dp;                  // [kTok][kCols]
    float* sc = sv + kTok * kCols;               // [kTok][4]: g, beta, k.q
    float* part = sc + kTok * 4;                 // [2][2][kRowGroups][kCols]
    const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * kCols;
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5, j = j0 + lane;
    const int len = min(lens[b], S), hk = h / (H / G);
    const bool col = j < V;
    float* sp = state + (((long)slots[b] * H + h) * D) * V;
    float M[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r * DPT + i;
        M[i] = (!fresh && col && d < D) ? sp[(long)d * V + j] : 0.f;
    }
    for (int x = threadIdx.x; x < 2 * kTok * Dp; x += 256) sm[x] = 0.f;       // the padding rows stay zero
    const float ea = expf(a_log[h]), db = dt_bias[h];
    // warp r prepares token t0 + r of every chunk; its raw numbers are fetched one chunk ahead, so that the loads fly during the
    // previous chunk's arithmetic
    constexpr int DL = DPT >= 4 ? DPT / 4 : 1;   // key coordinates per lane: D <= 8 DPT = 32 DL
    float qraw[DL], kraw[DL], vraw = 0.f, braw_ = 0.f, araw_ = 0.f;
    auto fetch = [&](int t) {
        if (t < len) {
            const T* qp = q + (long)b * qk_sb + (long)t * qk_st + (long)hk * D;
            const T* kp = k + (long)b * qk_sb + (long)t * qk_st + (long)hk * D;
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                qraw[i] = d < D ? ldf(qp + d) : 0.f;
                kraw[i] = d < D ? ldf(kp + d) : 0.f;
            }
            vraw = col ? ldf(v + (long)b * v_sb + (long)t * v_st + (long)h * V + j) : 0.f;
            const long o = (long)b * ba_sb + (long)t * ba_st + h;
            braw_ = braw[o];
            araw_ = araw[o];
        }
    };
    fetch(r);
    for (int t0 = 0; t0 < len; t0 += kTok) {
        __syncthreads();                         // the previous chunk's tokens are consumed
        if (t0 + r < len) {
            float qq = 0.f, kk = 0.f, qk = 0.f;
#pragma unroll
            for (int i = 0; i < DL; ++i) { qq = fmaf(qraw[i], qraw[i], qq); kk = fmaf(kraw[i], kraw[i], kk); qk = fmaf(qraw[i], kraw[i], qk); }
            qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
            const float iq = qscale / sqrtf(qq + 1e-6f), ik = 1.f / sqrtf(kk + 1e-6f);
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) { sq[r * Dp + d] = qraw[i] * iq; sk[r * Dp + d] = kraw[i] * ik; }
            }
            sv[r * kCols + lane] = vraw;
            if (lane == 0) {
                sc[r * 4 + 0] = expf(-ea * softplusf_(araw_ + db));
                sc[r * 4 + 1] = sigmoidf_(braw_);
                sc[r * 4 + 2] = qk * iq * ik;
            }
        }
        __syncthreads();
        fetch(t0 + kTok + r);
        const int nt = min(kTok, len - t0);
        for (int u = 0; u < nt; ++u) {
            const float* ku = sk + u * Dp + r * DPT;
            const float* qu = sq + u * Dp + r * DPT;
            float kr[DPT];
            float A = 0.f, Bq = 0.f;
            if (DPT >= 4) {
#pragma unroll
                for (int i = 0; i < DPT; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ku + i), q4 = *reinterpret_cast<const float4*>(qu + i);
                    kr[i] = k4.x; kr[i + 1] = k4.y; kr[i + 2] = k4.z; kr[i + 3] = k4.w;
                    A = fmaf(M[i], k4.x, fmaf(M[i + 1], k4.y, fmaf(M[i + 2], k4.z, fmaf(M[i + 3], k4.w, A))));
                    Bq = fmaf(M[i], q4.x, fmaf(M[i + 1], q4.y, fmaf(M[i + 2], q4.z, fmaf(M[i + 3], q4.w, Bq))));
                }
            } else {
#pragma unroll
                for (int i = 0; i < DPT; ++i) { kr[i] = ku[i]; A = fmaf(M[i], kr[i], A); Bq = fmaf(M[i], qu[i], Bq); }
            }
            float* pb = part + ((t0 + u) & 1) * 2 * kRowGroups * kCols;
            pb[r * kCols + lane] = A;
            pb[(kRowGroups + r) * kCols + lane] = Bq;
            __syncthreads();
            A = 0.f; Bq = 0.f;
#pragma unroll
            for (int w = 0; w < kRowGroups; ++w) { A += pb[w * kCols + lane]; Bq += pb[(kRowGroups + w) * kCols + lane]; }
            const float g = sc[u * 4], beta = sc[u * 4 + 1], kq = sc[u * 4 + 2];
            const float uv = beta * (sv[u * kCols + lane] - g * A);
            if (r == 0 && col) out[(((long)b * S + t0 + u) * H + h) * V + j] = fmaf(g, Bq, kq * uv);
#pragma unroll
            for (int i = 0; i < DPT; ++i) M[i] = fmaf(g, M[i], kr[i] * uv);
        }
    }
    if (col) {
        for (int t = len + r; t < S; t += kRowGroups) out[(((long)b * S + t) * H + h) * V + j] = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r * DPT + i;
            if (d < D && (len > 0 || fresh)) sp[(long)d * V + j] = M[i];
        }
    }
}

// The delta rule with one decay per head and key channel.  Same block shape and staging as gated_delta_kernel; araw [B,S,H,D] float
// (strides a_sb, a_st; heads one after another), dt_bias [H*D].
template <typename T, int DPT>
__global__ void __launch_bounds__(256) gated_delta_channel_kernel(
    const T* __restrict__ q, const T* __restrict__ k, long qk_sb, long qk_st, const T* __restrict__ v, long v_sb, long v_st,
    const float* __restrict__ braw, long b_sb, long b_st, const float* __restrict__ araw, long a_sb, long a_st,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* state, const int* __restrict__ slots,
    const int* __restrict__ lens, int fresh, int S, int H, int G, int D, int V, float qscale, float* __restrict__ out) {
    extern __shared__ float sm[];
    constexpr int Dp = DPT * kRowGroups;         // padded row count (>= D); rows past D hold zeros
    float* sk = sm;                              // [kTok][Dp] unit keys
    float* sg = sk + kTok * Dp;                  // [kTok][Dp] decays
    float* sgk = sg + kTok * Dp;                 // [kTok][Dp] decay * unit key
    float* sgq = sgk + kTok * Dp;                // [kTok][Dp] decay * unit query * qscale
    float* sv = sgq + kTok * Dp;                 // [kTok][kCols]
    float* sc = sv + kTok * kCols;               // [kTok][4]: beta, k.q
    float* part = sc + kTok * 4;                 // [2][2][kRowGroups][kCols]
    const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * kCols;
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5, j = j0 + lane;
    const int len = min(lens[b], S), hk = h / (H / G);
    const bool col = j < V;
    float* sp = state + (((long)slots[b] * H + h) * D) * V;
    float M[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r * DPT + i;
        M[i] = (!fresh && col && d < D) ? sp[(long)d * V + j] : 0.f;
    }
    for (int x = threadIdx.x; x < 4 * kTok * Dp; x += 256) sm[x] = 0.f;       // the padding rows stay zero
    const float ea = expf(a_log[h]);
    constexpr int DL = DPT >= 4 ? DPT / 4 : 1;   // key coordinates per lane: D <= 8 DPT = 32 DL
    float qraw[DL], kraw[DL], araw_[DL], db[DL], vraw = 0.f, braw_ = 0.f;
#pragma unroll
    for (int i = 0; i < DL; ++i) { const int d = lane + 32 * i; db[i] = d < D ? dt_bias[(long)h * D + d] : 0.f; }
    auto fetch = [&](int t) {
        if (t < len) {
            const T* qp = q + (long)b * qk_sb + (long)t * qk_st + (long)hk * D;
            const T* kp = k + (long)b * qk_sb + (long)t * qk_st + (long)hk * D;
            const float* ap = araw + (long)b * a_sb + (long)t * a_st + (long)h * D;
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                qraw[i] = d < D ? ldf(qp + d) : 0.f;
                kraw[i] = d < D ? ldf(kp + d) : 0.f;
                araw_[i] = d < D ? ap[d] : 0.f;
            }
            vraw = col ? ldf(v + (long)b * v_sb + (long)t * v_st + (long)h * V + j) : 0.f;
            braw_ = braw[(long)b * b_sb + (long)t * b_st + h];
        }
    };
    fetch(r);
    for (int t0 = 0; t0 < len; t0 += kTok) {
        __syncthreads();                         // the previous chunk's tokens are consumed
        if (t0 + r < len) {
            float qq = 0.f, kk = 0.f, qk = 0.f;
#pragma unroll
            for (int i = 0; i < DL; ++i) { qq = fmaf(qraw[i], qraw[i], qq); kk = fmaf(kraw[i], kraw[i], kk); qk = fmaf(qraw[i], kraw[i], qk); }
            qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
            const float iq = qscale / sqrtf(qq + 1e-6f), ik = 1.f / sqrtf(kk + 1e-6f);
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    const float g = expf(-ea * softplusf_(araw_[i] + db[i])), ku = kraw[i] * ik;
                    sk[r * Dp + d] = ku;
                    sg[r * Dp + d] = g;
                    sgk[r * Dp + d] = g * ku;
                    sgq[r * Dp + d] = g * (qraw[i] * iq);
                }
            }
            sv[r * kCols + lane] = vraw;
            if (lane == 0) {
                sc[r * 4 + 0] = sigmoidf_(braw_);
                sc[r * 4 + 1] = qk * iq * ik;
            }
        }
        __syncthreads();
        fetch(t0 + kTok + r);
        const int nt = min(kTok, len - t0);
        for (int u = 0; u < nt; ++u) {
            const float* ku = sk + u * Dp + r * DPT;
            const float* gu = sg + u * Dp + r * DPT;
            const float* gku = sgk + u * Dp + r * DPT;
            const float* gqu = sgq + u * Dp + r * DPT;
            float kr[DPT], gr[DPT];
            float A = 0.f, Bq = 0.f;
            if (DPT >= 4) {
#pragma unroll
                for (int i = 0; i < DPT; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ku + i), g4 = *reinterpret_cast<const float4*>(gu + i);
                    const float4 a4 = *reinterpret_cast<const float4*>(gku + i), q4 = *reinterpret_cast<const float4*>(gqu + i);
                    kr[i] = k4.x; kr[i + 1] = k4.y; kr[i + 2] = k4.z; kr[i + 3] = k4.w;
                    gr[i] = g4.x; gr[i + 1] = g4.y; gr[i + 2] = g4.z; gr[i + 3] = g4.w;
                    A = fmaf(M[i], a4.x, fmaf(M[i + 1], a4.y, fmaf(M[i + 2], a4.z, fmaf(M[i + 3], a4.w, A))));
                    Bq = fmaf(M[i], q4.x, fmaf(M[i + 1], q4.y, fmaf(M[i + 2], q4.z, fmaf(M[i + 3], q4.w, Bq))));
                }
            } else {
#pragma unroll
                for (int i = 0; i < DPT; ++i) { kr[i] = ku[i]; gr[i] = gu[i]; A = fmaf(M[i], gku[i], A); Bq = fmaf(M[i], gqu[i], Bq); }
            }
            float* pb = part + ((t0 + u) & 1) * 2 * kRowGroups * kCols;
            pb[r * kCols + lane] = A;
            pb[(kRowGroups + r) * kCols + lane] = Bq;
            __syncthreads();
            A = 0.f; Bq = 0.f;
#pragma unroll
            for (int w = 0; w < kRowGroups; ++w) { A += pb[w * kCols + lane]; Bq += pb[(kRowGroups + w) * kCols + lane]; }
            const float beta = sc[u * 4], kq = sc[u * 4 + 1];
            const float uv = beta * (sv[u * kCols + lane] - A);
            if (r == 0 && col) out[(((long)b * S + t0 + u) * H + h) * V + j] = fmaf(kq, uv, Bq);
#pragma unroll
            for (int i = 0; i < DPT; ++i) M[i] = fmaf(gr[i], M[i], kr[i] * uv);
        }
    }
    if (col) {
        for (int t = len + r; t < S; t += kRowGroups) out[(((long)b * S + t) * H + h) * V + j] = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r * DPT + i;
            if (d < D && (len > 0 || fresh)) sp[(long)d * V + j] = M[i];
        }
    }
}

template <typename T, int DPT>
__global__ void __launch_bounds__(256) ssd_kernel(
    const T* __restrict__ x, long x_sb, long x_st, const T* __restrict__ bm, const T* __restrict__ cm, long bc_sb, long bc_st,
    const float* __restrict__ dtraw, long dt_sb, long dt_st, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const float* __restrict__ dskip, float* state, const int* __restrict__ slots, const int* __restrict__ lens, int fresh, int S, int H,
    int G, int N, int V, float* __restrict__ out) {
    extern __shared__ float sm[];
    constexpr int Np = DPT * kRowGroups;         // padded row count (>= N); rows past N hold zeros
    float* sb = sm;                              // [kTok][Np] dt * b
    float* scm = sb + kTok * Np;                 // [kTok][Np] c
    float* sx = scm + kTok * Np;                 // [kTok][kCols]
    float* sc = sx + kTok * kCols;               // [kTok][2]: decay
    float* part = sc + kTok * 2;                 // [kTok][kRowGroups][kCols]
    const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * kCols;
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5, j = j0 + lane;
    const int len = min(lens[b], S), hg = h / (H / G);
    const bool col = j < V;
    float* sp = state + (((long)slots[b] * H + h) * N) * V;
    float M[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = r * DPT + i;
        M[i] = (!fresh && col && d < N) ? sp[(long)d * V + j] : 0.f;
    }
    for (int x = threadIdx.x; x < 2 * kTok * Np; x += 256) sm[x] = 0.f;       // the padding rows stay zero
    const float ea = expf(a_log[h]), db = dt_bias[h], ds = dskip[h];
    constexpr int DL = DPT >= 4 ? DPT / 4 : 1;   // state rows per lane when a warp prepares a token: N <= 8 DPT = 32 DL
    float braw[DL], craw[DL], xraw = 0.f, dtr = 0.f;
    auto fetch = [&](int t) {
        if (t < len) {
            const T* bp = bm + (long)b * bc_sb + (long)t * bc_st + (long)hg * N;
            const T* cp = cm + (long)b * bc_sb + (long)t * bc_st + (long)hg * N;
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                braw[i] = d < N ? ldf(bp + d) : 0.f;
                craw[i] = d < N ? ldf(cp + d) : 0.f;
            }
            xraw = col ? ldf(x + (long)b * x_sb + (long)t * x_st + (long)h * V + j) : 0.f;
            dtr = dtraw[(long)b * dt_sb + (long)t * dt_st + h];
        }
    };
    fetch(r);
    for (int t0 = 0; t0 < len; t0 += kTok) {
        __syncthreads();
        if (t0 + r < len) {
            const float dt = softplusf_(dtr + db);
#pragma unroll
            for (int i = 0; i < DL; ++i) {
                const int d = lane + 32 * i;
                if (d < N) { sb[r * Np + d] = dt * braw[i]; scm[r * Np + d] = craw[i]; }
            }
            sx[r * kCols + lane] = xraw;
            if (lane == 0) sc[r * 2] = expf(-ea * dt);
        }
        __syncthreads();
        fetch(t0 + kTok + r);
        // the read-out does not feed back into the state: the chunk's tokens run without a barrier between them, their row sums
        // meet afterwards (warp r folds and writes token t0 + r)
        const int nt = min(kTok, len - t0);
        float yp[kTok];
#pragma unroll
        for (int u = 0; u < kTok; ++u) {
            yp[u] = 0.f;
            if (u < nt) {
                const float* bu = sb + u * Np + r * DPT;
                const float* cu = scm + u * Np + r * DPT;
                const float dec = sc[u * 2], xv = sx[u * kCols + lane];
                float y = 0.f;
                if (DPT >= 4) {
#pragma unroll
                    for (int i = 0; i < DPT; i += 4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bu + i), c4 = *reinterpret_cast<const float4*>(cu + i);
                        M[i] = fmaf(dec, M[i], b4.x * xv); M[i + 1] = fmaf(dec, M[i + 1], b4.y * xv);
                        M[i + 2] = fmaf(dec, M[i + 2], b4.z * xv); M[i + 3] = fmaf(dec, M[i + 3], b4.w * xv);
                        y = fmaf(M[i], c4.x, fmaf(M[i + 1], c4.y, fmaf(M[i + 2], c4.z, fmaf(M[i + 3], c4.w, y))));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < DPT; ++i) { M[i] = fmaf(dec, M[i], bu[i] * xv); y = fmaf(M[i], cu[i], y); }
                }
                yp[u] = y;
            }
        }
#pragma unroll
        for (int u = 0; u < kTok; ++u) part[(u * kRowGroups + r) * kCols + lane] = yp[u];
        __syncthreads();
        if (r < nt && col) {
            float y = 0.f;
#pragma unroll
            for (int w = 0; w < kRowGroups; ++w) y += part[(r * kRowGroups + w) * kCols + lane];
            out[(((long)b * S + t0 + r) * H + h) * V + j] = fmaf(ds, sx[r * kCols + lane], y);
        }
    }
    if (col) {
        for (int t = len + r; t < S; t += kRowGroups) out[(((long)b * S + t) * H + h) * V + j] = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = r * DPT + i;
            if (d < N && (len > 0 || fresh)) sp[(long)d * V + j] = M[i];
        }
    }
}

static int rows_per_thread(int D) {
    const int need = (D + kRowGroups - 1) / kRowGroups;
    for (int p = 1; p <= 64; p *= 2)
        if (need <= p) return p;
    return 0;
}

bool gated_delta_scan(const void* q, const void* k, long qk_sb, long qk_st, const void* v, long v_sb, long v_st, int bf, const float* braw,
                      const float* araw, long ba_sb, long ba_st, const float* a_log, const float* dt_bias, float* state, const int* slots,
                      const int* lens, int fresh, int B, int S, int H, int G, int D, int V, float qscale, float* out, cudaStream_t s) {
    const int dpt = rows_per_thread(D);
    if (!dpt) return false;
    if (B == 0 || S == 0) return true;
    dim3 grid(H, B, (V + kCols - 1) / kCols), block(256);
    const size_t smem = sizeof(float) * (2 * kTok * dpt * kRowGroups + kTok * kCols + kTok * 4 + 2 * 2 * kRowGroups * kCols);
#define SEQMIX_GDR(T, P)                                                                                                              \
    gated_delta_kernel<T, P><<<grid, block, smem, s>>>((const T*)q, (const T*)k, qk_sb, qk_st, (const T*)v, v_sb, v_st, braw, araw, ba_sb, \
                                                       ba_st, a_log, dt_bias, state, slots, lens, fresh, S, H, G, D, V, qscale, out)
#define SEQMIX_GDR_T(P) do { if (bf) SEQMIX_GDR(bf16, P); else SEQMIX_GDR(float, P); } while (0)
    switch (dpt) {
        case 1: SEQMIX_GDR_T(1); break;
        case 2: SEQMIX_GDR_T(2); break;
        case 4: SEQMIX_GDR_T(4); break;
        case 8: SEQMIX_GDR_T(8); break;
        case 16: SEQMIX_GDR_T(16); break;
        case 32: SEQMIX_GDR_T(32); break;
        default: SEQMIX_GDR_T(64); break;
    }
#undef SEQMIX_GDR_T
#undef SEQMIX_GDR
    return true;
}

bool gated_delta_channel_scan(const void* q, const void* k, long qk_sb, long qk_st, const void* v, long v_sb, long v_st, int bf,
                              const float* braw, long b_sb, long b_st, const float* araw, long a_sb, long a_st, const float* a_log,
                              const float* dt_bias, float* state, const int* slots, const int* lens, int fresh, int B, int S, int H, int G,
                              int D, int V, float qscale, float* out, cudaStream_t s) {
    const int dpt = rows_per_thread(D);
    if (!dpt) return false;
    if (B == 0 || S == 0) return true;
    dim3 grid(H, B, (V + kCols - 1) / kCols), block(256);
    const size_t smem = sizeof(float) * (4 * kTok * dpt * kRowGroups + kTok * kCols + kTok * 4 + 2 * 2 * kRowGroups * kCols);
#define SEQMIX_GDC(T, P)                                                                                                              \
    do {                                                                                                                              \
        cudaFuncSetAttribute(gated_delta_channel_kernel<T, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);               \
        gated_delta_channel_kernel<T, P><<<grid, block, smem, s>>>((const T*)q, (const T*)k, qk_sb, qk_st, (const T*)v, v_sb, v_st, braw,  \
                                                                   b_sb, b_st, araw, a_sb, a_st, a_log, dt_bias, state, slots, lens, fresh, \
                                                                   S, H, G, D, V, qscale, out);                                       \
    } while (0)
#define SEQMIX_GDC_T(P) do { if (bf) SEQMIX_GDC(bf16, P); else SEQMIX_GDC(float, P); } while (0)
    switch (dpt) {
        case 1: SEQMIX_GDC_T(1); break;
        case 2: SEQMIX_GDC_T(2); break;
        case 4: SEQMIX_GDC_T(4); break;
        case 8: SEQMIX_GDC_T(8); break;
        case 16: SEQMIX_GDC_T(16); break;
        case 32: SEQMIX_GDC_T(32); break;
        default: SEQMIX_GDC_T(64); break;
    }
#undef SEQMIX_GDC_T
#undef SEQMIX_GDC
    return true;
}

bool ssd_scan(const void* x, long x_sb, long x_st, const void* bm, const void* cm, long bc_sb, long bc_st, int bf, const float* dtraw,
              long dt_sb, long dt_st, const float* a_log, const float* dt_bias, const float* dskip, float* state, const int* slots,
              const int* lens, int fresh, int B, int S, int H, int G, int N, int V, float* out, cudaStream_t s) {
    const int dpt = rows_per_thread(N);
    if (!dpt) return false;
    if (B == 0 || S == 0) return true;
    dim3 grid(H, B, (V + kCols - 1) / kCols), block(256);
    const size_t smem = sizeof(float) * (2 * kTok * dpt * kRowGroups + kTok * kCols + kTok * 2 + kTok * kRowGroups * kCols);
#define SEQMIX_SSD(T, P)                                                                                                              \
    ssd_kernel<T, P><<<grid, block, smem, s>>>((const T*)x, x_sb, x_st, (const T*)bm, (const T*)cm, bc_sb, bc_st, dtraw, dt_sb, dt_st,   \
                                               a_log, dt_bias, dskip, state, slots, lens, fresh, S, H, G, N, V, out)
#define SEQMIX_SSD_T(P) do { if (bf) SEQMIX_SSD(bf16, P); else SEQMIX_SSD(float, P); } while (0)
    switch (dpt) {
        case 1: SEQMIX_SSD_T(1); break;
        case 2: SEQMIX_SSD_T(2); break;
        case 4: SEQMIX_SSD_T(4); break;
        case 8: SEQMIX_SSD_T(8); break;
        case 16: SEQMIX_SSD_T(16); break;
        case 32: SEQMIX_SSD_T(32); break;
        default: SEQMIX_SSD_T(64); break;
    }
#undef SEQMIX_SSD_T
#undef SEQMIX_SSD
    return true;
}

}  // namespace seqmix
