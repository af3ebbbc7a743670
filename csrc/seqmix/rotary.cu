// Rotation by position of the query and key heads of a stacked projection, with a FLOAT result: the input row holds hq query heads
// and hk key heads of D numbers and then anything else (values, ...); the first `dims` coordinates of every query / key head turn by
// the angle p * inv_freq[i] (pair i = coordinates i and i + dims/2), queries are multiplied by q_scale, keys by k_scale, the rest of
// the row is copied.  Used where everything after the projection enters a recurrence and therefore stays float.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

// A block per token.  The angle of pair i is the same for every head, so a thread forms sin / cos ONCE for its pair and walks the
// heads (threads split into groups over the heads when the pairs are few); then all threads copy / scale what is not rotated.
template <typename T>
__global__ void __launch_bounds__(256) rotary_qkv_f32_kernel(const T* __restrict__ p, long p_sb, long p_st, int S, int C, int hq, int hk,
                                                             int D, int dims, const float* __restrict__ inv_freq,
                                                             const int* __restrict__ pos0, float q_scale, float k_scale,
                                                             float* __restrict__ out) {
    const int half = dims / 2, nh = hq + hk, tid = threadIdx.x;
    const long n = blockIdx.x;
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const T* x = p + (long)b * p_sb + (long)t * p_st;
    float* o = out + n * C;
    if (half > 0) {
        const int groups = max(1, min(nh, 256 / half));            // head groups that run side by side
        for (int u = tid; u < half * groups; u += 256) {
            const int g = u / half, i = u - g * half;
            float sn, cs;
            sincosf((float)(pos0[b] + t) * inv_freq[i], &sn, &cs);
            for (int h = g; h < nh; h += groups) {
                const float sc = h < hq ? q_scale : k_scale;
                const int c0 = h * D + i;
                const float a = ldf(x + c0), bb = ldf(x + c0 + half);
                o[c0] = (a * cs - bb * sn) * sc;
                o[c0 + half] = (bb * cs + a * sn) * sc;
            }
        }
    }
    const int rest = D - dims;                                       // coordinates of a head past the rotated ones: scaled only
    for (int u = tid; u < nh * rest; u += 256) {
        const int h = u / rest, c = h * D + dims + (u - h * rest);
        o[c] = ldf(x + c) * (h < hq ? q_scale : k_scale);
    }
    for (int c = nh * D + tid; c < C; c += 256) o[c] = ldf(x + c);   // past the heads: copied
}

void rotary_qkv_f32(const void* p, int bf, long p_sb, long p_st, int B, int S, int C, int hq, int hk, int D, int dims,
                    const float* inv_freq, const int* pos0, float q_scale, float k_scale, float* out, cudaStream_t s) {
    const long rows = (long)B * S;
    if (rows == 0 || C == 0) return;
    if (bf) rotary_qkv_f32_kernel<bf16><<<(unsigned)rows, 256, 0, s>>>((const bf16*)p, p_sb, p_st, S, C, hq, hk, D, dims, inv_freq, pos0, q_scale, k_scale, out);
    else rotary_qkv_f32_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)p, p_sb, p_st, S, C, hq, hk, D, dims, inv_freq, pos0, q_scale, k_scale, out);
}

}  // namespace seqmix
