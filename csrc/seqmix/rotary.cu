// Rotation by position of the query and key heads of a stacked projection, with a FLOAT result: the input row holds hq query heads
// and hk key heads of D numbers and then anything else (values, ...); the first `dims` coordinates of every query / key head turn by
// the angle p * inv_freq[i] (pair i = coordinates i and i + dims/2), queries are multiplied by q_scale, keys by k_scale, the rest of
// the row is copied.  Used where everything after the projection enters a recurrence and therefore stays float.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

// one thread per PAIR of a rotated stretch, or per single coordinate elsewhere: units per row = C - (hq + hk) * dims / 2
template <typename T>
__global__ void rotary_qkv_f32_kernel(const T* __restrict__ p, long p_sb, long p_st, int B, int S, int C, int hq, int hk, int D, int dims,
                                      const float* __restrict__ inv_freq, const int* __restrict__ pos0, float q_scale, float k_scale,
                                      float* __restrict__ out) {
    const int half = dims / 2, per_head = D - half, nrot = (hq + hk) * per_head, per_row = nrot + (C - (hq + hk) * D);
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)B * S * per_row) return;
    const long n = idx / per_row;
    const int u = (int)(idx - n * per_row), b = (int)(n / S), t = (int)(n - (long)b * S);
    const T* x = p + (long)b * p_sb + (long)t * p_st;
    float* o = out + n * C;
    if (u >= nrot) {                                 // past the heads: copied
        const int c = (hq + hk) * D + (u - nrot);
        o[c] = ldf(x + c);
        return;
    }
    const int h = u / per_head, i = u - h * per_head;
    const float sc = h < hq ? q_scale : k_scale;
    const int c0 = h * D;
    if (i < half) {
        float a = ldf(x + c0 + i), bb = ldf(x + c0 + i + half), sn, cs;
        sincosf((float)(pos0[b] + t) * inv_freq[i], &sn, &cs);
        o[c0 + i] = (a * cs - bb * sn) * sc;
        o[c0 + i + half] = (bb * cs + a * sn) * sc;
    } else {                                         // coordinates past the rotated ones: scaled only
        const int c = c0 + dims + (i - half);
        o[c] = ldf(x + c) * sc;
    }
}

void rotary_qkv_f32(const void* p, int bf, long p_sb, long p_st, int B, int S, int C, int hq, int hk, int D, int dims,
                    const float* inv_freq, const int* pos0, float q_scale, float k_scale, float* out, cudaStream_t s) {
    const long total = (long)B * S * ((hq + hk) * (D - dims / 2) + (C - (hq + hk) * D));
    if (total == 0) return;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (bf) rotary_qkv_f32_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)p, p_sb, p_st, B, S, C, hq, hk, D, dims, inv_freq, pos0, q_scale, k_scale, out);
    else rotary_qkv_f32_kernel<float><<<blocks, 256, 0, s>>>((const float*)p, p_sb, p_st, B, S, C, hq, hk, D, dims, inv_freq, pos0, q_scale, k_scale, out);
}

}  // namespace seqmix
