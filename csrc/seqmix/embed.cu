// Token embeddings written as the float residual stream.
//   embed_sinusoid: out[b,t,c] = table[token[b,t], c] * scale + (c even ? sin : cos)((pos0[b] + t) * inv_freq[c / 2])   (angles in float)
//   embed_bigram  : out[b,t,c] = table[token[b,t], c] * scale + pairs[r, c] with r = (previous token * mul_prev + token * mul_cur)
//                   mod buckets, and r = buckets (the table's last row) for a sequence's first token.  The previous token of a
//                   row's first token comes from prev[slot] (unless the rows start their sequences), and each row's last real
//                   token is left there.  A copy of the result in the model's dtype can be written beside the float one.
#include "seq_common.cuh"
#include "seqmix.h"

namespace seqmix {

template <typename T>
__global__ void embed_sinusoid_kernel(const long* __restrict__ tokens, const T* __restrict__ table, float scale,
                                      const float* __restrict__ inv_freq, const int* __restrict__ pos0, int S, int W, int vocab,
                                      float* __restrict__ out) {
    const long row = blockIdx.x;
    const int b = (int)(row / S), t = (int)(row - (long)b * S);
    const long tok = min(max(tokens[row], 0L), (long)vocab - 1);
    const float p = (float)(pos0[b] + t);
    const T* e = table + tok * W;
    float* o = out + row * W;
    for (int i = threadIdx.x; i < (W + 1) / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(p * inv_freq[i], &sn, &cs);
        o[2 * i] = fmaf(ldf(e + 2 * i), scale, sn);
        if (2 * i + 1 < W) o[2 * i + 1] = fmaf(ldf(e + 2 * i + 1), scale, cs);
    }
}

// The block of a row's first token reads the carried token and then leaves the row's last one, so no other block touches the slot.
template <typename T>
__global__ void embed_bigram_kernel(const long* __restrict__ tokens, const T* __restrict__ table, float scale, const T* __restrict__ pairs,
                                    long buckets, long mul_prev, long mul_cur, long* prev, const int* __restrict__ slots,
                                    const int* __restrict__ lens, int fresh, int S, int W, int vocab, float* __restrict__ out,
                                    T* __restrict__ out_lp) {
    __shared__ long s_prev;
    const long row = blockIdx.x;
    const int b = (int)(row / S), t = (int)(row - (long)b * S);
    const long tok = min(max(tokens[row], 0L), (long)vocab - 1);
    if (t > 0) {
        if (threadIdx.x == 0) s_prev = min(max(tokens[row - 1], 0L), (long)vocab - 1);
    } else if (threadIdx.x == 0) {
        const int len = min(lens[b], S);
        long* slot = prev ? prev + slots[b] : nullptr;
        s_prev = (fresh || !slot) ? -1 : *slot;
        if (slot && len > 0) *slot = min(max(tokens[row + len - 1], 0L), (long)vocab - 1);
    }
    __syncthreads();
    const T* e = table + tok * W;
    const T* pr = nullptr;
    if (pairs) pr = pairs + (s_prev < 0 ? buckets : (s_prev * mul_prev + tok * mul_cur) % buckets) * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = ldf(e + c) * scale;
        if (pr) v += ldf(pr + c);
        out[row * W + c] = v;
        if (out_lp) stf(out_lp + row * W + c, v);
    }
}

void embed_bigram(const long* tokens, const void* table, int bf, float scale, const void* pairs, long buckets, long mul_prev, long mul_cur,
                  long* prev, const int* slots, const int* lens, int fresh, int B, int S, int W, int vocab, float* out, void* out_lp,
                  cudaStream_t s) {
    if (B * S == 0) return;
    const int threads = W >= 512 ? 256 : 128;
    if (bf) embed_bigram_kernel<bf16><<<B * S, threads, 0, s>>>(tokens, (const bf16*)table, scale, (const bf16*)pairs, buckets, mul_prev, mul_cur,
                                                              prev, slots, lens, fresh, S, W, vocab, out, (bf16*)out_lp);
    else embed_bigram_kernel<float><<<B * S, threads, 0, s>>>(tokens, (const float*)table, scale, (const float*)pairs, buckets, mul_prev, mul_cur,
                                                             prev, slots, lens, fresh, S, W, vocab, out, (float*)out_lp);
}

void embed_sinusoid(const long* tokens, const void* table, int bf, float scale, const float* inv_freq, const int* pos0, int B, int S, int W,
                    int vocab, float* out, cudaStream_t s) {
    if (B * S == 0) return;
    const int threads = W >= 512 ? 256 : 128;
    if (bf) embed_sinusoid_kernel<bf16><<<B * S, threads, 0, s>>>(tokens, (const bf16*)table, scale, inv_freq, pos0, S, W, vocab, out);
    else embed_sinusoid_kernel<float><<<B * S, threads, 0, s>>>(tokens, (const float*)table, scale, inv_freq, pos0, S, W, vocab, out);
}

}  // namespace seqmix
