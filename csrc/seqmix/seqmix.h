// Launchers of the sequence-mixer kernels (raw pointers; `bf` / `*_bf16` flags: 1 = bfloat16 activations, 0 = float).
#pragma once
#include <cuda_runtime.h>

namespace seqmix {

void short_conv(const void* x, int in_bf16, long x_sb, long x_st, const float* w, const float* bias, void* state, const int* slots,
                const int* lens, int B, int S, int C, int taps, int fresh, int residual, int act, void* out, int out_bf16, cudaStream_t s);
void rms_norm(const void* x, int in_bf16, long x_stride, int rows, int C, const float* w, int w_stride, float eps, const void* gate,
              long gate_stride, void* out, int out_bf16, long out_stride, float* res, long res_stride, int center, cudaStream_t s);
// x (float, in place) <- norm(alpha * x + sigmoid(gate) * y) * w; gate may be null; lp (of y's dtype, may be null) gets a copy
void postnorm_gated(float* x, long x_stride, const void* y, long y_stride, const void* gate, long gate_stride, int bf, const float* w,
                    float alpha, float eps, int rows, int C, void* lp, long lp_stride, cudaStream_t s);
void latent_kv_store(const void* kv, int bf, long kv_sb, long kv_st, int B, int S, int C, int R, int dims, const float* nw, float eps,
                     const float* inv_freq, const int* pos0, const int* lens, const int* slots, void* cache, int ring, void* rows,
                     cudaStream_t s);
void rope_q(void* q, int bf, long q_sn, long q_sh, int N, int S, int H, int dims, const float* inv_freq, const int* pos0, cudaStream_t s);
void latent_window_attention(const void* qa, int bf, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys,
                             long key_sb, int ring, const int* key_index, const int* pos0, const int* lens, int B, int S, int H, int C,
                             int R, int window, float scale, void* out, long out_sn, long out_sh, cudaStream_t s);
// Single new tokens against their rings (latent_decode.cu): blocks over (ring chunk, sequence, head tile) leave partial softmaxes
// part_m / part_l [B, splits, H] and part_acc [B, splits, H, C] (float), which a second kernel merges into out[h, b, :].
int latent_ring_decode_splits(int ring);
bool latent_ring_decode_fits(int C, int R);
void latent_ring_decode(const void* qa, int bf, long qa_sn, long qa_sh, const void* qr, long qr_sn, long qr_sh, const void* keys,
                        long key_sb, int ring, const int* key_index, const int* pos0, const int* lens, int B, int H, int C, int R,
                        int window, float scale, float* part_m, float* part_l, float* part_acc, void* out, long out_sn, long out_sh,
                        cudaStream_t s);
// Prompt attention in the expanded form as one fused kernel (latent_prefill.cu; bfloat16, sizes in whole 16s up to 256): q [B,S,H,D+R],
// kx [B,S,H,D], rows [B,S,CR] (last R numbers: the shared rotated key part), v [B,S,H,VD] → out [B,S,H*VD].  false: sizes do not fit.
bool latent_prompt_attention_fits(int D, int R, int CR, int VD);
bool latent_prompt_attention(const void* q, const void* kx, const void* rows, const void* v, const int* lens, int B, int S, int H, int D,
                             int R, int CR, int VD, int window, float scale, void* out, cudaStream_t s);
void window_softmax(const float* scores, long rows, int span, float scale, int ring_mode, int H, int Qb, int nblk, int w_eff, int window,
                    const int* pos0, const int* lens, void* out, int out_bf16, cudaStream_t s);
// `decay` (one float per head, or null): a fixed decay per head instead of the projected z (retention); z and zbias are not read then.
bool gla_scan(const void* q, const void* k, const void* v, int bf, long sb, long st, const void* z, long z_sb, long z_st,
              const float* zbias, float inv_tau, float qscale, const float* decay, float* state, const int* slots, const int* lens,
              int fresh, int B, int S, int H, int D, int V, float* out, cudaStream_t s);
// One token per sequence (S == 1): a block per 64 value columns of a (sequence, head); false when the key size does not fit.
bool gla_step(const void* q, const void* k, const void* v, int bf, long sb, const void* z, long z_sb, const float* zbias, float inv_tau,
              float qscale, const float* decay, float* state, const int* slots, const int* lens, int fresh, int B, int H, int D, int V,
              float* out, cudaStream_t s);
// Chunked form of gla_scan for long runs of tokens (gla_chunked.cu): blk = (b * H + h) * chunks + c indexes Qe, Ke, Bc [blk, C, D],
// G [blk, D], Vf [blk, C, V], A [blk, C, C] with C = gla_chunk_tokens(); Sl [blk, D, V] = Ke^T Vf goes through gla_carry.
int gla_chunk_tokens();
void gla_chunk_prep(const void* q, const void* k, const void* v, int bf, long sb, long st, const void* z, long z_sb, long z_st,
                    const float* zbias, float inv_tau, float qscale, const float* decay, const int* lens, int B, int S, int H, int D, int V,
                    int chunks, float* Qe, float* Ke, float* Bc, float* G, float* Vf, float* A, cudaStream_t s);
void gla_carry(float* Sl, const float* G, float* state, const int* slots, int fresh, int B, int chunks, int H, int D, int V,
               cudaStream_t s);
void rglru_scan(const void* u, int bf, const float* gr, const float* gi, int wb, const float* rbias, const float* ibias,
                const float* lam_sp, const void* y, long y_sb, long y_st, float* state, const int* slots, const int* lens, int fresh,
                int B, int S, int W, void* out, cudaStream_t s);
// z, u, g: pre-activations [B,S,W] sharing the strides sb, st; state float [slots, W]; out [B,S,W] contiguous
void mingru_scan(const void* z, const void* u, const void* g, int bf, long sb, long st, float* state, const int* slots, const int* lens,
                 int fresh, int B, int S, int W, void* out, cudaStream_t s);
void xielu(const void* x, void* out, int bf, long n, float ap, float an, cudaStream_t s);
void relu_sq(const void* x, void* out, int bf, long n, cudaStream_t s);
void gelu_erf(const void* x, void* out, int bf, long n, cudaStream_t s);
void silu_mul(const void* gu, void* out, int bf, long rows, int F, cudaStream_t s);
void clamped_glu(const void* gu, void* out, int bf, long rows, int F, float limit, float slope, cudaStream_t s);
void sigmoid_gate_mul(void* x, int bf, const void* gate, int gate_bf, long gate_stride, long rows, int C, int rep, cudaStream_t s);
void rotary_qkv_f32(const void* p, int bf, long p_sb, long p_st, int B, int S, int C, int hq, int hk, int D, int dims,
                    const float* inv_freq, const int* pos0, float q_scale, float k_scale, float* out, cudaStream_t s);
// act 0: none, 1: gelu_erf, 2: silu(gate rows . x) * (up rows . x) with the gate rows stacked over the up rows (O/2 outputs),
// 3: the square of relu
void indexed_gemv(const void* w, const int* sel, const void* x, int bf, long x_stride, int M, int E, int O, int I, int act, void* out,
                  cudaStream_t s);
void moe_combine(const void* rows, const int* src, const float* weight, const void* base, const float* base_weight, int bf, int N, int top,
                 int C, void* out, cudaStream_t s);
// false: more experts than the kernel takes (256)
bool route_topk(const float* logits, const float* correction, int N, int E, int top, int n_real, int kind, float scale, float* w, long* idx,
                float* ident, cudaStream_t s);
void small_linear_f32(const void* w, int w_bf, const void* x, int x_bf, long x_stride, int N, int O, int I, float* out, cudaStream_t s);
void embed_sinusoid(const long* tokens, const void* table, int bf, float scale, const float* inv_freq, const int* pos0, int B, int S, int W,
                    int vocab, float* out, cudaStream_t s);
// pairs (may be null): [buckets + 1, W] of the table's dtype; prev (may be null): int64 per slot; out_lp (may be null): table's dtype
void embed_bigram(const long* tokens, const void* table, int bf, float scale, const void* pairs, long buckets, long mul_prev, long mul_cur,
                  long* prev, const int* slots, const int* lens, int fresh, int B, int S, int W, int vocab, float* out, void* out_lp,
                  cudaStream_t s);
void group_rms_norm_gated(const void* x, int in_bf16, long x_stride, const void* gate, int gate_bf16, long gate_stride, const float* w,
                          int wn, int rows, int C, int groups, float eps, int gate_first, void* out, long out_stride, float out_scale,
                          int sigmoid_gate, cudaStream_t s);
// Grouped-query sliding-window attention (window_attention.cu); false: sizes do not fit (value size above 512).
// window_qk_prepare: norm_all 0: an RMS norm per head (qw, kw hold D numbers), 1: one over all heads (H*D and G*D numbers); inv_freq
// (dims/2 numbers, or null): rotation of the first dims coordinates; k null: only the queries are prepared.
// score_bias (one float per query head, or null): sigmoid(score + bias) weights, not normalised, instead of a softmax.
void window_qk_prepare(void* q, long q_sb, long q_st, void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st, int bf,
                       const float* qw, const float* kw, int norm_all, float eps, const float* inv_freq, int dims, const int* pos0,
                       const int* lens, const int* slots, void* kcache, void* vcache, int ring, int B, int S, int H, int G, int D, int V,
                       cudaStream_t s);
bool window_attention_prompt(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                             const void* gate, long g_sb, long g_st, int bf, const int* lens, int B, int S, int H, int G, int D, int V,
                             int window, float scale, float softcap, const float* score_bias, void* out, long out_stride, float out_scale,
                             cudaStream_t s);
bool window_prompt_mma_fits(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                            int D, int V, const void* out, long out_stride);
void window_prompt_mma(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, const void* v, long v_sb, long v_st,
                       const void* gate, long g_sb, long g_st, const int* lens, int B, int S, int H, int G, int D, int V, int window,
                       float scale, float softcap, const float* score_bias, void* out, long out_stride, float out_scale, cudaStream_t s);
// part_m / part_l float [B, H, splits], part_acc float [B, H, splits, V] with splits = window_token_splits(...)
int window_token_splits(int ring, int B, int H, int G);
bool window_attention_token(const void* q, long q_sb, const void* kcache, const void* vcache, const void* gate, long g_sb, int bf,
                            const int* slots, const int* pos0, const int* lens, int ring, int B, int H, int G, int D, int V, int window,
                            float scale, float softcap, const float* score_bias, int splits, float* part_m, float* part_l, float* part_acc,
                            void* out, long out_stride, float out_scale, cudaStream_t s);
// Matrix-state recurrences with one decay per head and token (matrix_recurrence.cu); false: the state has too many rows.
bool gated_delta_scan(const void* q, const void* k, long qk_sb, long qk_st, const void* v, long v_sb, long v_st, int bf, const float* braw,
                      const float* araw, long ba_sb, long ba_st, const float* a_log, const float* dt_bias, float* state, const int* slots,
                      const int* lens, int fresh, int B, int S, int H, int G, int D, int V, float qscale, float* out, cudaStream_t s);
// The same rule with a decay per head and key channel: araw float [B,S,H,D] (strides a_sb, a_st), dt_bias [H*D].
bool gated_delta_channel_scan(const void* q, const void* k, long qk_sb, long qk_st, const void* v, long v_sb, long v_st, int bf,
                              const float* braw, long b_sb, long b_st, const float* araw, long a_sb, long a_st, const float* a_log,
                              const float* dt_bias, float* state, const int* slots, const int* lens, int fresh, int B, int S, int H, int G,
                              int D, int V, float qscale, float* out, cudaStream_t s);
bool ssd_scan(const void* x, long x_sb, long x_st, const void* bm, const void* cm, long bc_sb, long bc_st, int bf, const float* dtraw,
              long dt_sb, long dt_st, const float* a_log, const float* dt_bias, const float* dskip, float* state, const int* slots,
              const int* lens, int fresh, int B, int S, int H, int G, int N, int V, float* out, cudaStream_t s);

// Head-mixing attention (headmix_attention.cu, headmix_prefill.cu): queries mixed across heads into rows of G*D numbers, keys that
// double as values, a sink in the denominator, aligned chunks and / or a window.  ring > 0: single tokens against rings; 0: prompts.
void headmix_qk_prepare(const void* q, long q_sb, long q_st, const void* k, long k_sb, long k_st, int bf, const float* mixw, int dims,
                        const float* inv_freq, const int* pos0, const int* lens, const int* slots, void* kcache, void* vcache, int ring,
                        void* qmix, void* rows, int B, int S, int H, int G, int D, cudaStream_t s);
bool headmix_attend(const void* qmix, const void* keys, long key_sb, const void* vals, long v_sb, long v_stride, int bf, const float* sink,
                    const void* gate, long g_sb, long g_st, const int* slots, const int* pos0, const int* lens, int chunk, int window,
                    int ring, int B, int S, int H, int G, int D, void* out, long out_stride, cudaStream_t s);
// single tokens against the rings, all heads of a stretch of positions per block (headmix_decode.cu); part [B, stretches, H, D + 2] float
int headmix_token_stretches(int ring);
bool headmix_token_fits(int bf, int H, int G, int D, int ring, const void* qmix, const void* kcache, const void* vcache);
void headmix_token(const void* qmix, const void* kcache, const void* vcache, int bf, const float* sink, const void* gate, long g_sb,
                   const int* slots, const int* pos0, const int* lens, int chunk, int window, int ring, int B, int H, int G, int D,
                   float* part, void* out, long out_stride, cudaStream_t s);
bool headmix_prompt_mma_fits(const void* v, long v_sb, long v_st, int G, int D, const void* out, long out_stride);
void headmix_prompt_mma(const void* qmix, const void* keys, const void* v, long v_sb, long v_st, const float* sink, const void* gate,
                        long g_sb, long g_st, const int* lens, int B, int S, int H, int G, int D, int chunk, int window, void* out,
                        long out_stride, cudaStream_t s);

}  // namespace seqmix
