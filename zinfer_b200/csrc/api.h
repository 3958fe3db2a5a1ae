// C entry points of the kernel library.  Pointers are device pointers; `stream` is
// the CUDA stream the caller works on.  Each returns 0 on success, a cudaError_t
// (> 0) if the launch failed, or -1 if it refuses the sizes, with the reason in
// zi_last_error().  dtype tags: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* zi_last_error();

int zi_embed_gather(float* h, const void* table, int table_dtype, const int* ids, int T, int H, int V,
                    cudaStream_t stream);
// h[t] = scale * table[ids[t]] + bigram[row], row = (previous token * mul_prev + token * mul_cur) mod buckets, or row
// `buckets` for a request's first token (position 0).  The token before a step's first token of a request comes from
// last_token[state_slots[request]], which is then set to the request's last token of this step.
int zi_embed_bigram(float* h, const void* table, const void* bigram, int table_dtype, const int* ids, const int* positions,
                    const int* cu_q, const int* state_slots, int* last_token, int n_seqs, int T, int H, int V, float scale,
                    int buckets, long long mul_prev, long long mul_cur, cudaStream_t stream);
int zi_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_partials, int splits,
                   long long split_stride, const float* w, float eps, void* out, int out_dtype, const int* rows,
                   int n_rows, int H, cudaStream_t stream);
int zi_add_rmsnorm_scaled(float* h, const void* delta, int delta_dtype, const float* delta_partials, int splits,
                          long long split_stride, float delta_scale, const float* bias, const float* w, float eps,
                          void* out, int out_dtype, const int* rows, int n_rows, int H, cudaStream_t stream);
int zi_residual_add(float* h, const void* delta, int delta_dtype, long long n, cudaStream_t stream);
int zi_residual_add_scaled(float* h, const void* delta, int delta_dtype, float delta_scale, long long n,
                           cudaStream_t stream);
int zi_scale_f32(float* x, long long n, float s, cudaStream_t stream);
int zi_sigmoid_gate(void* out, int ldo, const void* x, int ldx, const void* g, int ldg, int dtype, int T, int width,
                    cudaStream_t stream);
// act: 0 silu, 1 the tanh form of gelu
int zi_gated_act(void* out, const void* gu, int dtype, int T, int I, int interleave, int act, cudaStream_t stream);
int zi_gated_act_partials(void* out, int dtype, const float* partials, int splits, long long split_stride, int T, int I,
                          int interleave, int act, cudaStream_t stream);
int zi_residual_add_partials(float* h, const float* partials, int splits, long long split_stride, long long n,
                             cudaStream_t stream);
int zi_patch_tokens(int* ids, const int* prev, const int* dst, const int* src, int n, cudaStream_t stream);
int zi_swiglu(void* out, const void* gu, int dtype, int T, int I, int interleave, cudaStream_t stream);
int zi_swiglu_partials(void* out, int dtype, const float* partials, int splits, long long split_stride, int T, int I,
                       int interleave, cudaStream_t stream);
int zi_gemm_tcgen05_swiglu(void* out, int out_dtype, const void* x, const void* w, int M, int N2, int K, int ldx,
                           int ldw, int ldo, int sm_count, cudaStream_t stream);
int zi_gemm_tcgen05_gated(void* out, int out_dtype, const void* x, const void* w, int M, int N2, int K, int ldx,
                          int ldw, int ldo, int act, int sm_count, cudaStream_t stream);
int zi_gemm_argmax_units(int N);
int zi_gemm_tcgen05_argmax(float* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw, int ldo,
                           float* cand_val, int* cand_idx, int sm_count, cudaStream_t stream);
int zi_rope_table(float* cos_t, float* sin_t, int n_pos, int d, float theta, cudaStream_t stream);
int zi_qk_norm_rope_store(const void* src, int dtype, int T, int src_stride, const float* partials, int splits,
                          long long split_stride, void* q_out, int q_stride, int nq, int nkv, int d, const float* qw,
                          const float* kw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                          const int* positions, void* kcache, void* vcache, const int* slots, int page_size,
                          int write_kv, cudaStream_t stream);

int zi_gemm_simt(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, int M, int N,
                 int K, int ldx, int ldw, int ldo, cudaStream_t stream);

// Batched (`batch` products sx/sw/so/sb elements apart) and grouped (per-tile weight group, gathered rows, sizes on
// the device) forms of the CUDA-core product; epilogue 0: none, 1: square of relu; tile_rows 16 or 64.
int zi_gemm_simt_general(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, int M, int N,
                         int K, int ldx, int ldw, int ldo, int batch, long long sx, long long sw, long long so,
                         const float* bias, long long sb, const int* row_src, const int* tile_group,
                         const int* n_tiles_dev, long long group_stride, int epilogue, int tile_rows,
                         cudaStream_t stream);

// Recurrent mixers: state [slots][taps][C] float32 (taps-1 carried inputs of the convolution, then S).
int zi_causal_conv(float* u, const void* x, int ldx, int dtype, const float* xb, const float* kern, const float* cb,
                   const float* state, int C, int taps, const int* cu_q, const int* state_slots, int n_seqs, int T,
                   cudaStream_t stream);
int zi_rglru_scan(void* out, int ldo, const float* u, const float* gates, int block_width, const float* rb,
                  const float* ib, const float* lam, float decay_scale, const void* y, int ldy, const float* yb,
                  const void* x, int ldx, const float* xb, int dtype, float* state, int C, int taps, const int* cu_q,
                  const int* state_slots, int n_seqs, cudaStream_t stream);

// The same recurrence in chunks of `chunk` tokens of the flat batch (four small kernels; sums associated per chunk).
long long zi_rglru_chunked_workspace_floats(int T, int C, int n_seqs, int chunk);
int zi_rglru_scan_chunked(void* out, int ldo, float* work, const float* u, const float* gates, int block_width,
                          const float* rb, const float* ib, const float* lam, float decay_scale, const void* y, int ldy,
                          const float* yb, const void* x, int ldx, const float* xb, int dtype, float* state, int C,
                          int taps, const int* cu_q, const int* state_slots, int n_seqs, int T, int chunk,
                          cudaStream_t stream);
// One token per request: convolution, gates, recurrence and gated output in one kernel.  yx rows: y branch, x branch.
int zi_rglru_decode(void* out, int ldo, const void* yx, int ld, int dtype, const float* yb, const float* xb,
                    const float* kern, const float* cb, const void* wg, int wg_dtype, int block_width, const float* rb,
                    const float* ib, const float* lam, float decay_scale, float* state, int C, int taps,
                    const int* state_slots, int n_seqs, cudaStream_t stream);

int zi_gemm_tcgen05_supported(const void* x, const void* w, int K, int ldx, int ldw);
long long zi_gemm_tcgen05_plan(int M, int N, int K, int sm_count, int* plan);
int zi_gemm_tcgen05(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K, int ldx, int ldw,
                    int ldo, float* workspace, long long workspace_bytes, int sm_count, int defer_reduce,
                    cudaStream_t stream);
// Grouped tensor-core product: every 128 rows of x multiply with one group of the stacked weight [groups * N, K].
int zi_gemm_tcgen05_grouped(void* out, int out_dtype, const void* x, const void* w, int rows, int N, int K, int ldx,
                            int ldw, int ldo, int groups, const int* tile_group, int relu2, int sm_count,
                            cudaStream_t stream);
// One tensor-core product per head in one launch (activations and results of the heads side by side in their rows).
int zi_gemm_tcgen05_heads(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K, int ldx, int ldw,
                          int ldo, int groups, int x_group_cols, int out_group_cols, int sm_count, cudaStream_t stream);
int zi_gemm_tcgen05_status();
int zi_gemm_tcgen05_pair_enable(int on);

int zi_paged_attention_tile_rows();
int zi_paged_attention(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                       const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                       const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                       int d, int page_size, int window, float scale, cudaStream_t stream);

// The same with dv <= d value columns read from rows of v_row elements (values may lie in the key rows).
// skip_from > 0: requests that bring that many tokens or more are left out (another kernel serves them);
// skip_single: so are requests that bring exactly one.
int zi_paged_attention_v(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                         const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                         const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                         int d, int dv, int v_row, int page_size, int window, float scale, int skip_from,
                         int skip_single, cudaStream_t stream);
// The same with a sink: `sink` keys of score 0 without a value, counted in the softmax's denominator only.
int zi_paged_attention_sink(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                            const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                            const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                            int d, int dv, int v_row, int page_size, int window, float scale, int skip_from,
                            int skip_single, float sink, cudaStream_t stream);
// The general form: values of any size dv, and with a window the first keep_first tokens of a request stay visible.
int zi_paged_attention_mask(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                            const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                            const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                            int d, int dv, int v_row, int page_size, int window, int keep_first, float scale,
                            int skip_from, int skip_single, float sink, cudaStream_t stream);
// The same with changes to the score: sink_logit [heads] (exp(sink_logit[h]) joins head h's denominator), softcap c
// (s <- c tanh(s / c) after the scale), dist_bias [heads][n_dist] (added by the distance query - key, after the cap;
// distances from n_dist - 1 on share the last entry).  Each is off when null or 0.
int zi_paged_attention_mods(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* kcache,
                            const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                            const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                            int d, int dv, int v_row, int page_size, int window, int keep_first, float scale,
                            int skip_from, int skip_single, float sink, const float* sink_logit, float softcap,
                            const float* dist_bias, int n_dist, cudaStream_t stream);
// The tensor-core kernels (mma.sync, softmax weights as two bfloat16 parts) with the same changes to the score.
int zi_attention_prefill_mma_mods(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                                  const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                                  const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                                  int d, int page_size, int window, float scale, const float* sink_logit, float softcap,
                                  const float* dist_bias, int n_dist, cudaStream_t stream);
int zi_attention_decode_mma_mods(void* out, int out_stride, float* workspace, const void* q, int q_stride, const void* kcache,
                                 const void* vcache, long long n_pages, const int* block_tables, int bt_stride,
                                 const int* cu_q, const int* kv_lens, const int* dec_seq, int n_dec, int nq, int nkv, int d,
                                 int page_size, int window, float scale, int splits, const float* sink_logit, float softcap,
                                 const float* dist_bias, int n_dist, cudaStream_t stream);
// A fused projection row [q heads | k heads | v heads | gate]: biases, an RMS norm over all of q and over all of k
// (weights per element), rotation of the first rot_dims dimensions of every q and k head, q and the gate columns into
// tensors of their own, k and v into the token's page slot.  The source may be 32-bit beside 16-bit results.
int zi_qkv_rows_prepare(const void* src, int src_dtype, int src_stride, const float* bias, void* q_out, int q_stride,
                        void* gate_out, int gate_stride, int n_gate, int out_dtype, int T, int nq, int nkv, int d, int dv,
                        const float* qw, const float* kw, float eps, int rot_dims, const float* cos_t, const float* sin_t,
                        int n_table_pos, const int* positions, void* kcache, void* vcache, const int* slots, int page_size,
                        cudaStream_t stream);
// RMS norm of rows of activations: out[t] = x[t] * w / sqrt(mean(x[t]^2) + eps).
int zi_rmsnorm_rows(void* out, int ldo, int out_dtype, const void* x, int ldx, int x_dtype, const float* w, float eps, int T,
                    int n, cudaStream_t stream);
// cos/sin [n_pos, half] of pos * freq[i], both times `magnitude`.
int zi_rope_table_freqs(float* cos_t, float* sin_t, int n_pos, int half, const float* freq, float magnitude,
                        cudaStream_t stream);
int zi_sigmoid_gate_grouped(void* out, int ldo, const void* x, int ldx, const void* g, int ldg, int dtype, int T, int width,
                            int group, cudaStream_t stream);
// out = g' * sigmoid(alpha g') * (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit).
int zi_clamped_gate(void* out, int dtype, const void* gu, int gu_dtype, const float* partials, int splits,
                    long long split_stride, int T, int I, int interleave, float limit, float alpha, float shift,
                    cudaStream_t stream);
// q/k norm, rotation of the first rot_dims dimensions of a head, page write; values of their own or the keys as projected.
int zi_qk_prepare(const void* src, int dtype, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv, int d,
                  int rot_dims, const float* qw, const float* kw, float eps, const float* cos_t, const float* sin_t,
                  int n_table_pos, const int* positions, void* kcache, void* vcache, const int* slots, int page_size,
                  int v_from_k, int write_kv, cudaStream_t stream);
// The same with value heads of dv elements (rows [q heads of d | k heads of d | v heads of dv]).
int zi_qk_prepare_v(const void* src, int dtype, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv, int d,
                    int dv, int rot_dims, const float* qw, const float* kw, float eps, const float* cos_t, const float* sin_t,
                    int n_table_pos, const int* positions, void* kcache, void* vcache, const int* slots, int page_size,
                    int v_from_k, int write_kv, cudaStream_t stream);
int zi_rope_table_scaled(float* cos_t, float* sin_t, int n_pos, int d, float theta, float factor, cudaStream_t stream);
// h += norm(sa * a + sb * b) * w (the norm of a sublayer's output), x_out = h in the activations' type; a and b whole
// or as split-K partial sums [splits][T][H].
int zi_norm_residual(float* h, const void* a, int a_dtype, const float* a_part, int a_splits, long long a_zstride, float sa,
                     const void* b, int b_dtype, const float* b_part, int b_splits, long long b_zstride, float sb,
                     const float* w, float eps, void* x_out, int out_dtype, int T, int H, cudaStream_t stream);
// h += sum of up to four updates (whole or split-K partial sums, each with a multiplier) + bias; out1 = norm(h) * w1 and,
// with w2, out2 = norm(h) * w2 (both norms share the root mean square).  With rows: picked rows, h unchanged.
int zi_sum_norm_pair(float* h, int n_terms, const void* const* whole, const int* dtypes, const float* const* part,
                     const int* splits, const long long* zstride, const float* scales, const float* bias, const float* w1,
                     const float* w2, float eps, void* out1, void* out2, int out_dtype, const int* rows, int n_rows, int H,
                     cudaStream_t stream);
int zi_cast_rows(void* out, int out_dtype, const float* h, long long n, cudaStream_t stream);
int zi_relu2(void* x, int dtype, long long n, cudaStream_t stream);
// Mixers with a matrix-valued state per head (linear attention with decays, with or without the delta rule).
int zi_short_conv(float* y, int ldy, const void* x, int ldx, int dtype, const float* kern, const float* tail,
                  long long slot_stride, int C, int taps, int act, const int* cu_q, const int* state_slots, int n_seqs,
                  int T, cudaStream_t stream);
int zi_short_conv_carry(float* tail, long long slot_stride, const void* x, int ldx, int dtype, int C, int taps,
                        const int* cu_q, const int* state_slots, int n_seqs, cudaStream_t stream);
int zi_decay(float* z, long long rows, int N, int D, const float* bias, const float* a_log, float inv_tau, int mode,
             cudaStream_t stream);
int zi_unit_norm(float* x, int ld, int T, int heads, int d, float eps, float scale, cudaStream_t stream);
int zi_sigmoid_rows(float* out, int ldo, const void* x, int ldx, int dtype, int rows, int W, cudaStream_t stream);
int zi_linear_recurrence(float* out, int ldo, const void* q, int ldq, const void* k, int ldk, int qk_dtype, const void* v,
                         int ldv, int v_dtype, const float* decay, int ldg, const float* beta, int ldb, float q_scale,
                         float* state, long long slot_stride, int H, int G, int D, int V, int delta, const int* cu_q,
                         const int* state_slots, int n_seqs, cudaStream_t stream);
int zi_head_norm_gate(void* out, int out_dtype, int ldo, const float* o, int ldi, const float* w, float eps,
                      const void* gate, int gate_dtype, int ldgate, int act, int T, int heads, int V, cudaStream_t stream);
int zi_moe_router_grouped(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype, int T,
                          int K, int NR, int top, int renormalize, int score_kind, int groups, int keep, float wscale,
                          cudaStream_t stream);
int zi_moe_route_grouped(int* chosen, float* weight, const float* logits, int T, int NR, int top, int renormalize,
                         int score_kind, int groups, int keep, float wscale, cudaStream_t stream);
// The same two with a correction [NR] added to the scores for the choice only (null: none).
int zi_moe_router_grouped_c(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype,
                            const float* correction, int T, int K, int NR, int top, int renormalize, int score_kind,
                            int groups, int keep, float wscale, cudaStream_t stream);
int zi_moe_route_grouped_c(int* chosen, float* weight, const float* logits, const float* correction, int T, int NR, int top,
                           int renormalize, int score_kind, int groups, int keep, float wscale, cudaStream_t stream);
// Latent attention: the cached row [normed latent | rotated key part] and the rotated query part of a token.
// Router by the logits themselves: z = W x + bias, the `top` largest chosen, weights = softmax over the chosen logits.
int zi_moe_router_top_logits(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype,
                             const float* bias, int T, int K, int NR, int top, cudaStream_t stream);
int zi_moe_route_top_logits(int* chosen, float* weight, const float* logits, const float* bias, int T, int NR, int top,
                            cudaStream_t stream);
int zi_latent_prepare(const void* src, int ld, int dtype, int T, int heads, int dim, int rd, int rank, int rot_dims,
                      const float* cw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                      const int* positions, void* q_eff, void* cache, const int* slots, int write_cache,
                      cudaStream_t stream);
// For a prompt's portion on the tensor cores: a request's cached rows gathered ([kv_pad, D], and the first `rank`
// columns transposed [rank, kv_pad]), and the causal softmax of the portion's score matrix.
int zi_latent_decode_mods(void* out, int out_stride, float* work, const void* q, int q_stride, int dtype, const void* cache,
                          const int* block_tables, int bt_stride, const int* cu_q, const int* kv_lens, const int* dec_seq,
                          int n_dec, int heads, int D, int rank, int page_size, float scale, int splits, int window,
                          const float* sink_logit, cudaStream_t stream);
int zi_latent_gather_from(void* keys, void* values_t, const void* cache, int dtype, const int* block_table, int page_size,
                          int kv_len, int kv_pad, int D, int rank, int kv_start, int kv_first, cudaStream_t stream);
// Softmax over a block's scores with a window and a learned sink; the weights as two parts, like zi_causal_softmax.
int zi_window_softmax(void* P, const float* S, int dtype, long long rows, int heads, int pos0, int key0, int n_cols, int window,
                      float scale, const float* sink_logit, cudaStream_t stream);
int zi_latent_prepare_rows(const void* q, int ldq, int q_dtype, const void* kv, int ldkv, int kv_dtype, int out_dtype, int T,
                           int heads, int dim, int rd, int rank, int rot_dims, int neighbours, const float* cw, float eps,
                           const float* cos_t, const float* sin_t, int n_table_pos, const int* positions, void* q_eff,
                           void* cache, const int* slots, int write_cache, cudaStream_t stream);
int zi_latent_gather(void* keys, void* values_t, const void* cache, int dtype, const int* block_table, int page_size,
                     int kv_len, int kv_pad, int D, int rank, cudaStream_t stream);
int zi_causal_softmax(void* P, const float* S, int dtype, long long rows, int heads, int ctx, int kv_pad, float scale,
                      cudaStream_t stream);
// Requests that bring one token: split-key attention over the latent rows, all heads of a group per fetched row.
long long zi_latent_decode_workspace_floats(int n_dec, int heads, int rank, int splits);
int zi_latent_decode(void* out, int out_stride, float* work, const void* q, int q_stride, int dtype, const void* cache,
                     const int* block_tables, int bt_stride, const int* cu_q, const int* kv_lens, const int* dec_seq,
                     int n_dec, int heads, int D, int rank, int page_size, float scale, int splits, cudaStream_t stream);
// Mixture of experts: choice and weights per token, the pairs laid out by expert, the weighted sum.
int zi_moe_route(int* chosen, float* weight, const float* logits, const float* correction, int T, int NR, int top,
                 int renormalize, cudaStream_t stream);
int zi_moe_router(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype,
                  const float* correction, int T, int K, int NR, int top, int renormalize, cudaStream_t stream);
int zi_moe_few_rows(void* out, int out_dtype, int ldo, const void* x, int dtype, int ldx, const void* w,
                    const int* row_src, const int* tile_group, const int* n_tiles_dev, int max_tiles, int N, int K,
                    int relu2, cudaStream_t stream);
int zi_moe_align(const int* chosen, int P, int top, int E, int tile_rows, int cap_tiles, int* row_token, int* row_self,
                 int* pair_row, int* tile_expert, int* n_tiles, cudaStream_t stream);
int zi_gather_rows(void* out, const void* x, int dtype, const int* row_src, int rows, int width, int ldx,
                   cudaStream_t stream);
int zi_moe_combine(void* out, const float* y, const void* x, int dtype, const int* chosen, const float* weight,
                   const int* pair_row, int T, int top, int E, int H, cudaStream_t stream);

int zi_attention_prefill_tile_rows();
int zi_attention_mma_supported(int nq, int nkv, int d, int decode);
int zi_attention_prefill_mma(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                             const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                             const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                             int d, int page_size, int window, float scale, cudaStream_t stream);
int zi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, const void* q, int q_stride,
                                           const void* kcache, const void* vcache);
int zi_attention_prefill_tcgen05(void* out, int out_stride, const void* q, int q_stride, int n_tokens,
                                 const void* kcache, const void* vcache, long long n_pages, const int* block_tables,
                                 int bt_stride, const int* cu_q, const int* kv_lens, const int* tile_seq,
                                 const int* tile_q0, int n_tiles, int nq, int nkv, int d, int page_size, int window,
                                 float scale, cudaStream_t stream);
// Both with the softmax weights as two bfloat16 parts where they meet the values, and a sink in the denominator.
int zi_attention_prefill_mma_sink(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                                  const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                                  const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                                  int d, int page_size, int window, float scale, float sink, cudaStream_t stream);
int zi_attention_decode_mma_sink(void* out, int out_stride, float* workspace, const void* q, int q_stride,
                                 const void* kcache, const void* vcache, long long n_pages, const int* block_tables,
                                 int bt_stride, const int* cu_q, const int* kv_lens, const int* dec_seq, int n_dec, int nq,
                                 int nkv, int d, int page_size, int window, float scale, int splits, float sink,
                                 cudaStream_t stream);
// The two kernels with a sink and a window that keeps a request's first keep_first tokens visible.
int zi_attention_prefill_mma_mask(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                                  const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                                  const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles, int nq, int nkv,
                                  int d, int page_size, int window, int keep_first, float scale, float sink,
                                  cudaStream_t stream);
int zi_attention_decode_mma_mask(void* out, int out_stride, float* workspace, const void* q, int q_stride, const void* kcache,
                                 const void* vcache, long long n_pages, const int* block_tables, int bt_stride,
                                 const int* cu_q, const int* kv_lens, const int* dec_seq, int n_dec, int nq, int nkv, int d,
                                 int page_size, int window, int keep_first, float scale, int splits, float sink,
                                 cudaStream_t stream);
long long zi_attention_decode_workspace_floats(int n_dec, int nq, int nkv, int d, int splits);
int zi_attention_decode_mma(void* out, int out_stride, float* workspace, const void* q, int q_stride,
                            const void* kcache, const void* vcache, long long n_pages, const int* block_tables, int bt_stride,
                            const int* cu_q, const int* kv_lens, const int* dec_seq, int n_dec, int nq, int nkv, int d,
                            int page_size, int window, float scale, int splits, cudaStream_t stream);

int zi_attention_decode_fused(void* out, int out_stride, float* workspace, const void* qkv, int qkv_stride,
                              const float* partials, int part_splits, long long part_zstride, const float* qw,
                              const float* kw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                              const int* positions, const int* slots, void* kcache, void* vcache, long long n_pages,
                              const int* block_tables, int bt_stride, const int* cu_q, const int* kv_lens,
                              const int* dec_seq, int n_dec, int nq, int nkv, int d, int page_size, int window,
                              float scale, int splits, cudaStream_t stream);

int zi_argmax_chunks(int R, int V);
int zi_argmax(int* out, const float* logits, int R, int V, int ld, void* workspace, cudaStream_t stream);
int zi_argmax_candidates(int* out, const float* cand_val, const int* cand_idx, int R, int units, cudaStream_t stream);
int zi_sample_ctas_per_row(int R, int sm_count);
int zi_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* rep, const float* pres, const float* freq,
              const int* count_rows, int* counts, const unsigned long long* seeds, const int* draw_index,
              cudaStream_t stream);
int zi_count_tokens(int* counts, const int* tokens, int n, int V, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
