// Causal attention of query tokens against the paged cache, for any mix of prompt
// portions and single decoded tokens, any head size up to 256 in steps of 2, any
// number of heads and groups, with an optional window that may also keep a request's
// first tokens visible (keep_first).  32-bit arithmetic on the
// CUDA cores (exact expf); the storage type alone differs between the float32 path
// and the plain bfloat16 path.  A query row visits its keys in ascending order in
// tiles aligned to multiples of BK, so its result does not depend on how the
// request was cut into steps or on what else is in the batch.
//
// Grid: (query tile of BQ tokens of one request, query head).  Pages are
// [page][kv head][offset][d]; the key at position j of request s lies in page
// block_tables[s][j / page_size] at offset j % page_size.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int BQ = 16, BK = 32, THREADS = 128, ROWS_PER_WARP = BQ / (THREADS / 32);

// Values may have another size than keys and may lie in the key rows themselves (a latent cache whose row
// serves as key and, in its first dv columns, as value): dv value columns are read from rows of
// v_row elements in `vcache`; the output has dv columns per head.  MAXJ * 32 bounds dv.
// With a window, query i sees key j <= i if i - j < window or j < keep_first.
// Changes to the score, each off unless given: softcap c (s <- c tanh(s / c) after the scale), dist_bias
// [heads][n_dist] (a bias by the distance i - j, distances from n_dist - 1 on share the last entry; added after
// the cap), sink_logit [heads] (exp(sink_logit[h]) joins head h's denominator; it has no value).
template <typename T, int MAXJ>
__global__ void __launch_bounds__(THREADS)
paged_attention_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q, int q_stride,
                       const T* __restrict__ kcache, const T* __restrict__ vcache,
                       const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                       const int* __restrict__ kv_lens, const int* __restrict__ tile_seq,
                       const int* __restrict__ tile_q0, int nq, int nkv, int d, int page_size, int window,
                       float scale, int dv, int v_row, int skip_from, int skip_single, float sink, int keep_first,
                       const float* __restrict__ sink_logit, float softcap, const float* __restrict__ dist_bias,
                       int n_dist) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  float* Qs = smem;                   // [BQ][d]
  float* Ks = Qs + BQ * d;            // [BK][d+1]
  float* Vs = Ks + BK * (d + 1);      // [BK][dv]
  float* Ss = Vs + BK * dv;           // [BQ][BK]

  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int h = blockIdx.y, kvh = h / (nq / nkv);
  const int tok0 = cu_q[seq], qlen = cu_q[seq + 1] - tok0, kvlen = kv_lens[seq];
  const int ctx = kvlen - qlen;  // tokens of this request already in the cache before this step
  const int nqv = min(BQ, qlen - q0);
  if (nqv <= 0 || (skip_from > 0 && qlen >= skip_from) || (skip_single && qlen == 1)) return;
  const int first_pos = ctx + q0, last_pos = first_pos + nqv - 1;
  const int kv_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int kv_end = last_pos + 1;
  // keys [0, keep_end) lie before the window and stay visible; the tiles between them and the window are skipped
  const int keep_end = window > 0 ? min(keep_first, kv_begin) : 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_tables + (size_t)seq * bt_stride;

  for (int e = tid; e < BQ * d; e += THREADS) {
    const int r = e / d, c = e % d;
    Qs[e] = r < nqv ? to_f32(q[(size_t)(tok0 + q0 + r) * q_stride + (size_t)h * d + c]) : 0.f;
  }

  float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][MAXJ];
#pragma unroll
  for (int i = 0; i < ROWS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) acc[i][j] = 0.f;
  }

  for (int kt = keep_end > 0 ? 0 : (kv_begin / BK) * BK; kt < kv_end; kt += BK) {
    if (kt >= keep_end && kt + BK <= kv_begin) {   // a tile wholly between the kept first tokens and the window
      kt = (kv_begin / BK) * BK - BK;
      continue;
    }
    __syncthreads();  // previous tile fully consumed (also orders the Q load the first time)
    for (int e = tid; e < BK * d; e += THREADS) {
      const int kk = e / d, c = e % d;
      const int j = kt + kk;
      float kval = 0.f;
      if ((j >= kv_begin || j < keep_end) && j < kv_end) {
        const int page = bt[j / page_size];
        if (page >= 0) kval = to_f32(kcache[(((size_t)page * nkv + kvh) * page_size + (j % page_size)) * d + c]);
      }
      Ks[kk * (d + 1) + c] = kval;
    }
    for (int e = tid; e < BK * dv; e += THREADS) {
      const int kk = e / dv, c = e % dv;
      const int j = kt + kk;
      float vval = 0.f;
      if ((j >= kv_begin || j < keep_end) && j < kv_end) {
        const int page = bt[j / page_size];
        if (page >= 0) vval = to_f32(vcache[(((size_t)page * nkv + kvh) * page_size + (j % page_size)) * v_row + c]);
      }
      Vs[e] = vval;
    }
    __syncthreads();

    float alpha[ROWS_PER_WARP];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
      const int r = warp * ROWS_PER_WARP + i;
      alpha[i] = 1.f;
      if (r >= nqv) continue;  // uniform within the warp
      const int pos = first_pos + r, j = kt + lane;
      const float* qr = Qs + r * d;
      const float* kr = Ks + lane * (d + 1);
      float s = 0.f;
      for (int c = 0; c < d; ++c) s = fmaf(qr[c], kr[c], s);
      s *= scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      const bool visible = j <= pos && (window <= 0 || j > pos - window || j < keep_first);
      if (!visible) s = -INFINITY;
      else if (dist_bias) s += dist_bias[(size_t)h * n_dist + min(pos - j, n_dist - 1)];   // not scaled, not capped
      const float m_new = fmaxf(m[i], warp_max(s));
      float p = 0.f;
      if (m_new != -INFINITY) {
        p = visible ? expf(s - m_new) : 0.f;
        alpha[i] = expf(m[i] - m_new);  // exp(-inf) = 0 on the first visible tile
      }
      l[i] = l[i] * alpha[i] + warp_sum(p);
      m[i] = m_new;
      Ss[r * BK + lane] = p;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
      const int r = warp * ROWS_PER_WARP + i;
      if (r >= nqv) continue;
#pragma unroll
      for (int j = 0; j < MAXJ; ++j) acc[i][j] *= alpha[i];
      for (int kk = 0; kk < BK; ++kk) {
        const float p = Ss[r * BK + kk];
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
          const int c = lane + 32 * j;
          if (c < dv) acc[i][j] = fmaf(p, Vs[kk * dv + c], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS_PER_WARP; ++i) {
    const int r = warp * ROWS_PER_WARP + i;
    if (r >= nqv) continue;
    // a sink: `sink` keys whose score is 0 and which have no value, counted in the denominator only
    // a learned sink: exp(sink_logit[h]) in the denominator, neither scaled nor capped
    const float inv = 1.0f / (sink_logit ? l[i] + expf(sink_logit[h] - m[i]) : (sink > 0.f ? l[i] + sink * expf(-m[i]) : l[i]));
    T* o = out + (size_t)(tok0 + q0 + r) * out_stride + (size_t)h * dv;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int c = lane + 32 * j;
      if (c < dv) o[c] = from_f32<T>(acc[i][j] * inv);
    }
  }
}
}  // namespace

extern "C" int zi_paged_attention_tile_rows() { return BQ; }

extern "C" int zi_paged_attention(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                  const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                  const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                  int n_tiles, int nq, int nkv, int d, int page_size, int window, float scale,
                                  cudaStream_t stream) {
  return zi_paged_attention_v(out, out_stride, q, q_stride, dtype, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                              tile_seq, tile_q0, n_tiles, nq, nkv, d, d, d, page_size, window, scale, 0, 0, stream);
}

extern "C" int zi_paged_attention_v(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                    const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                    const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                    int n_tiles, int nq, int nkv, int d, int dv, int v_row, int page_size, int window,
                                    float scale, int skip_from, int skip_single, cudaStream_t stream) {
  return zi_paged_attention_sink(out, out_stride, q, q_stride, dtype, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                                 tile_seq, tile_q0, n_tiles, nq, nkv, d, dv, v_row, page_size, window, scale, skip_from,
                                 skip_single, 0.f, stream);
}

extern "C" int zi_paged_attention_sink(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                       const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                       const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                       int n_tiles, int nq, int nkv, int d, int dv, int v_row, int page_size, int window,
                                       float scale, int skip_from, int skip_single, float sink, cudaStream_t stream) {
  return zi_paged_attention_mask(out, out_stride, q, q_stride, dtype, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                                 tile_seq, tile_q0, n_tiles, nq, nkv, d, dv, v_row, page_size, window, 0, scale, skip_from,
                                 skip_single, sink, stream);
}

// The general form: a sink, values of any size (dv columns of rows of v_row elements), and a window that
// keeps the first keep_first tokens of a request visible.
extern "C" int zi_paged_attention_mask(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                       const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                       const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                       int n_tiles, int nq, int nkv, int d, int dv, int v_row, int page_size, int window,
                                       int keep_first, float scale, int skip_from, int skip_single, float sink,
                                       cudaStream_t stream) {
  return zi_paged_attention_mods(out, out_stride, q, q_stride, dtype, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                                 tile_seq, tile_q0, n_tiles, nq, nkv, d, dv, v_row, page_size, window, keep_first, scale,
                                 skip_from, skip_single, sink, nullptr, 0.f, nullptr, 0, stream);
}

// The same with the changes to the score: a learned sink per head, a cap, a bias by distance.
extern "C" int zi_paged_attention_mods(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                       const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                       const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                       int n_tiles, int nq, int nkv, int d, int dv, int v_row, int page_size, int window,
                                       int keep_first, float scale, int skip_from, int skip_single, float sink,
                                       const float* sink_logit, float softcap, const float* dist_bias, int n_dist,
                                       cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!(softcap >= 0.f)) return zi_refuse("paged_attention: the cap on the scores must not be negative");
  if (dist_bias && n_dist <= 0) return zi_refuse("paged_attention: a bias by distance needs a table");
  if (sink_logit && sink != 0.f) return zi_refuse("paged_attention: a learned sink and a counted sink exclude each other");
  if (keep_first < 0) return zi_refuse("paged_attention: %d kept first tokens", keep_first);
  if (!(sink >= 0.f)) return zi_refuse("paged_attention: the sink's weight must not be negative");
  constexpr int WIDE = 20;   // value columns up to 640 (latent caches); 8 serves every ordinary head size
  if (d <= 0 || d > 32 * WIDE) return zi_refuse("paged_attention: head_dim %d is outside 1..%d", d, 32 * WIDE);
  if (dv <= 0 || dv > 32 * WIDE || v_row < dv) return zi_refuse("paged_attention: %d value columns of rows of %d, keys of %d", dv, v_row, d);
  if (nkv <= 0 || nq % nkv) return zi_refuse("paged_attention: %d query heads do not divide into %d kv heads", nq, nkv);
  if (page_size <= 0) return zi_refuse("paged_attention: page_size %d", page_size);
  const size_t smem = (size_t)(BQ * d + BK * (d + 1) + BK * dv + BQ * BK) * sizeof(float);
  dim3 grid(n_tiles, nq);
#define ZI_LAUNCH_ATTN(J)                                                                                          \
  do {                                                                                                             \
    auto kern = paged_attention_kernel<TT, J>;                                                                     \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      if (e != cudaSuccess) return zi_refuse("paged_attention: cannot get %zu bytes of shared memory", smem);      \
    }                                                                                                              \
    zi_launch(kern, dim3(grid), dim3(THREADS), smem, stream, (TT*)out, out_stride, (const TT*)q, q_stride,         \
              (const TT*)kcache, (const TT*)vcache, block_tables, bt_stride, cu_q, kv_lens, tile_seq, tile_q0, nq, \
              nkv, d, page_size, window, scale, dv, v_row, skip_from, skip_single, sink, keep_first, sink_logit,    \
              softcap, dist_bias, n_dist);                                                                         \
  } while (0)
  ZI_DISPATCH_DTYPE(dtype, TT, {
    if (dv <= 256) ZI_LAUNCH_ATTN(8);
    else ZI_LAUNCH_ATTN(WIDE);
  });
#undef ZI_LAUNCH_ATTN
  return zi_check_launch("paged_attention");
}

ZI_TRACE_SETTER(attention_generic)
