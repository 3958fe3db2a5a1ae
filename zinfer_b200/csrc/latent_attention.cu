// Latent attention keeps, per token, one row [c | k_rot]: a normed latent c of `rank` values from
// which every head's keys and values are linear maps, and `rd` rotated key values shared by all heads.
// With the key map folded into the query (q_lat = W_uk^T q_plain) the score of head h against a cached
// row is q_eff . row with q_eff = [q_lat | q_rot], and the head's output is W_uv applied to the
// softmax-weighted sum of the c parts: one cached row serves all heads, as keys and as values.
//
// This file holds the kernel that makes the cached row and the rotated query part from a token's
// projections; the attention over the rows is zi_paged_attention_v (attention_generic.cu) with one
// kv head whose values are the first `rank` columns of its keys.
#include "api.h"
#include "common.cuh"

namespace {
// One block per token.  q row: [heads, each (dim plain | rd rotated)]; kv row: [rank latent | rd key part].
// Rotary: of the rd values the first rot_dims are rotated, in pairs (i, i + rot_dims/2) or, with `neighbours`,
// in pairs (2i, 2i + 1); the rest pass.  The q row may be 32-bit or of the results' type; so may the kv row.
template <typename T>
__device__ __forceinline__ float turned(const T* x, int i, int rot_dims, int neighbours, const float* cs, const float* sn) {
  float v = to_f32(x[i]);
  if (i >= rot_dims) return v;
  const int half = rot_dims >> 1;
  if (neighbours) {
    const int p = i >> 1;
    float a = to_f32(x[2 * p]), b = to_f32(x[2 * p + 1]);
    rotate_pair(a, b, cs[p], sn[p]);
    return (i & 1) ? b : a;
  }
  if (i < half) {
    float a = v, b = to_f32(x[i + half]);
    rotate_pair(a, b, cs[i], sn[i]);
    return a;
  }
  float a = to_f32(x[i - half]), b = v;
  rotate_pair(a, b, cs[i - half], sn[i - half]);
  return b;
}

template <typename TQ, typename TS, typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const TQ* __restrict__ qsrc, int ldq, const TS* __restrict__ kvsrc, int ldkv, int heads, int dim, int rd,
                      int rank, int rot_dims, int neighbours, const float* __restrict__ cw, float eps,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_table_pos,
                      const int* __restrict__ positions, T* __restrict__ q_eff, T* __restrict__ cache,
                      const int* __restrict__ slots, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int D = rank + rd, half = rot_dims / 2;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= n_table_pos ? n_table_pos - 1 : pos);   // callers keep positions inside the table
  const float* cs = cos_t + (size_t)pos * half;
  const float* sn = sin_t + (size_t)pos * half;
  // the rotated part of every query head -> q_eff[t, h, rank ..]
  const TQ* qrow = qsrc + (size_t)t * ldq;
  for (int e = threadIdx.x; e < heads * rd; e += blockDim.x) {
    const int h = e / rd, i = e - h * rd;
    q_eff[((size_t)t * heads + h) * D + rank + i] =
        from_f32<T>(turned(qrow + (size_t)h * (dim + rd) + dim, i, rot_dims, neighbours, cs, sn));
  }
  if (!write_cache) return;
  const int slot = slots[t];
  if (slot < 0) return;      // a row that pads a captured batch
  const TS* kv = kvsrc + (size_t)t * ldkv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32(kv[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  T* out = cache + (size_t)slot * D;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) out[i] = from_f32<T>(norm_scale(to_f32(kv[i]), cw[i], inv));
  for (int i = threadIdx.x; i < rd; i += blockDim.x) out[rank + i] = from_f32<T>(turned(kv + rank, i, rot_dims, neighbours, cs, sn));
}

// A request's cached rows, gathered from its pages for the tensor-core products of a prompt's portion:
// keys[j, :] = row j (all D columns; rows kv_len .. kv_pad-1 are zero) and values_t[r, j] = row j's
// column r for r < rank (the latent part, transposed: the second product's weight-side operand), every
// value twice in a row ([rank, 2 kv_pad]: columns 2j and 2j+1 hold key j) because the softmax weights come
// as a high and a low part side by side; a prefix of 2k columns then serves the first k keys.
// One block takes 32 keys.
template <typename T>
__global__ void __launch_bounds__(256)
latent_gather_kernel(T* __restrict__ keys, T* __restrict__ values_t, const T* __restrict__ cache,
                     const int* __restrict__ block_table, int page_size, int kv_len, int kv_pad, int D, int rank,
                     int kv_start, int kv_first) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char raw[];
  T* tile = reinterpret_cast<T*>(raw);           // [32][D + 2]
  // row j of the outputs is the key at position kv_start + j; positions before kv_first (behind every window) are zero
  const int j0 = blockIdx.x * 32, pitch = D + 2;
  for (int e = threadIdx.x; e < 32 * D; e += blockDim.x) {
    const int kk = e / D, c = e - kk * D, j = j0 + kk;
    T v = from_f32<T>(0.f);
    if (j < kv_len && kv_start + j >= kv_first) {
      const int at = kv_start + j;
      const int page = block_table[at / page_size];
      if (page >= 0) v = cache[((size_t)page * page_size + (at % page_size)) * D + c];
    }
    tile[kk * pitch + c] = v;
    if (j < kv_pad) keys[(size_t)j * D + c] = v;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 32 * rank; e += blockDim.x) {
    const int r = e / 32, kk = e - r * 32, j = j0 + kk;
    if (j < kv_pad) {
      values_t[(size_t)r * 2 * kv_pad + 2 * j] = tile[kk * pitch + r];
      values_t[(size_t)r * 2 * kv_pad + 2 * j + 1] = tile[kk * pitch + r];
    }
  }
}

// Causal softmax over a portion's scores: row (t, h) of S [rows, kv_pad] (32-bit) belongs to the query at
// position ctx + t and sees keys 0 .. ctx + t; p = exp(scale * (S - max)) / sum there, 0 beyond (also in
// the padding columns).  The weights are 32-bit; for the second product each is written as two values of
// the activations' type, P[row, 2j] = round(p) and P[row, 2j+1] = round(p - P[row, 2j]), whose sum
// carries 16 bits of p, so that the product loses nothing a 32-bit weight would have kept.
template <typename T>
__global__ void __launch_bounds__(256)
causal_softmax_kernel(T* __restrict__ P, const float* __restrict__ S, int heads, int ctx, int kv_pad, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int visible = ctx + (int)(row / heads) + 1;
  const float* s = S + row * kv_pad;
  T* p = P + row * 2 * kv_pad;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < visible; j += blockDim.x) m = fmaxf(m, s[j]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  float sum = 0.f;
  for (int j = threadIdx.x; j < visible; j += blockDim.x) sum += expf(scale * (s[j] - m));
  const float inv = 1.0f / block_sum(sum, scratch);
  for (int j = threadIdx.x; j < kv_pad; j += blockDim.x) {
    const float w = j < visible ? expf(scale * (s[j] - m)) * inv : 0.f;
    const T hi = from_f32<T>(w);
    p[2 * j] = hi;
    p[2 * j + 1] = from_f32<T>(w - to_f32(hi));
  }
}

// The same with a window and a learned sink: column j of S is the key at position key0 + j; the query of row (t, h) at
// position pos0 + t sees the keys max(0, pos - window + 1) .. pos (window 0: all up to pos); exp(sink_logit[h]) joins
// the denominator (null: none).
template <typename T>
__global__ void __launch_bounds__(256)
window_softmax_kernel(T* __restrict__ P, const float* __restrict__ S, int heads, int pos0, int key0, int n_cols, int window,
                      float scale, const float* __restrict__ sink_logit) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const int pos = pos0 + (int)(row / heads), h = (int)(row % heads);
  const int lo = max(0, (window > 0 ? max(0, pos - window + 1) : 0) - key0), hi = min(n_cols, pos - key0 + 1);
  const float* s = S + row * n_cols;
  T* p = P + row * 2 * n_cols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY;
  for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) m = fmaxf(m, s[j]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  m *= scale;
  if (sink_logit) m = fmaxf(m, sink_logit[h]);
  float sum = 0.f;
  for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) sum += expf(scale * s[j] - m);
  sum = block_sum(sum, scratch);
  if (sink_logit) sum += expf(sink_logit[h] - m);
  const float inv = 1.0f / sum;
  for (int j = threadIdx.x; j < n_cols; j += blockDim.x) {
    const float w = j >= lo && j < hi ? expf(scale * s[j] - m) * inv : 0.f;
    const T hi_part = from_f32<T>(w);
    p[2 * j] = hi_part;
    p[2 * j + 1] = from_f32<T>(w - to_f32(hi_part));
  }
}

// ------------------------------------------------------------ single tokens: split-key decode
// A request that brings one token: its `heads` query rows [D] against its kv_len cached rows, which
// every head shares.  Block (key split, request, group of 16 heads): 256 threads walk the split's keys
// in tiles of 32 rows held in shared memory as 32-bit values; a row is fetched once for all heads of
// the group, as key (all D columns) and as value (the first `rank`).  32-bit arithmetic throughout.
//   scores   thread (warp w, lane) holds S[2w][key lane] and S[2w+1][key lane]
//   softmax  per head over the tile by warp shuffles, running maximum and sum per head
//   output   thread t owns columns (t % 128) + 128 j of heads (t / 128) * 8 .. + 7
// With more than one split the block leaves (maximum, sum, unnormalised output) per head in `work`
// [request][split][head][rank + 2] and latent_decode_merge adds the splits in order.
constexpr int LD_HEADS = 16, LD_KEYS = 32, LD_THREADS = 256, LD_MAXC = 5;   // rank <= 128 * LD_MAXC

template <typename T>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_kernel(T* __restrict__ out, int out_stride, float* __restrict__ work, const T* __restrict__ q, int q_stride,
                     const T* __restrict__ cache, const int* __restrict__ block_tables, int bt_stride,
                     const int* __restrict__ cu_q, const int* __restrict__ kv_lens, const int* __restrict__ dec_seq,
                     int heads, int D, int rank, int page_size, float scale, int splits, int window,
                     const float* __restrict__ sink_logit) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* qs = sm;                              // [LD_HEADS][D]
  const int KP = D + 4;                        // row pitch of ks: 16-byte accesses, no bank conflicts between rows
  float* ks = qs + LD_HEADS * D;               // [LD_KEYS][KP]
  float* ps = ks + LD_KEYS * KP;               // [LD_HEADS][LD_KEYS]
  float* al = ps + LD_HEADS * LD_KEYS;         // [LD_HEADS] rescale of this tile
  const int split = blockIdx.x, seq = dec_seq[blockIdx.y], h0 = blockIdx.z * LD_HEADS;
  const int nh = min(LD_HEADS, heads - h0);
  const int tok = cu_q[seq], kv_len = kv_lens[seq];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_tables + (size_t)seq * bt_stride;
  const bool vec8 = sizeof(T) == 2 && D % 8 == 0 && ((uintptr_t)cache & 15) == 0;
  // this split's keys: whole tiles, dealt out evenly; with a window the token sees its last `window` keys only
  const int kv_begin = window > 0 ? max(0, kv_len - window) : 0;
  const int first_tile = kv_begin / LD_KEYS;
  const int tiles = (kv_len + LD_KEYS - 1) / LD_KEYS - first_tile;
  const int per = (tiles + splits - 1) / splits;
  const int t_begin = first_tile + split * per, t_end = min(first_tile + tiles, t_begin + per);

  for (int h = warp; h < LD_HEADS; h += LD_THREADS / 32) {       // a warp per query row
    const T* qr = q + (size_t)tok * q_stride + (size_t)(h0 + h) * D;
    for (int c = lane; c < D; c += 32) qs[h * D + c] = h < nh ? to_f32(qr[c]) : 0.f;
  }
  const int ha = 2 * warp, hb = 2 * warp + 1;          // the two heads whose scores this thread forms
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int col = tid & 127, hg = (tid >> 7) * 8;       // output columns col + 128 j of heads hg .. hg + 7
  float acc[8][LD_MAXC];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < LD_MAXC; ++j) acc[i][j] = 0.f;

  for (int tile = t_begin; tile < t_end; ++tile) {
    const int k0 = tile * LD_KEYS;
    __syncthreads();     // the tile before is consumed (the first time: qs is written)
    for (int kk = warp; kk < LD_KEYS; kk += LD_THREADS / 32) {      // a warp per cached row: one page lookup
      const int j = k0 + kk;
      const int page = j < kv_len && j >= kv_begin ? bt[j / page_size] : -1;     // (pages behind the window may be gone)
      float* dst = ks + kk * KP;
      if (page < 0) {
        for (int c = lane; c < D; c += 32) dst[c] = 0.f;
      } else {
        const T* row = cache + ((size_t)page * page_size + (j % page_size)) * D;
        if (vec8) {        // 16 bytes a lane
          for (int c = lane * 8; c < D; c += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            *reinterpret_cast<float4*>(dst + c) = make_float4(__low2float(p2[0]), __high2float(p2[0]), __low2float(p2[1]), __high2float(p2[1]));
            *reinterpret_cast<float4*>(dst + c + 4) = make_float4(__low2float(p2[2]), __high2float(p2[2]), __low2float(p2[3]), __high2float(p2[3]));
          }
        } else {
          for (int c = lane; c < D; c += 32) dst[c] = to_f32(row[c]);
        }
      }
    }
    __syncthreads();
    float sa = 0.f, sb = 0.f;
    {
      const float4* kr = reinterpret_cast<const float4*>(ks + lane * KP);
      const float4* qa = reinterpret_cast<const float4*>(qs + ha * D);
      const float4* qb = reinterpret_cast<const float4*>(qs + hb * D);
      for (int c = 0; c < D / 4; ++c) {       // D is a multiple of 4 (checked by the launcher)
        const float4 kv = kr[c], a4 = qa[c], b4 = qb[c];
        sa = fmaf(a4.x, kv.x, fmaf(a4.y, kv.y, fmaf(a4.z, kv.z, fmaf(a4.w, kv.w, sa))));
        sb = fmaf(b4.x, kv.x, fmaf(b4.y, kv.y, fmaf(b4.z, kv.z, fmaf(b4.w, kv.w, sb))));
      }
    }
    const bool live = k0 + lane < kv_len && k0 + lane >= kv_begin;
    sa = live ? sa * scale : -INFINITY;
    sb = live ? sb * scale : -INFINITY;
    const float na = fmaxf(m_a, warp_max(sa)), nb = fmaxf(m_b, warp_max(sb));    // finite: a tile has a live key
    const float pa = live ? expf(sa - na) : 0.f, pb = live ? expf(sb - nb) : 0.f;
    const float ra = expf(m_a - na), rb = expf(m_b - nb);                        // exp(-inf) = 0 the first time
    l_a = l_a * ra + warp_sum(pa);
    l_b = l_b * rb + warp_sum(pb);
    m_a = na;
    m_b = nb;
    ps[ha * LD_KEYS + lane] = pa;
    ps[hb * LD_KEYS + lane] = pb;
    if (lane == 0) {
      al[ha] = ra;
      al[hb] = rb;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float r = al[hg + i];
#pragma unroll
      for (int j = 0; j < LD_MAXC; ++j) acc[i][j] *= r;
    }
    for (int kk = 0; kk < LD_KEYS; ++kk) {
      float v[LD_MAXC];
#pragma unroll
      for (int j = 0; j < LD_MAXC; ++j) v[j] = col + 128 * j < rank ? ks[kk * KP + col + 128 * j] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p = ps[(hg + i) * LD_KEYS + kk];
#pragma unroll
        for (int j = 0; j < LD_MAXC; ++j) acc[i][j] = fmaf(p, v[j], acc[i][j]);
      }
    }
  }
  // running maximum and sum of every head, for the threads that own its columns
  __syncthreads();
  if (lane == 0) {
    ps[ha] = m_a;
    ps[hb] = m_b;
    ps[LD_HEADS + ha] = l_a;
    ps[LD_HEADS + hb] = l_b;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int h = hg + i;
    if (h >= nh) continue;
    const float mh = ps[h], lh = ps[LD_HEADS + h];
    if (splits == 1) {
      // a learned sink: exp(sink_logit[head]) in the denominator, without a value
      const float inv = 1.0f / (sink_logit ? lh + expf(sink_logit[h0 + h] - mh) : lh);
      T* o = out + (size_t)tok * out_stride + (size_t)(h0 + h) * rank;
#pragma unroll
      for (int j = 0; j < LD_MAXC; ++j)
        if (col + 128 * j < rank) o[col + 128 * j] = from_f32<T>(acc[i][j] * inv);
    } else {
      float* w = work + (((size_t)blockIdx.y * splits + split) * heads + (h0 + h)) * (rank + 2);
      if (col == 0) {
        w[0] = mh;      // -inf and 0 when the split had no keys
        w[1] = lh;
      }
#pragma unroll
      for (int j = 0; j < LD_MAXC; ++j)
        if (col + 128 * j < rank) w[2 + col + 128 * j] = acc[i][j];
    }
  }
}

// out[token, head, :] = sum over splits of exp(m_s - m) O_s / sum over splits of exp(m_s - m) l_s, splits in order.
template <typename T>
__global__ void latent_decode_merge_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ work,
                                           const int* __restrict__ cu_q, const int* __restrict__ dec_seq, int heads,
                                           int rank, int splits, const float* __restrict__ sink_logit) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int tok = cu_q[dec_seq[r]];
  const float* w = work + ((size_t)r * splits * heads + h) * (rank + 2);
  const size_t stride = (size_t)heads * (rank + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, w[s * stride]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) l += w[s * stride + 1] * expf(w[s * stride] - m);
  if (sink_logit) l += expf(sink_logit[h] - m);
  const float inv = 1.0f / l;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) o = fmaf(w[s * stride + 2 + c], expf(w[s * stride] - m), o);
    out[(size_t)tok * out_stride + (size_t)h * rank + c] = from_f32<T>(o * inv);
  }
}
}  // namespace

extern "C" long long zi_latent_decode_workspace_floats(int n_dec, int heads, int rank, int splits) {
  return splits > 1 ? (long long)n_dec * splits * heads * (rank + 2) : 0;
}

extern "C" int zi_latent_decode(void* out, int out_stride, float* work, const void* q, int q_stride, int dtype,
                                const void* cache, const int* block_tables, int bt_stride, const int* cu_q,
                                const int* kv_lens, const int* dec_seq, int n_dec, int heads, int D, int rank,
                                int page_size, float scale, int splits, cudaStream_t stream) {
  return zi_latent_decode_mods(out, out_stride, work, q, q_stride, dtype, cache, block_tables, bt_stride, cu_q, kv_lens, dec_seq,
                               n_dec, heads, D, rank, page_size, scale, splits, 0, nullptr, stream);
}

// The same with a window (a token sees its last `window` keys; 0: all) and a learned sink per head (sink_logit [heads],
// exp of it in the denominator; null: none).
extern "C" int zi_latent_decode_mods(void* out, int out_stride, float* work, const void* q, int q_stride, int dtype,
                                     const void* cache, const int* block_tables, int bt_stride, const int* cu_q,
                                     const int* kv_lens, const int* dec_seq, int n_dec, int heads, int D, int rank,
                                     int page_size, float scale, int splits, int window, const float* sink_logit,
                                     cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (window < 0) return zi_refuse("latent_decode: a window of %d keys", window);
  if (rank > 128 * LD_MAXC || rank > D) return zi_refuse("latent_decode: a latent of %d values (rows of %d) is more than this kernel holds", rank, D);
  if (splits < 1 || (splits > 1 && !work)) return zi_refuse("latent_decode: %d splits need a workspace", splits);
  if (D % 4) return zi_refuse("latent_decode: rows of %d values are not whole 16-byte pieces", D);
  const size_t smem = (size_t)(LD_HEADS * D + LD_KEYS * (D + 4) + LD_HEADS * LD_KEYS + LD_HEADS) * sizeof(float);
  dim3 grid(splits, n_dec, (heads + LD_HEADS - 1) / LD_HEADS);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    auto kern = latent_decode_kernel<TT>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return zi_refuse("latent_decode: cannot get %zu bytes of shared memory", smem);
    zi_launch(kern, dim3(grid), dim3(LD_THREADS), smem, stream, (TT*)out, out_stride, work, (const TT*)q, q_stride,
              (const TT*)cache, block_tables, bt_stride, cu_q, kv_lens, dec_seq, heads, D, rank, page_size, scale, splits, window,
              sink_logit);
    if (splits > 1)
      zi_launch(latent_decode_merge_kernel<TT>, dim3(n_dec, heads), dim3(128), 0, stream, (TT*)out, out_stride,
                (const float*)work, cu_q, dec_seq, heads, rank, splits, sink_logit);
  });
  return zi_check_launch("latent_decode");
}

extern "C" int zi_latent_gather(void* keys, void* values_t, const void* cache, int dtype, const int* block_table,
                                int page_size, int kv_len, int kv_pad, int D, int rank, cudaStream_t stream) {
  return zi_latent_gather_from(keys, values_t, cache, dtype, block_table, page_size, kv_len, kv_pad, D, rank, 0, 0, stream);
}

// The same for the kv_len keys from position kv_start on; positions before kv_first are left zero (their pages may be gone).
extern "C" int zi_latent_gather_from(void* keys, void* values_t, const void* cache, int dtype, const int* block_table,
                                     int page_size, int kv_len, int kv_pad, int D, int rank, int kv_start, int kv_first,
                                     cudaStream_t stream) {
  if (kv_pad <= 0) return 0;
  if (kv_start < 0) return zi_refuse("latent_gather: keys from position %d", kv_start);
  if (rank > D || kv_len > kv_pad) return zi_refuse("latent_gather: rank %d of %d columns, %d of %d keys", rank, D, kv_len, kv_pad);
  const size_t smem = (size_t)32 * (D + 2) * (dtype == ZI_F32 ? 4 : 2);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    auto kern = latent_gather_kernel<TT>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return zi_refuse("latent_gather: cannot get %zu bytes of shared memory", smem);
    zi_launch(kern, dim3((kv_pad + 31) / 32), dim3(256), smem, stream, (TT*)keys, (TT*)values_t, (const TT*)cache,
              block_table, page_size, kv_len, kv_pad, D, rank, kv_start, kv_first);
  });
  return zi_check_launch("latent_gather");
}

extern "C" int zi_causal_softmax(void* P, const float* S, int dtype, long long rows, int heads, int ctx, int kv_pad,
                                 float scale, cudaStream_t stream) {
  if (rows <= 0 || kv_pad <= 0) return 0;
  if (rows > 0x7fffffffLL) return zi_refuse("causal_softmax: too many rows");
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(causal_softmax_kernel<TT>, dim3((unsigned)rows), dim3(256), 0, stream, (TT*)P, S,
                                         heads, ctx, kv_pad, scale));
  return zi_check_launch("causal_softmax");
}

extern "C" int zi_window_softmax(void* P, const float* S, int dtype, long long rows, int heads, int pos0, int key0, int n_cols,
                                 int window, float scale, const float* sink_logit, cudaStream_t stream) {
  if (rows <= 0 || n_cols <= 0) return 0;
  if (rows > 0x7fffffffLL) return zi_refuse("window_softmax: too many rows");
  if (!(scale > 0.f)) return zi_refuse("window_softmax: the scale must be positive");
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(window_softmax_kernel<TT>, dim3((unsigned)rows), dim3(256), 0, stream, (TT*)P, S,
                                         heads, pos0, key0, n_cols, window, scale, sink_logit));
  return zi_check_launch("window_softmax");
}

extern "C" int zi_latent_prepare(const void* src, int ld, int dtype, int T, int heads, int dim, int rd, int rank,
                                 int rot_dims, const float* cw, float eps, const float* cos_t, const float* sin_t,
                                 int n_table_pos, const int* positions, void* q_eff, void* cache, const int* slots,
                                 int write_cache, cudaStream_t stream) {
  const size_t elt = dtype == ZI_F32 ? 4 : 2;
  return zi_latent_prepare_rows(src, ld, dtype, (const char*)src + (size_t)heads * (dim + rd) * elt, ld, dtype, dtype, T, heads,
                                dim, rd, rank, rot_dims, 0, cw, eps, cos_t, sin_t, n_table_pos, positions, q_eff, cache, slots,
                                write_cache, stream);
}

// The same with the queries and the [latent | key part] rows in tensors of their own (queries that come from a
// projection of their own), each 32-bit or of the results' type, and with the rotation's pairs either (i, i + half)
// or, with `neighbours`, (2i, 2i + 1).
extern "C" int zi_latent_prepare_rows(const void* q, int ldq, int q_dtype, const void* kv, int ldkv, int kv_dtype, int out_dtype,
                                      int T, int heads, int dim, int rd, int rank, int rot_dims, int neighbours,
                                      const float* cw, float eps, const float* cos_t, const float* sin_t, int n_table_pos,
                                      const int* positions, void* q_eff, void* cache, const int* slots, int write_cache,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > rd) return zi_refuse("latent_prepare: %d rotated dimensions of %d", rot_dims, rd);
  if (n_table_pos <= 0 && rot_dims > 0) return zi_refuse("latent_prepare: the rotary table is empty");
#define ZI_LP(TQ, TS, TT)                                                                                               \
  zi_launch(latent_prepare_kernel<TQ, TS, TT>, dim3(T), dim3(128), 0, stream, (const TQ*)q, ldq, (const TS*)kv, ldkv, heads, \
            dim, rd, rank, rot_dims, neighbours, cw, eps, cos_t, sin_t, n_table_pos, positions, (TT*)q_eff, (TT*)cache, slots, \
            write_cache)
  using bf = __nv_bfloat16;
  if (out_dtype == ZI_F32 && q_dtype == ZI_F32 && kv_dtype == ZI_F32) ZI_LP(float, float, float);
  else if (out_dtype == ZI_BF16 && q_dtype == ZI_BF16 && kv_dtype == ZI_BF16) ZI_LP(bf, bf, bf);
  else if (out_dtype == ZI_BF16 && q_dtype == ZI_BF16 && kv_dtype == ZI_F32) ZI_LP(bf, float, bf);
  else if (out_dtype == ZI_BF16 && q_dtype == ZI_F32 && kv_dtype == ZI_F32) ZI_LP(float, float, bf);
  else return zi_refuse("latent_prepare: sources of types %d and %d cannot become results of type %d", q_dtype, kv_dtype, out_dtype);
#undef ZI_LP
  return zi_check_launch("latent_prepare");
}

ZI_TRACE_SETTER(latent_attention)
