// Routing of a mixture of experts: scores and choice per token, the layout of the chosen
// (token, expert) pairs for the grouped products, and the weighted sum of the experts' outputs.
// The grouped products themselves are zi_gemm_simt_general (gemm_simt.cu).  All arithmetic is 32-bit.
//
// A router has NR outputs: the first E are experts with weights, the last NR - E stand for
// "identity experts" whose output is their input.  Scores are a softmax over all NR outputs; the
// choice adds a correction per output to the score, the weight of a chosen expert is its score
// without the correction, optionally divided by the sum of the chosen scores.
#include <algorithm>
#include <cstdlib>
#include "api.h"
#include "common.cuh"

namespace {
constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}


// One warp per token.  Sums run over a fixed order of lanes, so a token's choice does not depend on
// the batch.  Ties go to the lower index.  z: the token's NR logits; score, pick: NR floats each of
// shared memory for this warp.
__device__ __forceinline__ void route_token(int* __restrict__ chosen, float* __restrict__ weight, const float* z,
                                            float* score, float* pick, const float* __restrict__ correction, int t,
                                            int NR, int top, int renormalize, int lane) {
  float m = -INFINITY;
  for (int j = lane; j < NR; j += 32) m = fmaxf(m, z[j]);
  m = warp_max(m);
  float sum = 0.f;
  for (int j = lane; j < NR; j += 32) {
    const float e = expf(z[j] - m);
    score[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int j = lane; j < NR; j += 32) {
    const float s = score[j] * inv;
    score[j] = s;
    pick[j] = s + (correction ? correction[j] : 0.f);
  }
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = lane; j < NR; j += 32) {
      const float v = pick[j];
      if (v > best) {      // ascending j: the first of equal values stays
        best = v;
        arg = j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    if (arg == 0x7fffffff) arg = 0;    // every remaining value is -inf or NaN
    const float s = score[arg];
    total += s;
    if (lane == 0) {
      chosen[(size_t)t * top + k] = arg;
      weight[(size_t)t * top + k] = s;
      pick[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0) {
    const float r = 1.0f / total;
    for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= r;
  }
}

// The choice among groups of neighbouring outputs: scores are sigmoid(z) (score_kind 1) or a softmax (0); the
// outputs form `groups` equal groups, a group's score is the sum of its two largest scores, and only outputs
// of the `keep` best groups can be chosen; the weight of a chosen output is its score times wscale, divided
// by the chosen scores' sum first if `renormalize`.  Ties go to the lower index.  A correction [NR], when given,
// is added to the scores wherever they are compared (groups and outputs), never to the weights.  score, pick,
// gsc: NR floats each of shared memory for this warp.
__device__ __forceinline__ void route_token_grouped(int* __restrict__ chosen, float* __restrict__ weight, const float* z,
                                                    float* score, float* pick, float* gsc, int t, int NR, int top,
                                                    int renormalize, int score_kind, int groups, int keep,
                                                    float wscale, int lane, const float* __restrict__ corr = nullptr) {
  if (score_kind == 1) {
    for (int j = lane; j < NR; j += 32) score[j] = 1.0f / (1.0f + expf(-z[j]));
  } else {
    float m = -INFINITY;
    for (int j = lane; j < NR; j += 32) m = fmaxf(m, z[j]);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < NR; j += 32) {
      const float e = expf(z[j] - m);
      score[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int j = lane; j < NR; j += 32) score[j] *= inv;
  }
  __syncwarp();
  const int per = NR / groups;
  for (int g = lane; g < groups; g += 32) {      // the two largest scores of the group
    float a = -INFINITY, b = -INFINITY;
    for (int i = 0; i < per; ++i) {
      const float v = score[g * per + i] + (corr ? corr[g * per + i] : 0.f);
      if (v > a) { b = a; a = v; }
      else if (v > b) b = v;
    }
    gsc[g] = per > 1 ? a + b : a;
  }
  __syncwarp();
  for (int j = lane; j < NR; j += 32) pick[j] = -INFINITY;
  __syncwarp();
  for (int n = 0; n < keep; ++n) {               // the best groups, one after the other
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int g = lane; g < groups; g += 32) {
      const float v = gsc[g];
      if (v > best) { best = v; arg = g; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) break;                // uniform: nothing is left
    for (int i = lane; i < per; i += 32) pick[arg * per + i] = score[arg * per + i] + (corr ? corr[arg * per + i] : 0.f);
    if (lane == 0) gsc[arg] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = lane; j < NR; j += 32) {
      const float v = pick[j];
      if (v > best) { best = v; arg = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;
    const float s = score[arg];
    total += s;
    if (lane == 0) {
      chosen[(size_t)t * top + k] = arg;
      weight[(size_t)t * top + k] = s * wscale;
      pick[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0) {
    const float r = 1.0f / total;
    for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= r;
  }
}

// The choice by the logits themselves: z + bias, the `top` largest chosen (ties to the lower index), and the
// weights are the softmax over the chosen logits only.  score: NR floats of shared memory for this warp.
__device__ __forceinline__ void route_token_top_logits(int* __restrict__ chosen, float* __restrict__ weight, const float* z,
                                                       float* score, const float* __restrict__ bias, int t, int NR, int top,
                                                       int lane) {
  for (int j = lane; j < NR; j += 32) score[j] = z[j] + (bias ? bias[j] : 0.f);
  __syncwarp();
  float first = 0.f, total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = lane; j < NR; j += 32) {
      const float v = score[j];
      if (v > best) { best = v; arg = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;
    if (k == 0) first = best;                 // the largest: the softmax's reference
    const float e = expf(best - first);
    total += e;
    if (lane == 0) {
      chosen[(size_t)t * top + k] = arg;
      weight[(size_t)t * top + k] = e;
      score[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float r = 1.0f / total;
    for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= r;
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_top_logits_kernel(int* __restrict__ chosen, float* __restrict__ weight, const float* __restrict__ logits,
                            const float* __restrict__ bias, int T, int NR, int top) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  route_token_top_logits(chosen, weight, logits + (size_t)t * NR, sm + (size_t)warp * NR, bias, t, NR, top, lane);
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_grouped_kernel(int* __restrict__ chosen, float* __restrict__ weight, const float* __restrict__ logits, int T,
                         int NR, int top, int renormalize, int score_kind, int groups, int keep, float wscale,
                         const float* __restrict__ correction) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* score = sm + (size_t)warp * 3 * NR;
  route_token_grouped(chosen, weight, logits + (size_t)t * NR, score, score + NR, score + 2 * NR, t, NR, top, renormalize,
                      score_kind, groups, keep, wscale, lane, correction);
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(int* __restrict__ chosen, float* __restrict__ weight, const float* __restrict__ logits,
                 const float* __restrict__ correction, int T, int NR, int top, int renormalize) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* score = sm + (size_t)warp * 2 * NR;   // softmax scores
  route_token(chosen, weight, logits + (size_t)t * NR, score, score + NR, correction, t, NR, top, renormalize, lane);
}

// The router's product and the choice in one kernel.  A block takes TOK tokens (the launcher below gives it one): their
// rows in shared memory as 32-bit values, a warp per router output at a time (lanes stride over the weight row; a token's
// partial sums meet in a fixed order that depends neither on the other tokens nor on the number of warps), then a
// warp per token chooses.  Prompts run blocks of 8 warps; a decode step runs up to 32 warps per token, one output
// each (23 -> 15 us for 8 tokens, 32 outputs, rows of 4,096).  32-bit multiply-adds whatever the operands' types.
// MODE 1: the choice among groups of outputs (route_token_grouped) instead of the softmax with a correction (0);
// MODE 2: the choice by the logits plus a bias with a softmax over the chosen (route_token_top_logits).
template <typename TX, typename TW, int MODE, int TOK, bool WIDE>
__global__ void __launch_bounds__(WIDE ? 1024 : 256)
moe_router_kernel(int* __restrict__ chosen, float* __restrict__ weight, const TX* __restrict__ x, int ldx,
                  const TW* __restrict__ w, const float* __restrict__ correction, int T, int K, int NR, int top,
                  int renormalize, int score_kind, int groups, int keep, float wscale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* xs = sm;                        // [TOK][K]
  float* zs = sm + (size_t)TOK * K;      // per token: [NR] logits, then [NR] scores, [NR] picks, [NR] group scores
  const int t0 = blockIdx.x * TOK, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int n_tok = min(TOK, T - t0);
  for (int i = 0; i < n_tok; ++i)
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[(size_t)i * K + k] = to_f32(x[(size_t)(t0 + i) * ldx + k]);
  __syncthreads();
  const bool vec = K % 4 == 0 && ((uintptr_t)w & 15) == 0;      // 8- or 16-byte pieces of a weight row
  for (int j = warp; j < NR; j += warps) {
    const TW* wr = w + (size_t)j * K;
    float acc[TOK];
    if (vec) {
      // four pieces of the row in flight per lane; a token's four partial sums meet in a fixed order
      float part[TOK][4];
#pragma unroll
      for (int i = 0; i < TOK; ++i) part[i][0] = part[i][1] = part[i][2] = part[i][3] = 0.f;
      int k = lane * 4;
      for (; k + 384 < K; k += 512) {
        float4 wv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) wv[u] = load4(wr + k + 128 * u);
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
          if (i < n_tok) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)i * K + k + 128 * u);
              part[i][u] = fmaf(xv.x, wv[u].x, fmaf(xv.y, wv[u].y, fmaf(xv.z, wv[u].z, fmaf(xv.w, wv[u].w, part[i][u]))));
            }
          }
        }
      }
      for (; k < K; k += 128) {
        const float4 wv = load4(wr + k);
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
          if (i < n_tok) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)i * K + k);
            part[i][0] = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, part[i][0]))));
          }
        }
      }
#pragma unroll
      for (int i = 0; i < TOK; ++i) acc[i] = (part[i][0] + part[i][1]) + (part[i][2] + part[i][3]);
    } else {
#pragma unroll
      for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
      for (int k = lane; k < K; k += 32) {
        const float wv = to_f32(wr[k]);
#pragma unroll
        for (int i = 0; i < TOK; ++i)
          if (i < n_tok) acc[i] = fmaf(xs[(size_t)i * K + k], wv, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
      if (i < n_tok) {        // uniform in the block
        const float v = warp_sum(acc[i]);
        if (lane == 0) zs[(size_t)i * 4 * NR + j] = v;
      }
    }
  }
  __syncthreads();
  for (int i = warp; i < n_tok; i += warps) {
    float* z = zs + (size_t)i * 4 * NR;
    if (MODE == 2)
      route_token_top_logits(chosen, weight, z, z + NR, correction, t0 + i, NR, top, lane);     // `correction` carries the bias
    else if (MODE == 1)
      route_token_grouped(chosen, weight, z, z + NR, z + 2 * NR, z + 3 * NR, t0 + i, NR, top, renormalize, score_kind, groups,
                          keep, wscale, lane, correction);
    else
      route_token(chosen, weight, z, z + NR, z + 2 * NR, correction, t0 + i, NR, top, renormalize, lane);
  }
}

// Few rows per expert (a decode step): out[r, n] = act(sum_k x[row_src[r], k] * w[e][n][k]) for the rows r of
// tile `blockIdx.y` (16 rows, one expert e).  A block takes groups of 16 output columns, a warp two of each: its lanes stream
// the weight rows once, in pieces of VEC values (16 bytes where the row length allows: 8 bfloat16 or 4 floats,
// else 8 bytes), four pieces of a lane in flight together, with the hint that they are not read again, and
// multiply them with the tile's rows in use (they come first in a tile), which lie in shared memory as 32-bit
// values, a chunk of columns at a time (as long as the rows in use leave room for).  With pieces of 8 values a row's chunk lies in shared memory in blocks of
// 256 columns whose halves of every piece are 128 floats apart, so that a warp's 16-byte reads meet no bank
// twice.  The weights are read once per tile: bound by memory, not by multiply-adds.  Needs K % 4 == 0.  Every
// output is one sum in a fixed order (lane-strided, then the lanes' partial sums), independent of the batch.
constexpr int FR_ROWS = 16, FR_WARPS = 8, FR_PER_WARP = 2, FR_COLS = FR_WARPS * FR_PER_WARP, FR_CHUNK = 1024, FR_UNROLL = 4;

template <typename T, int VEC> struct FewPiece;
template <> struct FewPiece<float, 4> {
  using Raw = float4;
  static __device__ __forceinline__ Raw ld(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void unpack(const Raw& r, float* o) { o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = r.w; }
};
__device__ __forceinline__ void few_unpack2(uint32_t raw, float* o) {
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw);
  o[0] = __low2float(a);
  o[1] = __high2float(a);
}
template <> struct FewPiece<__nv_bfloat16, 4> {
  using Raw = uint2;
  static __device__ __forceinline__ Raw ld(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ void unpack(const Raw& r, float* o) { few_unpack2(r.x, o); few_unpack2(r.y, o + 2); }
};
template <> struct FewPiece<__nv_bfloat16, 8> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw ld(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ void unpack(const Raw& r, float* o) {
    few_unpack2(r.x, o); few_unpack2(r.y, o + 2); few_unpack2(r.z, o + 4); few_unpack2(r.w, o + 6);
  }
};

// where column k of a row's chunk lies in shared memory (k a multiple of 4)
template <int VEC>
__device__ __forceinline__ int few_place(int k) {
  if (VEC == 4) return k;
  const int kk = k & 255;
  return (k & ~255) + ((kk & 4) << 5) + ((kk >> 3) << 2);      // half of the piece * 128 + lane * 4
}

// The block's work for a tile with at most R rows in use (R fixed when compiled, so that a tile of one or two rows
// carries no arithmetic or tests for sixteen).
template <typename TX, typename TW, typename TO, int VEC, int R>
__device__ __forceinline__ void few_rows_run(TO* __restrict__ out, int ldo, const TX* __restrict__ x, int ldx,
                                             const TW* __restrict__ wbase, const int* src, int used, int r0, int N, int K,
                                             int relu2, int col_groups, float* xs) {
  using Piece = FewPiece<TW, VEC>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int STEP = 32 * VEC;            // columns a warp takes at a time
  // the fewer rows are in use, the longer the chunk of each that fits: with up to four rows of 4,096 columns one pass
  const int chunk = max(FR_CHUNK, (FR_ROWS * FR_CHUNK / used) & ~255);
  const bool one_pass = chunk >= K;         // the rows are staged once and serve every column group of the block
  for (int cg = 0; cg < col_groups; ++cg) {
    const int nb = (blockIdx.x * col_groups + cg) * FR_COLS;
    if (nb >= N) break;
    const int n0 = nb + warp * FR_PER_WARP;
    const TW* wr[FR_PER_WARP];
#pragma unroll
    for (int j = 0; j < FR_PER_WARP; ++j) wr[j] = wbase + (size_t)(n0 + j < N ? n0 + j : 0) * K;
    float acc[FR_PER_WARP][R];
#pragma unroll
    for (int j = 0; j < FR_PER_WARP; ++j)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[j][r] = 0.f;
    for (int k0 = 0; k0 < K; k0 += chunk) {
      const int kc = min(chunk, K - k0);
      if (!(one_pass && cg > 0)) {
        __syncthreads();     // the chunk before is consumed
        for (int e = threadIdx.x * 4; e < used * kc; e += blockDim.x * 4) {
          const int r = e / kc, k = e - r * kc;
          *reinterpret_cast<float4*>(xs + r * chunk + few_place<VEC>(k)) = load4(x + (size_t)src[r] * ldx + k0 + k);
        }
        __syncthreads();
      }
      for (int kb = 0; kb < kc; kb += FR_UNROLL * STEP) {
        typename Piece::Raw raw[FR_UNROLL][FR_PER_WARP];
#pragma unroll
        for (int u = 0; u < FR_UNROLL; ++u) {     // every piece of this round is asked for before the first is used
          const int k = kb + u * STEP + lane * VEC;
#pragma unroll
          for (int j = 0; j < FR_PER_WARP; ++j)
            if (k < kc) raw[u][j] = Piece::ld(wr[j] + k0 + k);
        }
#pragma unroll
        for (int u = 0; u < FR_UNROLL; ++u) {
          const int k = kb + u * STEP + lane * VEC;
          if (k >= kc) continue;
          float wv[FR_PER_WARP][VEC];
#pragma unroll
          for (int j = 0; j < FR_PER_WARP; ++j) Piece::unpack(raw[u][j], wv[j]);
          const float* xk = xs + (VEC == 4 ? k : (kb + u * STEP) + lane * 4);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            if (R <= 2 || r < used) {       // with R of 1 or 2 every row is in use
#pragma unroll
              for (int h = 0; h < VEC / 4; ++h) {
                const float4 xv = *reinterpret_cast<const float4*>(xk + r * chunk + h * 128);
#pragma unroll
                for (int j = 0; j < FR_PER_WARP; ++j)
                  acc[j][r] = fmaf(wv[j][4 * h], xv.x, fmaf(wv[j][4 * h + 1], xv.y,
                                   fmaf(wv[j][4 * h + 2], xv.z, fmaf(wv[j][4 * h + 3], xv.w, acc[j][r]))));
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < FR_PER_WARP; ++j)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r >= used) continue;      // uniform in the block
        float v = warp_sum(acc[j][r]);
        if (lane == 0 && n0 + j < N) {
          if (relu2) {
            v = fmaxf(v, 0.f);
            v *= v;
          }
          out[(size_t)(r0 + r) * ldo + n0 + j] = from_f32<TO>(v);
        }
      }
  }
}

template <typename TX, typename TW, typename TO, int VEC>
__global__ void __launch_bounds__(FR_WARPS * 32)
moe_few_rows_kernel(TO* __restrict__ out, int ldo, const TX* __restrict__ x, int ldx, const TW* __restrict__ w,
                    const int* __restrict__ row_src, const int* __restrict__ tile_group,
                    const int* __restrict__ n_tiles_dev, int N, int K, int relu2, int col_groups) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= *n_tiles_dev) return;
  extern __shared__ float xs[];            // FR_ROWS * FR_CHUNK floats: [rows in use][chunk]
  __shared__ int src[FR_ROWS];
  __shared__ int n_used;
  const int r0 = blockIdx.y * FR_ROWS;
  if (threadIdx.x < FR_ROWS) src[threadIdx.x] = row_src[r0 + threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) {          // the rows in use come first
    int u = 0;
    while (u < FR_ROWS && src[u] >= 0) ++u;
    n_used = u;
  }
  __syncthreads();
  const int used = n_used;
  if (used == 0) return;
  const TW* wbase = w + (size_t)tile_group[blockIdx.y] * N * K;
#define ZI_FEW_RUN(R) few_rows_run<TX, TW, TO, VEC, R>(out, ldo, x, ldx, wbase, src, used, r0, N, K, relu2, col_groups, xs)
  if (used == 1) ZI_FEW_RUN(1);
  else if (used == 2) ZI_FEW_RUN(2);
  else if (used <= 4) ZI_FEW_RUN(4);
  else if (used <= 8) ZI_FEW_RUN(8);
  else ZI_FEW_RUN(16);
#undef ZI_FEW_RUN
}

// One block lays the P = T * top pairs out by expert.  Pairs of expert e take the rows
// off[e] .. off[e] + count[e] - 1, and off[e+1] - off[e] is count[e] rounded up to whole tiles of
// `tile_rows`, so that every tile of the grouped product has one expert.  Pairs that chose an
// identity expert (index >= E) take no row.
//   row_token[r]  token whose input row r multiplies (-1: padding)
//   row_self[r]   r where the row is in use, else -1
//   pair_row[p]   row of pair p (-1: an identity expert)
//   tile_expert[i], *n_tiles     the arrays have cap_tiles tiles (at least P / tile_rows + E); rows and tiles
//                                beyond the ones in use are marked -1 and expert 0
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ chosen, int P, int top, int E, int tile_rows, int cap_tiles,
                 int* __restrict__ row_token,
                 int* __restrict__ row_self, int* __restrict__ pair_row, int* __restrict__ tile_expert,
                 int* __restrict__ n_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int si[];
  int* count = si;            // [E]
  int* off = si + E;          // [E + 1]
  int* cursor = off + E + 1;  // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      const int nt = (count[e] + tile_rows - 1) / tile_rows;
      for (int i = 0; i < nt; ++i) tile_expert[tiles + i] = e;
      tiles += nt;
      o += nt * tile_rows;
    }
    off[E] = o;
    *n_tiles = tiles;
    for (int i = tiles; i < cap_tiles; ++i) tile_expert[i] = 0;   // tiles not in use still name a group that exists
  }
  __syncthreads();
  const int rows = cap_tiles * tile_rows;      // all rows the arrays have: a product may walk every tile
  for (int r = threadIdx.x; r < rows; r += blockDim.x) row_token[r] = row_self[r] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = chosen[p];
    int r = -1;
    if (e >= 0 && e < E) {
      r = off[e] + atomicAdd(&cursor[e], 1);
      row_token[r] = p / top;
      row_self[r] = r;
    }
    pair_row[p] = r;
  }
}

// out[r] = x[row_src[r]], or zeros where row_src[r] is -1: the tokens' rows in the order of the pairs.
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ row_src,
                                   int width, int ldx) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, src = row_src[r];
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)r * width + c] = src >= 0 ? x[(size_t)src * ldx + c] : from_f32<T>(0.f);
}

// out[t] = sum_k weight[t,k] * (expert output of pair (t,k), or x[t] for an identity expert), k ascending.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ x,
                                   const int* __restrict__ chosen, const float* __restrict__ weight,
                                   const int* __restrict__ pair_row, int top, int E, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const size_t p = (size_t)t * top + k;
    const int e = chosen[p];
    const float v = e < E ? y[(size_t)pair_row[p] * H + c] : to_f32(x[(size_t)t * H + c]);
    acc = fmaf(weight[p], v, acc);
  }
  out[(size_t)t * H + c] = from_f32<T>(acc);
}
}  // namespace

extern "C" int zi_moe_route(int* chosen, float* weight, const float* logits, const float* correction, int T, int NR,
                            int top, int renormalize, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > NR) return zi_refuse("moe_route: %d of %d outputs cannot be chosen", top, NR);
  const size_t smem = (size_t)ROUTE_WARPS * 2 * NR * sizeof(float);
  if (smem > 48 * 1024) return zi_refuse("moe_route: %d router outputs are more than this kernel holds", NR);
  zi_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, chosen,
            weight, logits, correction, T, NR, top, renormalize);
  return zi_check_launch("moe_route");
}

extern "C" int zi_moe_route_grouped(int* chosen, float* weight, const float* logits, int T, int NR, int top,
                                    int renormalize, int score_kind, int groups, int keep, float wscale,
                                    cudaStream_t stream) {
  return zi_moe_route_grouped_c(chosen, weight, logits, nullptr, T, NR, top, renormalize, score_kind, groups, keep, wscale, stream);
}

extern "C" int zi_moe_route_grouped_c(int* chosen, float* weight, const float* logits, const float* correction, int T, int NR,
                                      int top, int renormalize, int score_kind, int groups, int keep, float wscale,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > NR) return zi_refuse("moe_route: %d of %d outputs cannot be chosen", top, NR);
  if (groups <= 0 || NR % groups || keep <= 0 || keep > groups)
    return zi_refuse("moe_route: %d outputs in %d groups of which %d are kept", NR, groups, keep);
  if (top > keep * (NR / groups)) return zi_refuse("moe_route: %d outputs cannot be chosen from %d groups of %d", top, keep, NR / groups);
  if (score_kind != 0 && score_kind != 1) return zi_refuse("moe_route: unknown score %d", score_kind);
  const size_t smem = (size_t)ROUTE_WARPS * 3 * NR * sizeof(float);
  if (smem > 48 * 1024) return zi_refuse("moe_route: %d router outputs are more than this kernel holds", NR);
  zi_launch(moe_route_grouped_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, chosen,
            weight, logits, T, NR, top, renormalize, score_kind, groups, keep, wscale, correction);
  return zi_check_launch("moe_route_grouped");
}

static int launch_moe_router(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype,
                             const float* correction, int T, int K, int NR, int top, int renormalize, int mode,
                             int score_kind, int groups, int keep, float wscale, cudaStream_t stream) {
  const bool grouped = mode == 1;
  if (T <= 0) return 0;
  if (top <= 0 || top > NR) return zi_refuse("moe_router: %d of %d outputs cannot be chosen", top, NR);
  if (grouped) {
    if (groups <= 0 || NR % groups || keep <= 0 || keep > groups || top > keep * (NR / groups))
      return zi_refuse("moe_router: %d of %d outputs in %d groups of which %d are kept", top, NR, groups, keep);
    if (score_kind != 0 && score_kind != 1) return zi_refuse("moe_router: unknown score %d", score_kind);
  }
  // One token per block.  (The kernel can take several, so that the router's weights pass from the L2 once per block and not
  // once per token; measured on 2,048 tokens of 4,096 values and 32 outputs: 88 us with one token per block, 84 with two,
  // 103 with four, 144 with eight, whose rows leave room for one block per SM only: not kept.)
  constexpr int tok = 1;
  const size_t smem = (size_t)tok * (K + 4 * NR) * sizeof(float);
  if (smem > 200 * 1024) return zi_refuse("moe_router: rows of %d values and %d outputs are more than this kernel holds", K, NR);
  // few tokens: a warp per output, up to 32 warps, since the few blocks are bound by the latency of a warp's walk along a row
  const int threads = T > 32 ? 256 : std::min(1024, std::max(256, 32 * NR));
  using bf = __nv_bfloat16;
#define ZI_ROUTER_T(TX, TW, GG, WIDE)                                                                              \
  do {                                                                                                             \
    auto kern = moe_router_kernel<TX, TW, GG, 1, WIDE>;                                                            \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return zi_refuse("moe_router: cannot get %zu bytes of shared memory", smem);                                 \
    zi_launch(kern, dim3(T), dim3(threads), smem, stream, chosen, weight, (const TX*)x, ldx, (const TW*)w, correction, T, K, \
              NR, top, renormalize, score_kind, groups, keep, wscale);                                             \
  } while (0)
#define ZI_ROUTER_G(TX, TW, GG) do { if (threads > 256) ZI_ROUTER_T(TX, TW, GG, true); else ZI_ROUTER_T(TX, TW, GG, false); } while (0)
#define ZI_ROUTER(TX, TW) do { if (mode == 2) ZI_ROUTER_G(TX, TW, 2); else if (grouped) ZI_ROUTER_G(TX, TW, 1); else ZI_ROUTER_G(TX, TW, 0); } while (0)
  if (x_dtype == ZI_F32 && w_dtype == ZI_F32) ZI_ROUTER(float, float);
  else if (x_dtype == ZI_F32 && w_dtype == ZI_BF16) ZI_ROUTER(float, bf);
  else if (x_dtype == ZI_BF16 && w_dtype == ZI_F32) ZI_ROUTER(bf, float);
  else if (x_dtype == ZI_BF16 && w_dtype == ZI_BF16) ZI_ROUTER(bf, bf);
  else return zi_refuse("moe_router: unknown dtype tags %d, %d", x_dtype, w_dtype);
#undef ZI_ROUTER
#undef ZI_ROUTER_G
#undef ZI_ROUTER_T
  return zi_check_launch("moe_router");
}

extern "C" int zi_moe_router(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w, int w_dtype,
                             const float* correction, int T, int K, int NR, int top, int renormalize,
                             cudaStream_t stream) {
  return launch_moe_router(chosen, weight, x, x_dtype, ldx, w, w_dtype, correction, T, K, NR, top, renormalize, 0, 0, 1, 1,
                           1.0f, stream);
}

// The router's product and the choice among groups of outputs (zi_moe_route_grouped) in one kernel.
extern "C" int zi_moe_router_grouped(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w,
                                     int w_dtype, int T, int K, int NR, int top, int renormalize, int score_kind,
                                     int groups, int keep, float wscale, cudaStream_t stream) {
  return launch_moe_router(chosen, weight, x, x_dtype, ldx, w, w_dtype, nullptr, T, K, NR, top, renormalize, 1, score_kind,
                           groups, keep, wscale, stream);
}

extern "C" int zi_moe_router_grouped_c(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w,
                                       int w_dtype, const float* correction, int T, int K, int NR, int top, int renormalize,
                                       int score_kind, int groups, int keep, float wscale, cudaStream_t stream) {
  return launch_moe_router(chosen, weight, x, x_dtype, ldx, w, w_dtype, correction, T, K, NR, top, renormalize, 1, score_kind,
                           groups, keep, wscale, stream);
}

// The router's product, a bias on the logits, the `top` largest logits and the softmax over them alone, in one kernel.
extern "C" int zi_moe_router_top_logits(int* chosen, float* weight, const void* x, int x_dtype, int ldx, const void* w,
                                        int w_dtype, const float* bias, int T, int K, int NR, int top, cudaStream_t stream) {
  return launch_moe_router(chosen, weight, x, x_dtype, ldx, w, w_dtype, bias, T, K, NR, top, 0, 2, 0, 1, 1, 1.0f, stream);
}

// The same choice from logits already made.
extern "C" int zi_moe_route_top_logits(int* chosen, float* weight, const float* logits, const float* bias, int T, int NR,
                                       int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > NR) return zi_refuse("moe_route: %d of %d outputs cannot be chosen", top, NR);
  const size_t smem = (size_t)ROUTE_WARPS * NR * sizeof(float);
  if (smem > 48 * 1024) return zi_refuse("moe_route: %d router outputs are more than this kernel holds", NR);
  zi_launch(moe_route_top_logits_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, chosen,
            weight, logits, bias, T, NR, top);
  return zi_check_launch("moe_route_top_logits");
}

// Grouped product for tiles of 16 rows (see moe_few_rows_kernel).  x and w of one type (float32 or bfloat16),
// out float32 or that type.
extern "C" int zi_moe_few_rows(void* out, int out_dtype, int ldo, const void* x, int dtype, int ldx, const void* w,
                               const int* row_src, const int* tile_group, const int* n_tiles_dev, int max_tiles, int N,
                               int K, int relu2, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K % 4 || ldx % 4 || (uintptr_t)x % 16 || (uintptr_t)w % 16)
    return zi_refuse("moe_few_rows: rows of %d values (pitch %d) are not whole 16-byte pieces", K, ldx);
  const size_t smem = (size_t)FR_ROWS * FR_CHUNK * sizeof(float);
  static const int forced = [] { const char* e = getenv("ZINFER_B200_FEW_ROWS_GROUPS"); return e ? atoi(e) : 0; }();
  // two groups of 16 columns per block: the rows staged once serve both (measured at 8 requests: 91 -> 79 us for 23
  // experts of 4,096 x 2,048; four groups: no further gain and too few blocks for narrow experts)
  const int col_groups = forced > 0 ? forced : 2;
  dim3 grid((N + FR_COLS * col_groups - 1) / (FR_COLS * col_groups), max_tiles);
  using bf = __nv_bfloat16;
#define ZI_FEW(TX, TO, VEC)                                                                                        \
  do {                                                                                                             \
    auto kern = moe_few_rows_kernel<TX, TX, TO, VEC>;                                                                 \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)         \
      return zi_refuse("moe_few_rows: cannot get %zu bytes of shared memory", smem);                               \
    zi_launch(kern, dim3(grid), dim3(FR_WARPS * 32), smem, stream, (TO*)out, ldo, (const TX*)x, ldx, (const TX*)w, row_src, \
              tile_group, n_tiles_dev, N, K, relu2, col_groups);                                                   \
  } while (0)
  const bool wide = K % 8 == 0;        // bfloat16 rows in whole 16-byte pieces
  if (dtype == ZI_F32 && out_dtype == ZI_F32) ZI_FEW(float, float, 4);
  else if (dtype == ZI_BF16 && out_dtype == ZI_F32 && wide) ZI_FEW(bf, float, 8);
  else if (dtype == ZI_BF16 && out_dtype == ZI_F32) ZI_FEW(bf, float, 4);
  else if (dtype == ZI_BF16 && out_dtype == ZI_BF16 && wide) ZI_FEW(bf, bf, 8);
  else if (dtype == ZI_BF16 && out_dtype == ZI_BF16) ZI_FEW(bf, bf, 4);
  else return zi_refuse("moe_few_rows: operand type %d with results of type %d", dtype, out_dtype);
#undef ZI_FEW
  return zi_check_launch("moe_few_rows");
}

extern "C" int zi_moe_align(const int* chosen, int P, int top, int E, int tile_rows, int cap_tiles, int* row_token,
                            int* row_self, int* pair_row, int* tile_expert, int* n_tiles, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (cap_tiles < (P + tile_rows - 1) / tile_rows + E) return zi_refuse("moe_align: %d tiles cannot hold %d pairs of %d experts", cap_tiles, P, E);
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  if (smem > 48 * 1024) return zi_refuse("moe_align: %d experts are more than this kernel holds", E);
  zi_launch(moe_align_kernel, dim3(1), dim3(1024), smem, stream, chosen, P, top, E, tile_rows, cap_tiles, row_token,
            row_self, pair_row, tile_expert, n_tiles);
  return zi_check_launch("moe_align");
}

extern "C" int zi_gather_rows(void* out, const void* x, int dtype, const int* row_src, int rows, int width, int ldx,
                              cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(gather_rows_kernel<TT>, dim3(rows), dim3(256), 0, stream, (TT*)out, (const TT*)x,
                                         row_src, width, ldx));
  return zi_check_launch("gather_rows");
}

extern "C" int zi_moe_combine(void* out, const float* y, const void* x, int dtype, const int* chosen,
                              const float* weight, const int* pair_row, int T, int top, int E, int H,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  dim3 grid((H + 255) / 256, T);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(moe_combine_kernel<TT>, dim3(grid), dim3(256), 0, stream, (TT*)out, y, (const TT*)x,
                                         chosen, weight, pair_row, top, E, H));
  return zi_check_launch("moe_combine");
}

ZI_TRACE_SETTER(moe)
