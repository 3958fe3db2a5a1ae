// What follows a token's fused projection row when the changes span the whole row rather than one head:
//   zi_qkv_rows_prepare   [q heads | k heads | v heads | gate] -> biases, an RMS norm over ALL of q (and all of k)
//                         with a weight per element, rotation of the first rot_dims dimensions of every q and k head
//                         (pairs (i, i + rot_dims/2)), q into a tensor of its own, k and v into the token's page slot,
//                         the gate columns into a tensor of their own
//   zi_rmsnorm_rows       RMS norm of rows of activations (a latent between two projections)
// 32-bit arithmetic; the source may be 32-bit while the results have the activations' type, so that a bias or a norm
// meets the product's unrounded sums.  One block per token; every sum runs in an order that depends on the row only.
#include "api.h"
#include "common.cuh"

namespace {
// few tokens in bfloat16 (a decode step): more threads a token, since the walk is latency; the 32-bit path keeps one
// block size, so that its sums' order depends on nothing but the row
constexpr int ROW_THREADS = 256, ROW_THREADS_FEW = 1024;

template <typename TS>
__device__ __forceinline__ float row_at(const TS* x, const float* bias, int e) {
  return to_f32(x[e]) + (bias ? bias[e] : 0.f);
}

// One part (q or k) of the row: n_heads heads of d values starting at `x`, written to dst(head, i).
template <typename TS, typename T, class Dst>
__device__ __forceinline__ void finish_part(const TS* x, const float* bias, int n_heads, int d, const float* w, float eps,
                                            int rot_dims, const float* cs, const float* sn, float* scratch, Dst dst) {
  const int n = n_heads * d, half = rot_dims >> 1;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const float v = row_at(x, bias, e);
      ss = fmaf(v, v, ss);
    }
    inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  }
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int hd = e / d, i = e - hd * d;
    float v = row_at(x, bias, e);
    if (w) v = norm_scale(v, w[e], inv);
    if (i < rot_dims) {
      const int p = i < half ? e + half : e - half;       // the other element of the pair
      float o = row_at(x, bias, p);
      if (w) o = norm_scale(o, w[p], inv);
      if (i < half) {
        rotate_pair(v, o, cs[i], sn[i]);
      } else {
        rotate_pair(o, v, cs[i - half], sn[i - half]);
      }
    }
    dst(hd, i, from_f32<T>(v));
  }
}

template <typename TS, typename T>
__global__ void __launch_bounds__(ROW_THREADS_FEW)
qkv_rows_kernel(const TS* __restrict__ src, int src_stride, const float* __restrict__ bias, T* __restrict__ q_out,
                int q_stride, T* __restrict__ gate_out, int gate_stride, int n_gate, int nq, int nkv, int d, int dv,
                const float* __restrict__ qw, const float* __restrict__ kw, float eps, int rot_dims,
                const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_table_pos,
                const int* __restrict__ positions, T* __restrict__ kcache, T* __restrict__ vcache,
                const int* __restrict__ slots, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const TS* row = src + (size_t)t * src_stride;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= n_table_pos && n_table_pos > 0 ? n_table_pos - 1 : pos);   // the host refuses such positions
  const int half = rot_dims >> 1;
  const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
  const int rd = cos_t ? rot_dims : 0;
  const int qn = nq * d, kn = nkv * d, vn = nkv * dv;
  T* qo = q_out + (size_t)t * q_stride;
  finish_part<TS, T>(row, bias, nq, d, qw, eps, rd, cs, sn, scratch,
                     [&](int hd, int i, T v) { qo[hd * d + i] = v; });
  for (int e = threadIdx.x; e < n_gate; e += blockDim.x)
    gate_out[(size_t)t * gate_stride + e] = from_f32<T>(row_at(row + qn + kn + vn, bias ? bias + qn + kn + vn : nullptr, e));
  const int slot = slots[t];
  if (slot < 0) return;        // a row that pads a captured batch
  const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
  finish_part<TS, T>(row + qn, bias ? bias + qn : nullptr, nkv, d, kw, eps, rd, cs, sn, scratch,
                     [&](int hd, int i, T v) { kcache[((page * nkv + hd) * page_size + off) * d + i] = v; });
  for (int e = threadIdx.x; e < vn; e += blockDim.x) {
    const int hd = e / dv, i = e - hd * dv;
    vcache[((page * nkv + hd) * page_size + off) * dv + i] = from_f32<T>(row_at(row + qn + kn, bias ? bias + qn + kn : nullptr, e));
  }
}

template <typename TS, typename T>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_rows_kernel(T* __restrict__ out, int ldo, const TS* __restrict__ x, int ldx, const float* __restrict__ w, float eps,
                    int n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const TS* xr = x + (size_t)blockIdx.x * ldx;
  float ss = 0.f;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const float v = to_f32(xr[e]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  for (int e = threadIdx.x; e < n; e += blockDim.x)
    out[(size_t)blockIdx.x * ldo + e] = from_f32<T>(norm_scale(to_f32(xr[e]), w[e], inv));
}
}  // namespace

#define ZI_DISPATCH_SRC_OUT(sd, od, TS, TT, ...)                                                   \
  do {                                                                                             \
    if ((sd) == ZI_F32 && (od) == ZI_F32) { using TS = float; using TT = float; __VA_ARGS__; }      \
    else if ((sd) == ZI_F32 && (od) == ZI_BF16) { using TS = float; using TT = __nv_bfloat16; __VA_ARGS__; } \
    else if ((sd) == ZI_BF16 && (od) == ZI_BF16) { using TS = __nv_bfloat16; using TT = __nv_bfloat16; __VA_ARGS__; } \
    else return zi_refuse("a source of type %d cannot become results of type %d", (int)(sd), (int)(od)); \
  } while (0)

extern "C" int zi_qkv_rows_prepare(const void* src, int src_dtype, int src_stride, const float* bias, void* q_out,
                                   int q_stride, void* gate_out, int gate_stride, int n_gate, int out_dtype, int T, int nq,
                                   int nkv, int d, int dv, const float* qw, const float* kw, float eps, int rot_dims,
                                   const float* cos_t, const float* sin_t, int n_table_pos, const int* positions,
                                   void* kcache, void* vcache, const int* slots, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0) return zi_refuse("qkv_rows_prepare: %d and %d heads of %d and %d", nq, nkv, d, dv);
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > d) return zi_refuse("qkv_rows_prepare: %d rotated dimensions of a head of %d", rot_dims, d);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("qkv_rows_prepare: cos and sin tables go together");
  if ((qw == nullptr) != (kw == nullptr)) return zi_refuse("qkv_rows_prepare: q and k are normed together or not at all");
  if (!kcache || !vcache || !slots || page_size <= 0) return zi_refuse("qkv_rows_prepare: keys and values need pages and slots");
  if (n_gate < 0 || (n_gate > 0 && !gate_out)) return zi_refuse("qkv_rows_prepare: %d gate columns without a place", n_gate);
  ZI_DISPATCH_SRC_OUT(src_dtype, out_dtype, TS, TT,
                      zi_launch(qkv_rows_kernel<TS, TT>, dim3(T), dim3(T <= 64 && out_dtype == ZI_BF16 ? ROW_THREADS_FEW : ROW_THREADS), 0, stream,
                                (const TS*)src, src_stride, bias,
                                (TT*)q_out, q_stride, (TT*)gate_out, gate_stride, n_gate, nq, nkv, d, dv, qw, kw, eps, rot_dims,
                                cos_t, sin_t, n_table_pos, positions, (TT*)kcache, (TT*)vcache, slots, page_size));
  return zi_check_launch("qkv_rows_prepare");
}

extern "C" int zi_rmsnorm_rows(void* out, int ldo, int out_dtype, const void* x, int ldx, int x_dtype, const float* w,
                               float eps, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  ZI_DISPATCH_SRC_OUT(x_dtype, out_dtype, TS, TT,
                      zi_launch(rmsnorm_rows_kernel<TS, TT>, dim3(T), dim3(ROW_THREADS), 0, stream, (TT*)out, ldo, (const TS*)x,
                                ldx, w, eps, n));
  return zi_check_launch("rmsnorm_rows");
}

ZI_TRACE_SETTER(projection_rows)
