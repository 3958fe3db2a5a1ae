// Memory-bound kernels around the matrix products: embedding gather, residual add
// fused with RMSNorm, per-head q/k RMSNorm fused with rotary positions and the
// write of keys and values into cache pages, SwiGLU, and the rotary table.
// All arithmetic is 32-bit; only loads and stores touch bfloat16.
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------- embedding gather
template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ h, const T* __restrict__ table,
                                    const int* __restrict__ ids, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* out = h + (size_t)t * H;
  if (id < 0 || id >= V) {  // the host refuses such ids; never read out of bounds
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f32(row[i]);
}

extern "C" int zi_embed_gather(float* h, const void* table, int table_dtype, const int* ids, int T, int H,
                               int V, cudaStream_t stream) {
  if (T <= 0) return 0;
  ZI_DISPATCH_DTYPE(table_dtype, TT,
                    zi_launch(embed_gather_kernel<TT>, dim3(T), dim3(256), 0, stream, h, (const TT*)table, ids, H, V));
  return zi_check_launch("embed_gather");
}

// ------------------------------------------- embedding with a hashed table of token pairs
// One block per token.  The token before: the one before it in this step's portion, or, for the portion's first
// token, what the request's slot holds from the step before (nothing at position 0: the table's last row).  The
// block of a portion's first token reads the slot and then stores the portion's last token there, so no other
// block touches the slot.
template <typename T>
__global__ void embed_bigram_kernel(float* __restrict__ h, const T* __restrict__ table, const T* __restrict__ bigram,
                                    const int* __restrict__ ids, const int* __restrict__ positions,
                                    const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                    int* __restrict__ last_token, int n_seqs, int H, int V, float scale, int buckets,
                                    long long mul_prev, long long mul_cur) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int lo = 0, hi = n_seqs - 1;                 // the request whose portion holds token t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int start = cu_q[lo], end = cu_q[lo + 1];
  const int id = ids[t];
  int prev = -1;
  if (positions[t] > 0) prev = t > start ? ids[t - 1] : last_token[state_slots[lo]];
  __syncthreads();                             // every thread has read the slot before it is overwritten
  if (t == start && threadIdx.x == 0 && end > start) last_token[state_slots[lo]] = ids[end - 1];
  float* out = h + (size_t)t * H;
  if (id < 0 || id >= V) {  // the host refuses such ids; never read out of bounds
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  if (bigram == nullptr) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
    return;
  }
  long long r = buckets;
  if (prev >= 0) {
    r = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    if (r < 0) r += buckets;
  }
  const T* pair = bigram + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = fmaf(to_f32(row[i]), scale, to_f32(pair[i]));
}

extern "C" int zi_embed_bigram(float* h, const void* table, const void* bigram, int table_dtype, const int* ids,
                               const int* positions, const int* cu_q, const int* state_slots, int* last_token, int n_seqs,
                               int T, int H, int V, float scale, int buckets, long long mul_prev, long long mul_cur,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_seqs <= 0 || !cu_q || !state_slots || !last_token || !positions)
    return zi_refuse("embed_bigram: the step's request arrays and the slots of the last tokens are needed");
  if (bigram && buckets <= 0) return zi_refuse("embed_bigram: %d buckets", buckets);
  ZI_DISPATCH_DTYPE(table_dtype, TT,
                    zi_launch(embed_bigram_kernel<TT>, dim3(T), dim3(256), 0, stream, h, (const TT*)table, (const TT*)bigram, ids,
                              positions, cu_q, state_slots, last_token, n_seqs, H, V, scale, buckets, mul_prev, mul_cur));
  return zi_check_launch("embed_bigram");
}

// ------------------------------------------------------------ residual add + RMSNorm
// h[row] += delta[row] (when delta is given), out[r] = h[row] * w / sqrt(mean(h[row]^2) + eps).
// With `rows` (a gather of picked rows, possibly with repeats) h itself is not modified.
// One block per row; the sum of squares is taken in a fixed order.
// The update may also come as split-K partial sums: dpart[z][row][i], z < splits, added in order.
// The update is multiplied by `dscale` as it is added (a residual multiplier; 1 changes no bit), and
// `bias` [H], when given, is added to every row as well (a vector a model adds between two layers).
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ dpart, int splits, size_t zstride,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H, float dscale,
                                   const float* __restrict__ bias) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* hr = h + (size_t)row * H;
  float ss = 0.f;
  if (dpart) {
    const float* dr = dpart + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float d = 0.f;
      for (int z = 0; z < splits; ++z) d += dr[z * zstride + i];
      float v = fmaf(dscale, d, hr[i]);
      if (bias) v += bias[i];
      if (!rows) hr[i] = v;
      ss += v * v;
    }
  } else if (delta) {
    const TD* dr = delta + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = fmaf(dscale, to_f32(dr[i]), hr[i]);
      if (bias) v += bias[i];
      if (!rows) hr[i] = v;
      ss += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i];
      if (bias) {
        v += bias[i];
        if (!rows) hr[i] = v;
      }
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* o = out + (size_t)r * H;
  if (!rows) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(hr[i] * w[i] * inv);
  } else {
    // picked rows: h is left as it is (a row may be picked twice), the sum is formed again
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i];
      if (dpart) {
        float d = 0.f;
        for (int z = 0; z < splits; ++z) d += dpart[z * zstride + (size_t)row * H + i];
        v = fmaf(dscale, d, v);
      } else if (delta) {
        v = fmaf(dscale, to_f32(delta[(size_t)row * H + i]), v);
      }
      if (bias) v += bias[i];
      o[i] = from_f32<TO>(v * w[i] * inv);
    }
  }
}

// The same with the row held in registers: one read of h and delta, one write of h and
// of the result.  Needs H % 4 == 0 and H <= 4 * VPT * blockDim.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

// PART: the update comes as split-K partial sums (`dpart`), else whole (`delta`) or not at all.
// EXTRA: the update is multiplied by dscale and a bias vector may be added (compiled apart: the plain
// add keeps its code).
template <typename TD, typename TO, int VPT, bool PART, bool EXTRA>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ dpart, int splits, size_t zstride,
                                       const float* __restrict__ w, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int H, int n_rows, float dscale,
                                       const float* __restrict__ bias) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int nvec = H >> 2;
  float4 ww[VPT];   // the norm's weights do not depend on the kernel before this one
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    ww[i] = idx < nvec ? Vec4<float>::load(w + 4 * idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  // Many rows (a prompt): as many blocks as are resident at once walk the rows, so that there is no
  // last, partly filled round of blocks and the blocks of an SM drift apart (one loads while another stores).
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
  const int row = rows ? rows[r] : r;
  float* hr = h + (size_t)row * H;
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float4 a = Vec4<float>::load(hr + 4 * idx);
      if (PART) {
        // the splits are read eight (then four) at a time so that their loads are in flight
        // together; they are still added in order of z
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* base = dpart + (size_t)row * H + 4 * idx;
        int z = 0;
        for (; z + 8 <= splits; z += 8) {
          float4 p[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) p[j] = Vec4<float>::load(base + (size_t)(z + j) * zstride);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            d.x += p[j].x; d.y += p[j].y; d.z += p[j].z; d.w += p[j].w;
          }
        }
        for (; z + 4 <= splits; z += 4) {
          const float4 p0 = Vec4<float>::load(base + (size_t)z * zstride);
          const float4 p1 = Vec4<float>::load(base + (size_t)(z + 1) * zstride);
          const float4 p2 = Vec4<float>::load(base + (size_t)(z + 2) * zstride);
          const float4 p3 = Vec4<float>::load(base + (size_t)(z + 3) * zstride);
          d.x = (((d.x + p0.x) + p1.x) + p2.x) + p3.x;
          d.y = (((d.y + p0.y) + p1.y) + p2.y) + p3.y;
          d.z = (((d.z + p0.z) + p1.z) + p2.z) + p3.z;
          d.w = (((d.w + p0.w) + p1.w) + p2.w) + p3.w;
        }
        for (; z < splits; ++z) {
          const float4 p = Vec4<float>::load(base + (size_t)z * zstride);
          d.x += p.x; d.y += p.y; d.z += p.z; d.w += p.w;
        }
        if (EXTRA) {
          a.x = fmaf(dscale, d.x, a.x); a.y = fmaf(dscale, d.y, a.y); a.z = fmaf(dscale, d.z, a.z); a.w = fmaf(dscale, d.w, a.w);
        } else {
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
        if (!EXTRA && !rows) Vec4<float>::store(hr + 4 * idx, a);   // picked rows leave h as it is (a row may be picked twice)
      } else if (delta) {
        const float4 d = Vec4<TD>::load(delta + (size_t)row * H + 4 * idx);
        if (EXTRA) {
          a.x = fmaf(dscale, d.x, a.x); a.y = fmaf(dscale, d.y, a.y); a.z = fmaf(dscale, d.z, a.z); a.w = fmaf(dscale, d.w, a.w);
        } else {
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
        if (!EXTRA && !rows) Vec4<float>::store(hr + 4 * idx, a);
      }
      if (EXTRA) {
        if (bias) {
          const float4 b = Vec4<float>::load(bias + 4 * idx);
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (!rows && (PART || delta || bias)) Vec4<float>::store(hr + 4 * idx, a);
      }
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec)
      Vec4<TO>::store(o + 4 * idx, make_float4(v[i].x * ww[i].x * inv, v[i].y * ww[i].y * inv, v[i].z * ww[i].z * inv,
                                               v[i].w * ww[i].w * inv));
  }
  }
}

// SMs of the current device (asked once).
static int sm_count_of_current_device() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sms = n;
    else
      return 148;
  }
  return sms;
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* h, const void* delta, const float* dpart, int splits, size_t zstride,
                              const float* w, float eps, void* out, const int* rows, int n_rows, int H,
                              float dscale, const float* bias, cudaStream_t stream) {
  const bool aligned = H % 4 == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)bias % 16 == 0) &&
                       ((uintptr_t)out % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)dpart % 16 == 0) &&
                       zstride % 4 == 0;
  const int nvec = H / 4;
  const bool extra = dscale != 1.0f || bias != nullptr;
  // few rows (decode): one vector per thread, so that a row's loads are all in flight at once
  // many rows (a prompt): blocks of 512 with two vectors a thread keep the most bytes in flight per SM (measured:
  // 8,192 rows of 4,096 in 70 us against 76 with 256 threads and 97 with 128)
  const int threads = n_rows <= 256 ? (nvec > 512 ? 1024 : nvec > 256 ? 512 : 256) : (nvec >= 1024 ? 512 : 256);
  if (aligned && nvec <= threads * 8) {
    const int vpt = (nvec + threads - 1) / threads;
    // as many blocks as are resident at once (asked once per kernel and block size), or one per row if those are fewer
#define ZI_LAUNCH_VPT(V, P, X)                                                                                     \
  do {                                                                                                             \
    auto kern = add_rmsnorm_vec_kernel<TD, TO, V, P, X>;                                                           \
    static int per_sm[3] = {0, 0, 0};                                                                              \
    int& slot = per_sm[threads == 256 ? 0 : threads == 512 ? 1 : 2];                                               \
    if (slot == 0 && (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&slot, kern, threads, 0) != cudaSuccess || slot < 1)) \
      slot = 1;                                                                                                    \
    const int resident = sm_count_of_current_device() * slot;                                                      \
    zi_launch(kern, dim3(n_rows < resident ? n_rows : resident), dim3(threads), 0, stream, h, (const TD*)delta, dpart, \
              splits, zstride, w, eps, (TO*)out, rows, H, n_rows, dscale, bias);                                   \
  } while (0)
#define ZI_LAUNCH_PART(V)                                \
  do {                                                   \
    if (extra) {                                         \
      if (dpart) ZI_LAUNCH_VPT(V, true, true);           \
      else ZI_LAUNCH_VPT(V, false, true);                \
    } else {                                             \
      if (dpart) ZI_LAUNCH_VPT(V, true, false);          \
      else ZI_LAUNCH_VPT(V, false, false);               \
    }                                                    \
  } while (0)
    if (vpt <= 1) ZI_LAUNCH_PART(1);
    else if (vpt <= 2) ZI_LAUNCH_PART(2);
    else if (vpt <= 4) ZI_LAUNCH_PART(4);
    else ZI_LAUNCH_PART(8);
#undef ZI_LAUNCH_PART
#undef ZI_LAUNCH_VPT
  } else {
    const int t2 = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    zi_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(t2), 0, stream, h, (const TD*)delta, dpart, splits, zstride, w, eps, (TO*)out,
                                                          rows, H, dscale, bias);
  }
  return zi_check_launch("add_rmsnorm");
}

extern "C" int zi_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_partials, int splits,
                              long long split_stride, const float* w, float eps, void* out, int out_dtype,
                              const int* rows, int n_rows, int H, cudaStream_t stream) {
  return zi_add_rmsnorm_scaled(h, delta, delta_dtype, delta_partials, splits, split_stride, 1.0f, nullptr, w, eps, out,
                               out_dtype, rows, n_rows, H, stream);
}

extern "C" int zi_add_rmsnorm_scaled(float* h, const void* delta, int delta_dtype, const float* delta_partials,
                                     int splits, long long split_stride, float delta_scale, const float* bias,
                                     const float* w, float eps, void* out, int out_dtype, const int* rows, int n_rows,
                                     int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (delta && delta_partials) return zi_refuse("add_rmsnorm: give the update either whole or as partial sums");
  ZI_DISPATCH_DTYPE(delta_dtype, TD, ZI_DISPATCH_DTYPE(out_dtype, TO, {
                      return launch_add_rmsnorm<TD, TO>(h, delta, delta_partials, splits, (size_t)split_stride, w, eps,
                                                        out, rows, n_rows, H, delta_scale, bias, stream);
                    }));
  return 0;
}

// Plain add of the last pending update into the residual stream (rows optional).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n, float dscale) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] = fmaf(dscale, to_f32(delta[i]), h[i]);
}

extern "C" int zi_residual_add(float* h, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
  return zi_residual_add_scaled(h, delta, delta_dtype, 1.0f, n, stream);
}

extern "C" int zi_residual_add_scaled(float* h, const void* delta, int delta_dtype, float delta_scale, long long n,
                                      cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  ZI_DISPATCH_DTYPE(delta_dtype, TD,
                    zi_launch(residual_add_kernel<TD>, dim3(blocks), dim3(threads), 0, stream, h, (const TD*)delta, (size_t)n, delta_scale));
  return zi_check_launch("residual_add");
}

// --------------------------------------------------------------------------- SwiGLU
// gu is [T, 2I].  interleave == 0: gate in the first I columns, up in the last I.
// interleave == 64: blocks of 128 columns hold 64 gate then the 64 up values of the same
// features.  out[t,i] = act(g) * u, act = silu (ZI_ACT_SILU) or the tanh form of gelu (ZI_ACT_GELU_TANH).
template <int ACT>
__device__ __forceinline__ float gated(float g, float u) {
  if (ACT == ZI_ACT_GELU_TANH) return gelu_tanh_f32(g) * u;
  return g / (1.0f + expf(-g)) * u;
}
__device__ __forceinline__ void gate_up_columns(int i, int I, int interleave, int& gcol, int& ucol) {
  if (interleave) {
    gcol = (i / interleave) * 2 * interleave + (i % interleave);
    ucol = gcol + interleave;
  } else {
    gcol = i;
    ucol = i + I;
  }
}

template <typename T, int ACT>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total, int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  const float g = to_f32(gu[t * 2 * I + gc]);
  const float u = to_f32(gu[t * 2 * I + uc]);
  out[idx] = from_f32<T>(gated<ACT>(g, u));
}

// gate and up given as split-K partial sums part[z][t][2I]; four elements per thread.
template <typename T, int ACT>
__global__ void swiglu_partials_kernel(T* __restrict__ out, const float* __restrict__ part, int splits, size_t zstride,
                                       int I, size_t total_vec, int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I >> 2;
  const size_t t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 4;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  for (int z0 = 0; z0 < splits; z0 += 4) {   // four splits' loads in flight together, added in order of z
    float4 a[4], b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float* p = part + (size_t)(z0 + j) * zstride + t * 2 * I;
      const bool on = z0 + j < splits;
      a[j] = on ? *reinterpret_cast<const float4*>(p + gc) : make_float4(0.f, 0.f, 0.f, 0.f);
      b[j] = on ? *reinterpret_cast<const float4*>(p + uc) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (z0 + j < splits) {
        g.x += a[j].x; g.y += a[j].y; g.z += a[j].z; g.w += a[j].w;
        u.x += b[j].x; u.y += b[j].y; u.z += b[j].z; u.w += b[j].w;
      }
    }
  }
  Vec4<T>::store(out + t * I + i, make_float4(gated<ACT>(g.x, u.x), gated<ACT>(g.y, u.y), gated<ACT>(g.z, u.z),
                                              gated<ACT>(g.w, u.w)));
}

// Eight elements per thread (16-byte loads of bfloat16, two of float); needs I % 8 == 0.
template <typename T, int ACT>
__global__ void swiglu_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total_vec,
                                  int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I >> 3;
  const size_t t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  const T* g = gu + t * 2 * I + gc;
  const T* u = gu + t * 2 * I + uc;
  T* o = out + t * I + i;
#pragma unroll
  for (int k = 0; k < 8; k += 4) {
    const float4 gv = Vec4<T>::load(g + k), uv = Vec4<T>::load(u + k);
    Vec4<T>::store(o + k, make_float4(gated<ACT>(gv.x, uv.x), gated<ACT>(gv.y, uv.y), gated<ACT>(gv.z, uv.z),
                                      gated<ACT>(gv.w, uv.w)));
  }
}

// The clamped gate: g <- min(g, limit), u <- clamp(u, -limit, limit), out = g * sigmoid(alpha * g) * (u + shift).
// gate and up come whole or as split-K partial sums added in order; any width.
template <typename T, typename TS>
__global__ void clamped_gate_kernel(T* __restrict__ out, const TS* __restrict__ gu, const float* __restrict__ part, int splits,
                                    size_t zstride, int I, size_t total, int interleave, float limit, float alpha,
                                    float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  float g, u;
  if (part) {
    g = u = 0.f;
    for (int z = 0; z < splits; ++z) {
      g += part[(size_t)z * zstride + t * 2 * I + gc];
      u += part[(size_t)z * zstride + t * 2 * I + uc];
    }
  } else {
    g = to_f32(gu[t * 2 * I + gc]);
    u = to_f32(gu[t * 2 * I + uc]);
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  out[idx] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
}

__device__ __forceinline__ float clamped_gated(float g, float u, float limit, float alpha, float shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + shift);
}

// Eight elements per thread (16-byte loads of bfloat16, two of float); needs I % 8 == 0 and one type throughout.
template <typename T>
__global__ void clamped_gate_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total_vec, int interleave,
                                        float limit, float alpha, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I >> 3;
  const size_t t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  const T* g = gu + t * 2 * I + gc;
  const T* u = gu + t * 2 * I + uc;
  T* o = out + t * I + i;
#pragma unroll
  for (int k = 0; k < 8; k += 4) {
    const float4 gv = Vec4<T>::load(g + k), uv = Vec4<T>::load(u + k);
    Vec4<T>::store(o + k, make_float4(clamped_gated(gv.x, uv.x, limit, alpha, shift), clamped_gated(gv.y, uv.y, limit, alpha, shift),
                                      clamped_gated(gv.z, uv.z, limit, alpha, shift), clamped_gated(gv.w, uv.w, limit, alpha, shift)));
  }
}

extern "C" int zi_clamped_gate(void* out, int dtype, const void* gu, int gu_dtype, const float* partials, int splits,
                               long long split_stride, int T, int I, int interleave, float limit, float alpha, float shift,
                               cudaStream_t stream) {
  if (interleave && (interleave % 8 || I % interleave)) return zi_refuse("clamped_gate: interleave %d does not fit I = %d", interleave, I);
  if (!(limit > 0.f)) return zi_refuse("clamped_gate: the limit must be positive");
  if ((gu == nullptr) == (partials == nullptr)) return zi_refuse("clamped_gate: gate and up come whole or as partial sums");
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  if (!partials && gu_dtype == dtype && I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const size_t total_vec = total / 8;
    ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(clamped_gate_vec_kernel<TT>, dim3((unsigned)((total_vec + 255) / 256)), dim3(256), 0,
                                           stream, (TT*)out, (const TT*)gu, I, total_vec, interleave, limit, alpha, shift));
    return zi_check_launch("clamped_gate");
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    if (partials || gu_dtype == ZI_F32)
      zi_launch(clamped_gate_kernel<TT, float>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const float*)gu, partials, splits,
                (size_t)split_stride, I, total, interleave, limit, alpha, shift);
    else
      zi_launch(clamped_gate_kernel<TT, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (TT*)out, (const __nv_bfloat16*)gu,
                partials, splits, (size_t)split_stride, I, total, interleave, limit, alpha, shift);
  });
  return zi_check_launch("clamped_gate");
}

#define ZI_DISPATCH_ACT(act, ACT, ...)                                              \
  do {                                                                             \
    if ((act) == ZI_ACT_SILU) { constexpr int ACT = ZI_ACT_SILU; __VA_ARGS__; }     \
    else if ((act) == ZI_ACT_GELU_TANH) { constexpr int ACT = ZI_ACT_GELU_TANH; __VA_ARGS__; } \
    else return zi_refuse("unknown activation tag %d", (int)(act));                \
  } while (0)

extern "C" int zi_swiglu_partials(void* out, int dtype, const float* partials, int splits, long long split_stride,
                                  int T, int I, int interleave, cudaStream_t stream) {
  return zi_gated_act_partials(out, dtype, partials, splits, split_stride, T, I, interleave, ZI_ACT_SILU, stream);
}

extern "C" int zi_swiglu(void* out, const void* gu, int dtype, int T, int I, int interleave, cudaStream_t stream) {
  return zi_gated_act(out, gu, dtype, T, I, interleave, ZI_ACT_SILU, stream);
}

extern "C" int zi_gated_act_partials(void* out, int dtype, const float* partials, int splits, long long split_stride,
                                     int T, int I, int interleave, int act, cudaStream_t stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  if (I % 4 || (uintptr_t)partials % 16 || (uintptr_t)out % 8 || split_stride % 4)
    return zi_refuse("swiglu_partials: needs I %% 4 == 0 and aligned buffers");
  const size_t total_vec = total / 4;
  ZI_DISPATCH_ACT(act, ACT, ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(swiglu_partials_kernel<TT, ACT>, dim3((unsigned)((total_vec + 255) / 256)), dim3(256), 0, stream,
                                   (TT*)out, partials, splits, (size_t)split_stride, I, total_vec, interleave)));
  return zi_check_launch("swiglu_partials");
}

extern "C" int zi_gated_act(void* out, const void* gu, int dtype, int T, int I, int interleave, int act,
                            cudaStream_t stream) {
  if (interleave && (interleave % 8 || I % interleave)) return zi_refuse("swiglu: interleave %d does not fit I = %d", interleave, I);
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  if (I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const size_t total_vec = total / 8;
    const unsigned blocks = (unsigned)((total_vec + threads - 1) / threads);
    ZI_DISPATCH_ACT(act, ACT, ZI_DISPATCH_DTYPE(dtype, TT,
                      zi_launch(swiglu_vec_kernel<TT, ACT>, dim3(blocks), dim3(threads), 0, stream, (TT*)out, (const TT*)gu, I, total_vec, interleave)));
    return zi_check_launch("swiglu");
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  ZI_DISPATCH_ACT(act, ACT, ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(swiglu_kernel<TT, ACT>, dim3(blocks), dim3(threads), 0, stream, (TT*)out, (const TT*)gu, I, total, interleave)));
  return zi_check_launch("swiglu");
}

// --------------------------------------------------------------------- rotary table
// cos/sin [n_pos, d/2] by the 32-bit recipe: exponent = 2i/d, p = theta^exponent,
// inv_freq = 1/p, angle = pos * inv_freq, each step rounded to float.  pow, cos and
// sin are evaluated in double and rounded once, so the table holds the correctly
// rounded value of each 32-bit step.
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int n_pos, int half,
                                  int d, float theta, float factor) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_pos * half) return;
  const int pos = (int)(idx / half), i = (int)(idx % half);
  const float exponent = (float)(2 * i) / (float)d;
  const float p = (float)pow((double)theta, (double)exponent);
  const float inv_freq = (1.0f / p) / factor;      // linear scaling: every frequency divided by `factor` (1: none)
  const float angle = (float)pos * inv_freq;
  cos_t[idx] = (float)cos((double)angle);
  sin_t[idx] = (float)sin((double)angle);
}

extern "C" int zi_rope_table_scaled(float* cos_t, float* sin_t, int n_pos, int d, float theta, float factor,
                                    cudaStream_t stream) {
  if (d <= 0 || d % 2) return zi_refuse("rope_table: head_dim %d is not even", d);
  if (!(factor > 0.f)) return zi_refuse("rope_table: the scaling factor must be positive");
  const size_t total = (size_t)n_pos * (d / 2);
  if (total == 0) return 0;
  zi_launch(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, cos_t, sin_t, n_pos, d / 2, d, theta,
            factor);
  return zi_check_launch("rope_table");
}

// cos/sin [n_pos, half] of the angles pos * freq[i] for frequencies the caller made (a model's own rescaling of
// them), both multiplied by `magnitude`: the angle is a 32-bit product, cos and sin are evaluated in double and
// rounded once.
__global__ void rope_table_freqs_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int n_pos, int half,
                                        const float* __restrict__ freq, float magnitude) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_pos * half) return;
  const int pos = (int)(idx / half), i = (int)(idx % half);
  const float angle = (float)pos * freq[i];
  cos_t[idx] = (float)(cos((double)angle) * (double)magnitude);
  sin_t[idx] = (float)(sin((double)angle) * (double)magnitude);
}

extern "C" int zi_rope_table_freqs(float* cos_t, float* sin_t, int n_pos, int half, const float* freq, float magnitude,
                                   cudaStream_t stream) {
  if (half <= 0 || !freq) return zi_refuse("rope_table: no frequencies");
  const size_t total = (size_t)n_pos * half;
  if (total == 0) return 0;
  zi_launch(rope_table_freqs_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, cos_t, sin_t, n_pos, half, freq,
            magnitude);
  return zi_check_launch("rope_table_freqs");
}

extern "C" int zi_rope_table(float* cos_t, float* sin_t, int n_pos, int d, float theta, cudaStream_t stream) {
  return zi_rope_table_scaled(cos_t, sin_t, n_pos, d, theta, 1.0f, stream);
}

// ------------------------------------------- q/k RMSNorm + rotary + write into pages
// One warp per (token, head) of the fused projection row [q heads | k heads | v heads].
// q heads: normed, rotated, written to q_out (which may be the source itself).  k heads:
// normed, rotated, written to the key page slot of the token.  v heads: copied to the
// value page slot.  The source row is either `src` (activation dtype) or split-K partial
// sums part[z][t][width] that are added in order.  Pages are [page][kv head][offset][d].
template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* src, int src_stride, const float* __restrict__ part,
                                          int splits, size_t zstride, int part_width, T* q_out,
                                          int q_stride, int nq, int nkv, int d, const float* __restrict__ qw,
                                          const float* __restrict__ kw, float eps, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int n_table_pos,
                                          const int* __restrict__ positions, T* __restrict__ kcache,
                                          T* __restrict__ vcache, const int* __restrict__ slots, int page_size,
                                          int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  const int half = d >> 1;
  // one block per token; its warps take the heads in turn
  for (int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5); head < n_heads;
       head += gridDim.y * (blockDim.x >> 5)) {
  auto load = [&](int i) -> float {
    if (part) {
      const float* p = part + (size_t)t * part_width + (size_t)head * d + i;
      float v = 0.f;
      int z = 0;
      for (; z + 4 <= splits; z += 4) {   // four loads in flight, added in order
        const float p0 = p[(size_t)z * zstride], p1 = p[(size_t)(z + 1) * zstride];
        const float p2 = p[(size_t)(z + 2) * zstride], p3 = p[(size_t)(z + 3) * zstride];
        v = (((v + p0) + p1) + p2) + p3;
      }
      for (; z < splits; ++z) v += p[(size_t)z * zstride];
      return v;
    }
    return to_f32(src[(size_t)t * src_stride + (size_t)head * d + i]);
  };

  T* dst;
  if (head < nq) {
    dst = q_out + (size_t)t * q_stride + (size_t)head * d;
  } else {
    const int slot = slots[t];
    if (slot < 0) continue;
    const int kvh = (head - nq) % nkv;
    T* base = head < nq + nkv ? kcache : vcache;
    dst = base + (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * d;
  }
  if (head >= nq + nkv) {  // value head: copy
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(load(i));
    continue;
  }
  // the head's pairs (i, i + d/2) this lane owns, read once into registers (d <= 256)
  constexpr int MAXP = 4;
  float a[MAXP], b[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int i = lane + 32 * j;
    a[j] = b[j] = 0.f;
    if (i < half) {
      a[j] = load(i);
      b[j] = load(i + half);
      ss = sum_squares_step(ss, a[j], b[j]);
    }
  }
  const float* w = head < nq ? qw : kw;
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)d + eps);
  }
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;  // the host refuses such positions
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int i = lane + 32 * j;
    if (i >= half) continue;
    float x = a[j], y = b[j];
    if (w) {
      x = norm_scale(x, w[i], inv);
      y = norm_scale(y, w[i + half], inv);
    }
    if (cos_t) rotate_pair(x, y, cos_t[(size_t)pos * half + i], sin_t[(size_t)pos * half + i]);
    dst[i] = from_f32<T>(x);
    dst[i + half] = from_f32<T>(y);
  }
  }  // heads
}

// The same for many tokens of bfloat16 rows (prompt portions), 16 bytes per access: HALF / 8
// lanes share a (token, head), each with 8 consecutive elements of the head's first half and
// the 8 that pair with them in the second; a warp works on 32 / (HALF / 8) heads at once.
// d in {16, 32, 64, 128, 256}.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_vec_kernel(const __nv_bfloat16* src, int src_stride, __nv_bfloat16* q_out,   // may be the same rows
                              int q_stride, int nq, int nkv, const float* __restrict__ qw,
                              const float* __restrict__ kw, float eps, const float* __restrict__ cos_t,
                              const float* __restrict__ sin_t, int n_table_pos, const int* __restrict__ positions,
                              __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                              const int* __restrict__ slots, int page_size, int n_heads, long long n_items) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HALF = D / 2, LPI = HALF / 8;            // lanes per (token, head)
  const long long item_raw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPI;
  const bool in_range = item_raw < n_items;
  const long long item = in_range ? item_raw : n_items - 1;   // lanes past the end load a valid row and store nothing
  const int sub = threadIdx.x % LPI;
  const int t = (int)(item / n_heads), head = (int)(item % n_heads);
  const int i0 = sub * 8;
  const __nv_bfloat16* sp = src + (size_t)t * src_stride + (size_t)head * D + i0;
  const uint4 ra = *reinterpret_cast<const uint4*>(sp), rb = *reinterpret_cast<const uint4*>(sp + HALF);
  float a[8], b[8];
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
    a[2 * j] = fa.x;
    a[2 * j + 1] = fa.y;
    b[2 * j] = fb.x;
    b[2 * j + 1] = fb.y;
  }
  // the sum of squares of the head, by every lane of the warp (no lane leaves before the shuffles)
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = sum_squares_step(ss, a[j], b[j]);
#pragma unroll
  for (int o = LPI / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, LPI);
  if (!in_range) return;
  __nv_bfloat16* dst;
  if (head < nq) {
    dst = q_out + (size_t)t * q_stride + (size_t)head * D + i0;
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kvh = (head - nq) % nkv;
    __nv_bfloat16* base = head < nq + nkv ? kcache : vcache;
    dst = base + (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * D + i0;
  }
  if (head >= nq + nkv) {        // value head: copy
    *reinterpret_cast<uint4*>(dst) = ra;
    *reinterpret_cast<uint4*>(dst + HALF) = rb;
    return;
  }
  const float* w = head < nq ? qw : kw;
  const float inv = w ? 1.0f / sqrtf(ss / (float)D + eps) : 1.f;
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;  // the host refuses such positions
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (w) {
      a[j] = norm_scale(a[j], w[i0 + j], inv);
      b[j] = norm_scale(b[j], w[i0 + j + HALF], inv);
    }
    if (cos_t) rotate_pair(a[j], b[j], cos_t[(size_t)pos * HALF + i0 + j], sin_t[(size_t)pos * HALF + i0 + j]);
  }
  uint4 oa, ob;
  __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
  __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    qa[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
    qb[j] = __floats2bfloat162_rn(b[2 * j], b[2 * j + 1]);
  }
  *reinterpret_cast<uint4*>(dst) = oa;
  *reinterpret_cast<uint4*>(dst + HALF) = ob;
}

template <int D>
static void launch_qk_vec(const void* src, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv,
                          const float* qw, const float* kw, float eps, const float* cos_t, const float* sin_t,
                          int n_table_pos, const int* positions, void* kcache, void* vcache, const int* slots,
                          int page_size, int n_heads, cudaStream_t stream) {
  const long long n_items = (long long)T * n_heads;
  const long long threads = n_items * (D / 16);
  zi_launch(qk_norm_rope_store_vec_kernel<D>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream,
            (const __nv_bfloat16*)src, src_stride, (__nv_bfloat16*)q_out, q_stride, nq, nkv, qw, kw, eps, cos_t, sin_t,
            n_table_pos, positions, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slots, page_size, n_heads, n_items);
}

extern "C" int zi_qk_norm_rope_store(const void* src, int dtype, int T, int src_stride, const float* partials,
                                     int splits, long long split_stride, void* q_out, int q_stride, int nq, int nkv,
                                     int d, const float* qw, const float* kw, float eps, const float* cos_t,
                                     const float* sin_t, int n_table_pos, const int* positions, void* kcache,
                                     void* vcache, const int* slots, int page_size, int write_kv,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || d % 2 || d > 256) return zi_refuse("qk_norm_rope_store: head_dim %d is not an even number up to 256", d);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("qk_norm_rope_store: cos and sin tables go together");
  if ((src == nullptr) == (partials == nullptr)) return zi_refuse("qk_norm_rope_store: give the rows either whole or as partial sums");
  if (write_kv && (!kcache || !vcache || !slots || page_size <= 0))
    return zi_refuse("qk_norm_rope_store: writing keys and values needs pages and slots");
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  // more than a few tokens of bfloat16 rows: the kernel with 16-byte accesses
  const bool vec = T > 16 && dtype == ZI_BF16 && src && (d == 16 || d == 32 || d == 64 || d == 128 || d == 256) &&
                   src_stride % 8 == 0 && q_stride % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                   (!write_kv || ((uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0)) &&
                   (!qw || (uintptr_t)qw % 16 == 0) && (!kw || (uintptr_t)kw % 16 == 0);
  if (vec) {
#define ZI_QK_VEC(DD)                                                                                            \
  launch_qk_vec<DD>(src, T, src_stride, q_out, q_stride, nq, nkv, qw, kw, eps, cos_t, sin_t, n_table_pos, positions, \
                    kcache, vcache, slots, page_size, n_heads, stream)
    if (d == 16) ZI_QK_VEC(16);
    else if (d == 32) ZI_QK_VEC(32);
    else if (d == 64) ZI_QK_VEC(64);
    else if (d == 128) ZI_QK_VEC(128);
    else ZI_QK_VEC(256);
#undef ZI_QK_VEC
    return zi_check_launch("qk_norm_rope_store");
  }
  // few tokens (decode): a warp per head, so that all heads run at once; many tokens: 8 warps share a token's heads
  const int warps = T <= 256 ? 4 : 8;
  dim3 grid(T, T <= 256 ? (n_heads + warps - 1) / warps : 1);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(qk_norm_rope_store_kernel<TT>, dim3(grid), dim3(warps * 32), 0, stream, 
                                   (const TT*)src, src_stride, partials, splits, (size_t)split_stride, n_heads * d,
                                   (TT*)q_out, q_stride, nq, nkv, d, qw, kw, eps, cos_t, sin_t, n_table_pos, positions,
                                   (TT*)kcache, (TT*)vcache, slots, page_size, write_kv));
  return zi_check_launch("qk_norm_rope_store");
}

// h[i] += sum over splits of part[z][i], in order of z (for consumers that take no partial sums).
__global__ void residual_add_partials_kernel(float* __restrict__ h, const float* __restrict__ part, int splits,
                                             size_t zstride, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float d = 0.f;
  for (int z = 0; z < splits; ++z) d += part[z * zstride + i];
  h[i] += d;
}

extern "C" int zi_residual_add_partials(float* h, const float* partials, int splits, long long split_stride,
                                        long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(residual_add_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, h, partials, splits,
                                                                             (size_t)split_stride, (size_t)n);
  return zi_check_launch("residual_add_partials");
}

// ids[dst[i]] = prev[src[i]] for i < n with dst[i] >= 0: the tokens a step feeds that were
// sampled by the step before it are taken on the device, so the host need not wait for them.
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ prev, const int* __restrict__ dst,
                                    const int* __restrict__ src, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && dst[i] >= 0) ids[dst[i]] = prev[src[i]];
}

extern "C" int zi_patch_tokens(int* ids, const int* prev, const int* dst, const int* src, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, prev, dst, src, n);
  return zi_check_launch("patch_tokens");
}

// ------------------------------- q/k norm + rotation of part of a head + page write, general form
// Rows [q heads | k heads | v heads], or [q heads | k heads] with the values taken from the keys AS
// PROJECTED (before norm and rotation; v_from_k).  The rotation turns the first rot_dims dimensions of a
// head in pairs (i, i + rot_dims/2) by tables [positions, rot_dims/2]; the rest passes unchanged.  One
// warp per (token, head); q is rewritten in place.
template <typename T>
__global__ void qk_prepare_kernel(const T* src, int src_stride, T* q_out, int q_stride, int nq, int nkv, int d,
                                  int rot_dims, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_table_pos,
                                  const int* __restrict__ positions, T* __restrict__ kcache, T* __restrict__ vcache,
                                  const int* __restrict__ slots, int page_size, int v_from_k, int write_kv, int T_,
                                  int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_heads = nq + (write_kv ? (v_from_k ? nkv : 2 * nkv) : 0);
  const int wi = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wi >= T_ * n_heads) return;
  const int t = wi / n_heads, head = wi % n_heads;
  const T* x = src + (size_t)t * src_stride + (size_t)head * d;
  if (head >= nq + nkv) {              // a value head of its own (dv elements, behind all key heads): copy
    const int slot = slots[t];
    if (slot < 0) return;
    const int kvh = head - nq - nkv;
    const T* xv = src + (size_t)t * src_stride + (size_t)(nq + nkv) * d + (size_t)kvh * dv;
    const size_t at = (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * dv;
    for (int i = lane; i < dv; i += 32) vcache[at + i] = xv[i];
    return;
  }
  T* dst;
  T* vdst = nullptr;
  if (head < nq) {
    dst = q_out + (size_t)t * q_stride + (size_t)head * d;
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kvh = (head - nq) % nkv;
    const size_t at = (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * d;
    dst = kcache + at;
    if (v_from_k) vdst = vcache + at;
  }
  const float* w = head < nq ? qw : kw;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = to_f32(x[i]);
    ss = fmaf(v, v, ss);
    if (vdst) vdst[i] = x[i];
  }
  float inv = 1.f;
  if (w) inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;   // the host refuses such positions
  const int half = rot_dims >> 1;
  for (int i = lane; i < half; i += 32) {
    float a = to_f32(x[i]), b = to_f32(x[i + half]);
    if (w) {
      a = norm_scale(a, w[i], inv);
      b = norm_scale(b, w[i + half], inv);
    }
    if (cos_t) rotate_pair(a, b, cos_t[(size_t)pos * half + i], sin_t[(size_t)pos * half + i]);
    dst[i] = from_f32<T>(a);
    dst[i + half] = from_f32<T>(b);
  }
  for (int i = rot_dims + lane; i < d; i += 32) {
    float a = to_f32(x[i]);
    if (w) a = norm_scale(a, w[i], inv);
    dst[i] = from_f32<T>(a);
  }
}

extern "C" int zi_qk_prepare(const void* src, int dtype, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv,
                             int d, int rot_dims, const float* qw, const float* kw, float eps, const float* cos_t,
                             const float* sin_t, int n_table_pos, const int* positions, void* kcache, void* vcache,
                             const int* slots, int page_size, int v_from_k, int write_kv, cudaStream_t stream) {
  return zi_qk_prepare_v(src, dtype, T, src_stride, q_out, q_stride, nq, nkv, d, d, rot_dims, qw, kw, eps, cos_t, sin_t,
                         n_table_pos, positions, kcache, vcache, slots, page_size, v_from_k, write_kv, stream);
}

extern "C" int zi_qk_prepare_v(const void* src, int dtype, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv,
                               int d, int dv, int rot_dims, const float* qw, const float* kw, float eps, const float* cos_t,
                               const float* sin_t, int n_table_pos, const int* positions, void* kcache, void* vcache,
                               const int* slots, int page_size, int v_from_k, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dv <= 0 || (v_from_k && dv != d)) return zi_refuse("qk_prepare: values of %d elements beside keys of %d", dv, d);
  if (d <= 0 || rot_dims < 0 || rot_dims % 2 || rot_dims > d)
    return zi_refuse("qk_prepare: %d rotated dimensions of a head of %d", rot_dims, d);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("qk_prepare: cos and sin tables go together");
  if (write_kv && (!kcache || !vcache || !slots || page_size <= 0)) return zi_refuse("qk_prepare: writing keys and values needs pages and slots");
  const int n_heads = nq + (write_kv ? (v_from_k ? nkv : 2 * nkv) : 0);
  const int warps = 4;
  const unsigned blocks = (unsigned)(((size_t)T * n_heads + warps - 1) / warps);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(qk_prepare_kernel<TT>, dim3(blocks), dim3(warps * 32), 0, stream, (const TT*)src,
                                         src_stride, (TT*)q_out, q_stride, nq, nkv, d, cos_t ? rot_dims : 0, qw, kw, eps, cos_t,
                                         sin_t, n_table_pos, positions, (TT*)kcache, (TT*)vcache, slots, page_size, v_from_k,
                                         write_kv, T, dv));
  return zi_check_launch("qk_prepare");
}

// ------------------------------------------- norm of a sublayer's OUTPUT, then the residual sum
// h += norm(sa * a + sb * b) * w with norm(y) = y / sqrt(mean(y^2) + eps); x_out = h in the activations' type
// (what the next sublayer reads).  b may be absent.  a and b each come whole or as split-K partial sums
// part[z][row][H] that are added in order.  One block per row, 32-bit throughout.
// one operand's value at `at`: whole, or the sum of its partial sums in order, four loads in flight
template <typename TA>
__device__ __forceinline__ float operand_at(const TA* a, const float* ap, int as, size_t az, size_t at) {
  if (!ap) return to_f32(a[at]);
  const float* p = ap + at;
  float v = 0.f;
  int z = 0;
  for (; z + 4 <= as; z += 4) {
    const float p0 = p[(size_t)z * az], p1 = p[(size_t)(z + 1) * az], p2 = p[(size_t)(z + 2) * az], p3 = p[(size_t)(z + 3) * az];
    v = (((v + p0) + p1) + p2) + p3;
  }
  for (; z < as; ++z) v += p[(size_t)z * az];
  return v;
}

// ------------------------- several updates into the residual stream, then one or two norms of it
// h[row] += sum_i scale_i * term_i[row] (+ bias), in the order of the terms; out1 = h * w1 / rms(h), and with w2 also
// out2 = h * w2 / rms(h): two norms of the same row share their root mean square (a block whose two sublayers
// read the same stream).  A term comes whole (float32 or bfloat16) or as split-K partial sums [splits][T][H] added
// in order.  With `rows` (picked rows, repeats allowed) h is left as it is.  One block per row, which it keeps in
// shared memory, so every operand is read once; 32-bit throughout.
struct SumTerm {
  const void* whole;
  const float* part;
  int dtype, splits;
  long long zstride;
  float scale;
};
struct SumTerms {
  SumTerm t[4];
  int n;
};

__device__ __forceinline__ float sum_term_at(const SumTerm& t, size_t at) {
  if (t.part) return operand_at((const float*)nullptr, t.part, t.splits, (size_t)t.zstride, at);
  return t.dtype == ZI_BF16 ? to_f32(((const __nv_bfloat16*)t.whole)[at]) : ((const float*)t.whole)[at];
}

template <typename TO>
__global__ void __launch_bounds__(1024)
sum_norm_pair_kernel(float* __restrict__ h, SumTerms terms, const float* __restrict__ bias, const float* __restrict__ w1,
                     const float* __restrict__ w2, float eps, TO* __restrict__ out1, TO* __restrict__ out2,
                     const int* __restrict__ rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  extern __shared__ float ys[];
  const int r = blockIdx.x;
  const size_t row = (size_t)(rows ? rows[r] : r) * H;
  float ss = 0.f;
  for (int c0 = threadIdx.x; c0 < H; c0 += 4 * blockDim.x) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {      // four columns of a thread at a time: their loads are in flight together
      const int c = c0 + u * blockDim.x;
      v[u] = 0.f;
      if (c < H) {
        v[u] = h[row + c];
        for (int i = 0; i < terms.n; ++i) v[u] = fmaf(terms.t[i].scale, sum_term_at(terms.t[i], row + c), v[u]);
        if (bias) v[u] += bias[c];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * blockDim.x;
      if (c < H) {
        ys[c] = v[u];
        if (!rows && (terms.n > 0 || bias)) h[row + c] = v[u];
        ss = fmaf(v[u], v[u], ss);
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o1 = out1 + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) o1[c] = from_f32<TO>(ys[c] * w1[c] * inv);
  if (w2) {
    TO* o2 = out2 + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o2[c] = from_f32<TO>(ys[c] * w2[c] * inv);
  }
}

// Many rows (a prompt) whose updates all come whole and whose width is a multiple of 4 up to 8,192: 16-byte accesses,
// 256 threads a row, the row held in registers between the sum of squares and the norms.  The terms are added in the
// same order as above, so a row's sum is the same number on either kernel.
template <typename TO>
__global__ void __launch_bounds__(256)
sum_norm_pair_vec_kernel(float* __restrict__ h, SumTerms terms, const float* __restrict__ bias, const float* __restrict__ w1,
                         const float* __restrict__ w2, float eps, TO* __restrict__ out1, TO* __restrict__ out2,
                         const int* __restrict__ rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  constexpr int MAXV = 8;                 // 4-wide pieces per thread
  const int r = blockIdx.x;
  const size_t row = (size_t)(rows ? rows[r] : r) * H;
  const bool writes_h = !rows && (terms.n > 0 || bias);
  float4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 256 + threadIdx.x) * 4;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < H) {
      v[i] = Vec4<float>::load(h + row + c);
      for (int t = 0; t < terms.n; ++t) {
        const SumTerm& term = terms.t[t];
        const float4 u = term.dtype == ZI_BF16 ? Vec4<__nv_bfloat16>::load((const __nv_bfloat16*)term.whole + row + c)
                                               : Vec4<float>::load((const float*)term.whole + row + c);
        v[i] = make_float4(fmaf(term.scale, u.x, v[i].x), fmaf(term.scale, u.y, v[i].y), fmaf(term.scale, u.z, v[i].z),
                           fmaf(term.scale, u.w, v[i].w));
      }
      if (bias) {
        const float4 bv = Vec4<float>::load(bias + c);
        v[i] = make_float4(v[i].x + bv.x, v[i].y + bv.y, v[i].z + bv.z, v[i].w + bv.w);
      }
      if (writes_h) Vec4<float>::store(h + row + c, v[i]);
      ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o1 = out1 + (size_t)r * H;
  TO* o2 = w2 ? out2 + (size_t)r * H : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 256 + threadIdx.x) * 4;
    if (c < H) {
      const float4 a = Vec4<float>::load(w1 + c);
      Vec4<TO>::store(o1 + c, make_float4(v[i].x * a.x * inv, v[i].y * a.y * inv, v[i].z * a.z * inv, v[i].w * a.w * inv));
      if (o2) {
        const float4 b = Vec4<float>::load(w2 + c);
        Vec4<TO>::store(o2 + c, make_float4(v[i].x * b.x * inv, v[i].y * b.y * inv, v[i].z * b.z * inv, v[i].w * b.w * inv));
      }
    }
  }
}

// terms: n_terms entries of (whole, dtype, part, splits, zstride, scale), given as parallel arrays on the host.
extern "C" int zi_sum_norm_pair(float* h, int n_terms, const void* const* whole, const int* dtypes, const float* const* part,
                                const int* splits, const long long* zstride, const float* scales, const float* bias,
                                const float* w1, const float* w2, float eps, void* out1, void* out2, int out_dtype,
                                const int* rows, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0 || H <= 0) return 0;
  if (n_terms < 0 || n_terms > 4) return zi_refuse("sum_norm_pair: %d updates (at most 4)", n_terms);
  if (!w1 || !out1 || (w2 && !out2)) return zi_refuse("sum_norm_pair: a norm needs its weight and its output");
  SumTerms terms = {};
  terms.n = n_terms;
  for (int i = 0; i < n_terms; ++i) {
    if ((whole[i] == nullptr) == (part[i] == nullptr)) return zi_refuse("sum_norm_pair: give update %d either whole or as partial sums", i);
    if (whole[i] && dtypes[i] != ZI_F32 && dtypes[i] != ZI_BF16) return zi_refuse("sum_norm_pair: unknown dtype tag %d", dtypes[i]);
    terms.t[i] = SumTerm{whole[i], part[i], dtypes[i], splits[i], zstride[i], scales[i]};
  }
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return zi_refuse("sum_norm_pair: rows of %d values are more than this kernel holds", H);
  const int threads = H >= 4096 ? 1024 : (H >= 2048 ? 512 : 256);
  auto al16 = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; };
  bool vec = n_rows > 256 && H % 4 == 0 && H <= 8192 && al16(h) && al16(bias) && al16(w1) && al16(w2) && al16(out1) && al16(out2);
  for (int i = 0; i < n_terms; ++i) vec = vec && whole[i] && al16(whole[i]);
  if (vec) {
    ZI_DISPATCH_DTYPE(out_dtype, TO, {
      zi_launch(sum_norm_pair_vec_kernel<TO>, dim3(n_rows), dim3(256), 0, stream, h, terms, bias, w1, w2, eps, (TO*)out1,
                (TO*)out2, rows, H);
    });
    return zi_check_launch("sum_norm_pair");
  }
  ZI_DISPATCH_DTYPE(out_dtype, TO, {
    auto kern = sum_norm_pair_kernel<TO>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return zi_refuse("sum_norm_pair: cannot get %zu bytes of shared memory", smem);
    zi_launch(kern, dim3(n_rows), dim3(threads), smem, stream, h, terms, bias, w1, w2, eps, (TO*)out1, (TO*)out2, rows, H);
  });
  return zi_check_launch("sum_norm_pair");
}

// Many rows (a prompt): the GPU is full of rows, a block of 256 threads reads its row's update twice (the second time
// from cache) and keeps nothing in shared memory.
template <typename TA, typename TB, typename TO>
__global__ void __launch_bounds__(256)
norm_residual_rows_kernel(float* __restrict__ h, const TA* __restrict__ a, const float* __restrict__ ap, int as, size_t az, float sa,
                          const TB* __restrict__ b, const float* __restrict__ bp, int bs, size_t bz, float sb,
                          const float* __restrict__ w, float eps, TO* __restrict__ x_out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t row = (size_t)blockIdx.x * H;
  const bool has_b = b != nullptr || bp != nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float y = sa * operand_at(a, ap, as, az, row + c);
    if (has_b) y = fmaf(sb, operand_at(b, bp, bs, bz, row + c), y);
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float y = sa * operand_at(a, ap, as, az, row + c);
    if (has_b) y = fmaf(sb, operand_at(b, bp, bs, bz, row + c), y);
    const float v = h[row + c] + y * inv * w[c];
    h[row + c] = v;
    if (x_out) x_out[row + c] = from_f32<TO>(v);
  }
}

// Many rows whose updates come whole (no partial sums) and whose width is a multiple of 4 up to 8,192: 16-byte
// accesses, the row's update read once and kept in registers between the sum of squares and the add.
template <typename TA, typename TB, typename TO, bool HAS_B>
__global__ void __launch_bounds__(256)
norm_residual_vec_kernel(float* __restrict__ h, const TA* __restrict__ a, float sa, const TB* __restrict__ b, float sb,
                         const float* __restrict__ w, float eps, TO* __restrict__ x_out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  constexpr int MAXV = 8;                 // 4-wide pieces per thread
  const size_t row = (size_t)blockIdx.x * H;
  float4 y[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 256 + threadIdx.x) * 4;
    y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < H) {
      const float4 va = Vec4<TA>::load(a + row + c);
      y[i] = make_float4(sa * va.x, sa * va.y, sa * va.z, sa * va.w);
      if (HAS_B) {
        const float4 vb = Vec4<TB>::load(b + row + c);
        y[i] = make_float4(fmaf(sb, vb.x, y[i].x), fmaf(sb, vb.y, y[i].y), fmaf(sb, vb.z, y[i].z), fmaf(sb, vb.w, y[i].w));
      }
      ss = fmaf(y[i].x, y[i].x, fmaf(y[i].y, y[i].y, fmaf(y[i].z, y[i].z, fmaf(y[i].w, y[i].w, ss))));
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = (i * 256 + threadIdx.x) * 4;
    if (c < H) {
      const float4 hv = Vec4<float>::load(h + row + c), wv = Vec4<float>::load(w + c);
      const float4 v = make_float4(hv.x + y[i].x * inv * wv.x, hv.y + y[i].y * inv * wv.y, hv.z + y[i].z * inv * wv.z,
                                   hv.w + y[i].w * inv * wv.w);
      Vec4<float>::store(h + row + c, v);
      if (x_out) Vec4<TO>::store(x_out + row + c, v);
    }
  }
}

// Few rows (a decode step): a row's loads are spread over up to 1024 threads, four columns of a thread in flight
// together, and the summed update is kept in shared memory so that partial sums are read once.
template <typename TA, typename TB, typename TO>
__global__ void __launch_bounds__(1024)
norm_residual_kernel(float* __restrict__ h, const TA* __restrict__ a, const float* __restrict__ ap, int as, size_t az, float sa,
                     const TB* __restrict__ b, const float* __restrict__ bp, int bs, size_t bz, float sb,
                     const float* __restrict__ w, float eps, TO* __restrict__ x_out, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  extern __shared__ float ys[];          // the row's summed update (H floats), so that partial sums are read once
  const size_t row = (size_t)blockIdx.x * H;
  const bool has_b = b != nullptr || bp != nullptr;
  float ss = 0.f;
  // four columns of a thread at a time: their loads (and those of their partial sums) are in flight together
  for (int c0 = threadIdx.x; c0 < H; c0 += 4 * blockDim.x) {
    float y[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * blockDim.x;
      y[u] = 0.f;
      if (c < H) {
        y[u] = sa * operand_at(a, ap, as, az, row + c);
        if (has_b) y[u] = fmaf(sb, operand_at(b, bp, bs, bz, row + c), y[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * blockDim.x;
      if (c < H) {
        ys[c] = y[u];
        ss = fmaf(y[u], y[u], ss);
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = h[row + c] + ys[c] * inv * w[c];
    h[row + c] = v;
    if (x_out) x_out[row + c] = from_f32<TO>(v);
  }
}

extern "C" int zi_norm_residual(float* h, const void* a, int a_dtype, const float* a_part, int a_splits, long long a_zstride,
                                float sa, const void* b, int b_dtype, const float* b_part, int b_splits, long long b_zstride,
                                float sb, const float* w, float eps, void* x_out, int out_dtype, int T, int H,
                                cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  if ((a == nullptr) == (a_part == nullptr)) return zi_refuse("norm_residual: give the update either whole or as partial sums");
  if (b && b_part) return zi_refuse("norm_residual: give the second update either whole or as partial sums");
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return zi_refuse("norm_residual: rows of %d values are more than this kernel holds", H);
  // few rows (a decode step): a row's loads are spread over as many threads as it has columns in fours; many rows fill the GPU anyway
  const int threads = H >= 4096 ? 1024 : (H >= 2048 ? 512 : 256);
  auto al16 = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; };
  const bool vec = a && !a_part && !b_part && H % 4 == 0 && H <= 8192 && al16(h) && al16(a) && al16(b) && al16(w) && al16(x_out);
#define ZI_NR(TA, TB, TO)                                                                                               \
  do {                                                                                                                  \
    if (T > 512 && vec) {                                                                                               \
      if (b) zi_launch(norm_residual_vec_kernel<TA, TB, TO, true>, dim3(T), dim3(256), 0, stream, h, (const TA*)a, sa,  \
                       (const TB*)b, sb, w, eps, (TO*)x_out, H);                                                        \
      else zi_launch(norm_residual_vec_kernel<TA, TB, TO, false>, dim3(T), dim3(256), 0, stream, h, (const TA*)a, sa,   \
                     (const TB*)b, sb, w, eps, (TO*)x_out, H);                                                          \
      break;                                                                                                            \
    }                                                                                                                   \
    if (T > 512) {                                                                                                      \
      zi_launch(norm_residual_rows_kernel<TA, TB, TO>, dim3(T), dim3(256), 0, stream, h, (const TA*)a, a_part, a_splits, \
                (size_t)a_zstride, sa, (const TB*)b, b_part, b_splits, (size_t)b_zstride, sb, w, eps, (TO*)x_out, H);   \
      break;                                                                                                            \
    }                                                                                                                   \
    auto kern = norm_residual_kernel<TA, TB, TO>;                                                                       \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return zi_refuse("norm_residual: cannot get %zu bytes of shared memory", smem);                                   \
    zi_launch(kern, dim3(T), dim3(threads), smem, stream, h, (const TA*)a, a_part, a_splits, (size_t)a_zstride, sa, (const TB*)b, \
              b_part, b_splits, (size_t)b_zstride, sb, w, eps, (TO*)x_out, H);                                          \
  } while (0)
  ZI_DISPATCH_DTYPE(a ? a_dtype : ZI_F32, TA, ZI_DISPATCH_DTYPE(b ? b_dtype : ZI_F32, TB, ZI_DISPATCH_DTYPE(out_dtype, TO, ZI_NR(TA, TB, TO))));
#undef ZI_NR
  return zi_check_launch("norm_residual");
}

// the 32-bit residual stream in the activations' type
template <typename TO>
__global__ void cast_rows_kernel(TO* __restrict__ out, const float* __restrict__ h, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<TO>(h[i]);
}

extern "C" int zi_cast_rows(void* out, int out_dtype, const float* h, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  ZI_DISPATCH_DTYPE(out_dtype, TO, zi_launch(cast_rows_kernel<TO>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                                             (TO*)out, h, (size_t)n));
  return zi_check_launch("cast_rows");
}

// x <- relu(x)^2 in place
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float v = fmaxf(to_f32(x[i]), 0.f);
    x[i] = from_f32<T>(v * v);
  }
}

template <typename T>
__global__ void relu2_vec_kernel(T* __restrict__ x, size_t n4) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    float4 v = Vec4<T>::load(x + 4 * i);
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    Vec4<T>::store(x + 4 * i, make_float4(v.x * v.x, v.y * v.y, v.z * v.z, v.w * v.w));
  }
}

extern "C" int zi_relu2(void* x, int dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 == 0 && ((uintptr_t)x & 15) == 0) {
    const size_t n4 = (size_t)n / 4;
    ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(relu2_vec_kernel<TT>, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, stream, (TT*)x, n4));
    return zi_check_launch("relu2");
  }
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(relu2_kernel<TT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (TT*)x, (size_t)n));
  return zi_check_launch("relu2");
}

ZI_TRACE_SETTER(elementwise)

// ------------------------------------------------------------------- small elementwise pieces
// x[i] *= s over a 32-bit array (a model's multiplier on its logits).
__global__ void scale_f32_kernel(float* __restrict__ x, size_t n, float s) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

extern "C" int zi_scale_f32(float* x, long long n, float s, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(scale_f32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (size_t)n, s);
  return zi_check_launch("scale_f32");
}

// out[t, c] = x[t, c] * sigmoid(g[t, c]) for rows of `width` values with free row pitches (an output gate).
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, int ldo, const T* __restrict__ x, int ldx, const T* __restrict__ g,
                                    int ldg, int width, size_t total, int group) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / width;
  const int c = (int)(idx - t * width);
  const float gv = to_f32(g[t * ldg + c / group]);
  out[t * ldo + c] = from_f32<T>(to_f32(x[t * ldx + c]) / (1.0f + expf(-gv)));
}

extern "C" int zi_sigmoid_gate(void* out, int ldo, const void* x, int ldx, const void* g, int ldg, int dtype, int T,
                               int width, cudaStream_t stream) {
  return zi_sigmoid_gate_grouped(out, ldo, x, ldx, g, ldg, dtype, T, width, 1, stream);
}

// The same with one gate value for every `group` neighbouring columns (a gate per head): g has width / group columns.
extern "C" int zi_sigmoid_gate_grouped(void* out, int ldo, const void* x, int ldx, const void* g, int ldg, int dtype, int T,
                                       int width, int group, cudaStream_t stream) {
  const size_t total = (size_t)T * width;
  if (total == 0) return 0;
  if (group <= 0 || width % group) return zi_refuse("sigmoid_gate: %d columns do not form groups of %d", width, group);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(sigmoid_gate_kernel<TT>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                         (TT*)out, ldo, (const TT*)x, ldx, (const TT*)g, ldg, width, total, group));
  return zi_check_launch("sigmoid_gate");
}
