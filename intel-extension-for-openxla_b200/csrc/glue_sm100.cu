// The memory-bound steps between the custom calls of a decoder layer: row normalisation
// (LayerNorm / RMSNorm, with or without a learned gain), rotary embedding (interleaved pairs as in
// GPT-J, or half-split pairs as in Gemma) applied in place to the q and k slices of a fused QKV
// projection, and the residual add that closes the block.
// XLA emits these as loop fusions around the custom calls (they are not custom calls in the
// reference); they live here so that a layer built from the library's GEMM and attention calls is
// not dominated by many small framework kernels.  Each is one pass over its operands with 16-byte
// accesses: the bound is HBM bandwidth, the cost is (bytes read + bytes written) / bandwidth.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace ixk {
namespace glue {

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormVecs = 4;          // 16-byte vectors a thread keeps in registers: cols <= 8192
constexpr int kVecElems = 8;          // 16-bit elements per 16-byte vector

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (kBf16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}
template <bool kBf16>
__device__ __forceinline__ float round_trip(float v) {   // value after a store in the 16-bit type
  if constexpr (kBf16) return __bfloat162float(__float2bfloat16_rn(v));
  else return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                    // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < kNormThreads / 32 ? scratch[lane] : 0.0f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

// One CTA per row; the row stays in registers between the statistics and the write.
// `gain` (may be null): y = normalised * (gain_offset + gain[col]), one rounding.
template <bool kBf16, bool kRms>
__global__ void __launch_bounds__(kNormThreads) row_norm_kernel(const uint4* x, uint4* y,  // may be one buffer: no __restrict__
                                                                int cols, int64_t ldx_vec, int64_t ldy_vec, float eps,
                                                                const uint4* __restrict__ gain, float gain_offset) {
  __shared__ float scratch[kNormThreads / 32];
  const int nvec = cols / kVecElems;
  const uint4* xr = x + static_cast<int64_t>(blockIdx.x) * ldx_vec;
  uint4* yr = y + static_cast<int64_t>(blockIdx.x) * ldy_vec;
  float v[kNormVecs][kVecElems];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int idx = threadIdx.x + i * kNormThreads;
    if (idx < nvec) {
      const uint4 w = xr[idx];
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack2<kBf16>(words[j]);
        v[i][2 * j] = f.x;
        v[i][2 * j + 1] = f.y;
        sum += kRms ? f.x * f.x + f.y * f.y : f.x + f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kVecElems; ++j) v[i][j] = 0.0f;
    }
  }
  const float inv_n = 1.0f / static_cast<float>(cols);
  float mean = 0.0f, rstd;
  if constexpr (kRms) {
    rstd = rsqrtf(block_sum(sum, scratch) * inv_n + eps);
  } else {
    mean = block_sum(sum, scratch) * inv_n;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormVecs; ++i) {
      if (threadIdx.x + i * kNormThreads < nvec) {
#pragma unroll
        for (int j = 0; j < kVecElems; ++j) {
          const float d = v[i][j] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
    rstd = rsqrtf(block_sum(sq, scratch) * inv_n + eps);
  }
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int idx = threadIdx.x + i * kNormThreads;
    if (idx < nvec) {
      uint32_t words[4];
      if (gain != nullptr) {
        const uint4 gw = gain[idx];
        const uint32_t gwords[4] = {gw.x, gw.y, gw.z, gw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = unpack2<kBf16>(gwords[j]);
          words[j] = pack2<kBf16>((v[i][2 * j] - mean) * rstd * (gain_offset + g.x),
                                  (v[i][2 * j + 1] - mean) * rstd * (gain_offset + g.y));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          words[j] = pack2<kBf16>((v[i][2 * j] - mean) * rstd, (v[i][2 * j + 1] - mean) * rstd);
      }
      yr[idx] = make_uint4(words[0], words[1], words[2], words[3]);
    }
  }
}

// One thread per 16-byte vector = four (even, odd) pairs of one head of one token.
template <bool kBf16>
__global__ void rotary_kernel(uint4* __restrict__ x, const float4* __restrict__ cos_t, const float4* __restrict__ sin_t,
                              int64_t total_vecs, int vecs_per_head, int heads, int seq_len,
                              int64_t token_stride_vec, int64_t head_stride_vec) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int vec = static_cast<int>(i % vecs_per_head);
    const int64_t th = i / vecs_per_head;
    const int head = static_cast<int>(th % heads);
    const int64_t token = th / heads;
    const int pos = static_cast<int>(token % seq_len);
    uint4* p = x + token * token_stride_vec + head * head_stride_vec + vec;
    const uint4 w = *p;
    const float4 c = cos_t[static_cast<int64_t>(pos) * vecs_per_head + vec];
    const float4 s = sin_t[static_cast<int64_t>(pos) * vecs_per_head + vec];
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack2<kBf16>(words[j]);
      out[j] = pack2<kBf16>(f.x * cs[j] - f.y * sn[j], f.x * sn[j] + f.y * cs[j]);
    }
    *p = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// Half-split rotary (the convention of the Gemma and Llama families): element i < rotary_dim / 2
// pairs with element i + rotary_dim / 2.  One thread per 16-byte vector of the first half and its
// partner vector in the second half.
template <bool kBf16>
__global__ void rotary_half_kernel(uint4* __restrict__ x, const float4* __restrict__ cos_t, const float4* __restrict__ sin_t,
                                   int64_t total_vecs, int vecs_per_half, int heads, int seq_len,
                                   int64_t token_stride_vec, int64_t head_stride_vec) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int vec = static_cast<int>(i % vecs_per_half);
    const int64_t th = i / vecs_per_half;
    const int head = static_cast<int>(th % heads);
    const int64_t token = th / heads;
    const int pos = static_cast<int>(token % seq_len);
    uint4* p1 = x + token * token_stride_vec + head * head_stride_vec + vec;
    uint4* p2 = p1 + vecs_per_half;
    const uint4 w1 = *p1, w2 = *p2;
    // 8 angles per vector: two float4 of the [seq_len, rotary_dim / 2] tables
    const int64_t t = (static_cast<int64_t>(pos) * vecs_per_half + vec) * 2;
    const float4 c0 = cos_t[t], c1 = cos_t[t + 1], s0 = sin_t[t], s1 = sin_t[t + 1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t a[4] = {w1.x, w1.y, w1.z, w1.w}, b[4] = {w2.x, w2.y, w2.z, w2.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f1 = unpack2<kBf16>(a[j]), f2 = unpack2<kBf16>(b[j]);
      o1[j] = pack2<kBf16>(f1.x * cs[2 * j] - f2.x * sn[2 * j], f1.y * cs[2 * j + 1] - f2.y * sn[2 * j + 1]);
      o2[j] = pack2<kBf16>(f2.x * cs[2 * j] + f1.x * sn[2 * j], f2.y * cs[2 * j + 1] + f1.y * sn[2 * j + 1]);
    }
    *p1 = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *p2 = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// This step's keys and values into the cache (the dynamic-update-slice of a decode step): one
// thread per 16-byte vector of one (batch, head) row of K or V.
__global__ void kv_append_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new, uint4* __restrict__ k_cache,
                                 uint4* __restrict__ v_cache, int64_t total_vecs, int vecs_per_head, int heads,
                                 int64_t new_batch_vec, int64_t new_head_vec, int64_t cache_batch_vec, int64_t cache_head_vec,
                                 int64_t cache_offset_vec) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < 2 * total_vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const bool is_v = i >= total_vecs;
    const int64_t j = is_v ? i - total_vecs : i;
    const int vec = static_cast<int>(j % vecs_per_head);
    const int64_t bh = j / vecs_per_head;
    const int head = static_cast<int>(bh % heads);
    const int64_t b = bh / heads;
    const int64_t src = b * new_batch_vec + head * new_head_vec + vec;
    const int64_t dst = cache_offset_vec + b * cache_batch_vec + head * cache_head_vec + vec;
    if (is_v) v_cache[dst] = v_new[src];
    else k_cache[dst] = k_new[src];
  }
}

// out = x + round(partial + bias): the sum with the bias is rounded to the storage type first,
// like a framework that materialises (partial + bias) before the residual add.
template <bool kBf16>
__global__ void residual_add_kernel(const uint4* x, const uint4* partial,  // out may alias either: no __restrict__
                                    const uint4* __restrict__ bias, uint4* out, int64_t total_vecs,
                                    int vecs_per_row) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vecs;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 a = x[i], p = partial[i];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, pw[4] = {p.x, p.y, p.z, p.w};
    uint32_t bw[4] = {0, 0, 0, 0};
    if (bias != nullptr) {
      const uint4 b = bias[i % vecs_per_row];
      bw[0] = b.x; bw[1] = b.y; bw[2] = b.z; bw[3] = b.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = unpack2<kBf16>(aw[j]), fp = unpack2<kBf16>(pw[j]), fb = unpack2<kBf16>(bw[j]);
      const float t0 = bias != nullptr ? round_trip<kBf16>(fp.x + fb.x) : fp.x;
      const float t1 = bias != nullptr ? round_trip<kBf16>(fp.y + fb.y) : fp.y;
      o[j] = pack2<kBf16>(fa.x + t0, fa.y + t1);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int elementwise_grid(int64_t total_vecs, int threads, int sm_count) {
  const int64_t want = (total_vecs + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count) * 8;     // eight resident CTAs of 256 threads per SM
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace
}  // namespace glue
}  // namespace ixk

using namespace ixk;

extern "C" {

static int row_norm_impl(int dtype, int kind, int64_t rows, int64_t cols, const void* x, int64_t ldx, void* y, int64_t ldy,
                         float eps, const void* gain, float gain_offset, void* stream) {
  clear_error();
  if (gain != nullptr && !glue::aligned16(gain)) return fail(IXK_INVALID_ARGUMENT, "row_norm: gain must be 16-byte aligned");
  if (dtype != IXK_BF16 && dtype != IXK_F16) return fail(IXK_UNIMPLEMENTED, "row_norm: dtype must be BF16 or F16");
  if (kind != IXK_NORM_LAYER && kind != IXK_NORM_RMS) return fail(IXK_INVALID_ARGUMENT, "row_norm: unknown kind");
  if (rows < 0 || cols <= 0 || (rows > 0 && (x == nullptr || y == nullptr)))
    return fail(IXK_INVALID_ARGUMENT, "row_norm: null or negative argument");
  if (cols % glue::kVecElems || ldx % glue::kVecElems || ldy % glue::kVecElems || ldx < cols || ldy < cols ||
      !glue::aligned16(x) || !glue::aligned16(y))
    return fail(IXK_INVALID_ARGUMENT, "row_norm: cols and row strides must be multiples of 8 elements, pointers 16-byte aligned");
  if (cols > glue::kNormThreads * glue::kNormVecs * glue::kVecElems)
    return fail(IXK_UNIMPLEMENTED, "row_norm: rows longer than 8192 elements");
  if (rows > 0x7fffffff) return fail(IXK_UNIMPLEMENTED, "row_norm: more than 2^31-1 rows");
  DeviceInfo info;
  if (int st = get_device_info(&info)) return st;
  if (rows == 0) return IXK_OK;
  const dim3 grid(static_cast<unsigned>(rows));
  auto s = static_cast<cudaStream_t>(stream);
  const uint4* xv = static_cast<const uint4*>(x);
  uint4* yv = static_cast<uint4*>(y);
  const uint4* gv = static_cast<const uint4*>(gain);
  const int64_t lx = ldx / glue::kVecElems, ly = ldy / glue::kVecElems;
  const int c = static_cast<int>(cols);
  if (dtype == IXK_BF16) {
    if (kind == IXK_NORM_RMS) glue::row_norm_kernel<true, true><<<grid, glue::kNormThreads, 0, s>>>(xv, yv, c, lx, ly, eps, gv, gain_offset);
    else glue::row_norm_kernel<true, false><<<grid, glue::kNormThreads, 0, s>>>(xv, yv, c, lx, ly, eps, gv, gain_offset);
  } else {
    if (kind == IXK_NORM_RMS) glue::row_norm_kernel<false, true><<<grid, glue::kNormThreads, 0, s>>>(xv, yv, c, lx, ly, eps, gv, gain_offset);
    else glue::row_norm_kernel<false, false><<<grid, glue::kNormThreads, 0, s>>>(xv, yv, c, lx, ly, eps, gv, gain_offset);
  }
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

int ixk_row_norm(int dtype, int kind, int64_t rows, int64_t cols, const void* x, int64_t ldx, void* y, int64_t ldy,
                 float eps, void* stream) {
  IXK_API_RANGE("ixk_row_norm");
  return row_norm_impl(dtype, kind, rows, cols, x, ldx, y, ldy, eps, nullptr, 0.0f, stream);
}

int ixk_row_norm_gain(int dtype, int kind, int64_t rows, int64_t cols, const void* x, int64_t ldx, const void* gain,
                      float gain_offset, void* y, int64_t ldy, float eps, void* stream) {
  IXK_API_RANGE("ixk_row_norm_gain");
  if (gain == nullptr) {
    clear_error();
    return fail(IXK_INVALID_ARGUMENT, "row_norm: gain is NULL");
  }
  return row_norm_impl(dtype, kind, rows, cols, x, ldx, y, ldy, eps, gain, gain_offset, stream);
}

static int rotary_impl(bool half_split, int dtype, void* x, int64_t tokens, int64_t seq_len, int64_t heads, int64_t rotary_dim,
                       int64_t token_stride, int64_t head_stride, const float* cos_table, const float* sin_table,
                       void* stream) {
  clear_error();
  if (half_split && rotary_dim % (2 * glue::kVecElems))
    return fail(IXK_INVALID_ARGUMENT, "rotary: the half-split form needs rotary_dim to be a multiple of 16 elements");
  if (dtype != IXK_BF16 && dtype != IXK_F16) return fail(IXK_UNIMPLEMENTED, "rotary: dtype must be BF16 or F16");
  if (tokens < 0 || seq_len <= 0 || heads <= 0 || rotary_dim <= 0 ||
      (tokens > 0 && (x == nullptr || cos_table == nullptr || sin_table == nullptr)))
    return fail(IXK_INVALID_ARGUMENT, "rotary: null or non-positive argument");
  if (tokens % seq_len) return fail(IXK_INVALID_ARGUMENT, "rotary: tokens must be a multiple of seq_len");
  if (rotary_dim % glue::kVecElems || token_stride % glue::kVecElems || head_stride % glue::kVecElems ||
      head_stride < rotary_dim || !glue::aligned16(x) || !glue::aligned16(cos_table) || !glue::aligned16(sin_table))
    return fail(IXK_INVALID_ARGUMENT, "rotary: rotary_dim and strides must be multiples of 8 elements, pointers 16-byte aligned");
  DeviceInfo info;
  if (int st = get_device_info(&info)) return st;
  const int vph = static_cast<int>(rotary_dim / glue::kVecElems) / (half_split ? 2 : 1);
  const int64_t total = tokens * heads * vph;
  if (total == 0) return IXK_OK;
  const int grid = glue::elementwise_grid(total, 256, info.sm_count);
  auto s = static_cast<cudaStream_t>(stream);
  auto* xv = static_cast<uint4*>(x);
  auto* cv = reinterpret_cast<const float4*>(cos_table);
  auto* sv = reinterpret_cast<const float4*>(sin_table);
  const int h = static_cast<int>(heads), sl = static_cast<int>(seq_len);
  const int64_t ts = token_stride / glue::kVecElems, hs = head_stride / glue::kVecElems;
  if (half_split) {
    if (dtype == IXK_BF16) glue::rotary_half_kernel<true><<<grid, 256, 0, s>>>(xv, cv, sv, total, vph, h, sl, ts, hs);
    else glue::rotary_half_kernel<false><<<grid, 256, 0, s>>>(xv, cv, sv, total, vph, h, sl, ts, hs);
  } else {
    if (dtype == IXK_BF16) glue::rotary_kernel<true><<<grid, 256, 0, s>>>(xv, cv, sv, total, vph, h, sl, ts, hs);
    else glue::rotary_kernel<false><<<grid, 256, 0, s>>>(xv, cv, sv, total, vph, h, sl, ts, hs);
  }
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

int ixk_rotary_interleaved(int dtype, void* x, int64_t tokens, int64_t seq_len, int64_t heads, int64_t rotary_dim,
                           int64_t token_stride, int64_t head_stride, const float* cos_table, const float* sin_table,
                           void* stream) {
  IXK_API_RANGE("ixk_rotary_interleaved");
  return rotary_impl(false, dtype, x, tokens, seq_len, heads, rotary_dim, token_stride, head_stride, cos_table, sin_table, stream);
}

int ixk_rotary_half(int dtype, void* x, int64_t tokens, int64_t seq_len, int64_t heads, int64_t rotary_dim,
                    int64_t token_stride, int64_t head_stride, const float* cos_table, const float* sin_table,
                    void* stream) {
  IXK_API_RANGE("ixk_rotary_half");
  return rotary_impl(true, dtype, x, tokens, seq_len, heads, rotary_dim, token_stride, head_stride, cos_table, sin_table, stream);
}

int ixk_kv_append(int dtype, int64_t batch, int64_t heads, int64_t head_dim, const void* k_new, const void* v_new,
                  int64_t new_batch_stride, int64_t new_head_stride, void* k_cache, void* v_cache, int64_t cache_batch_stride,
                  int64_t cache_token_stride, int64_t cache_head_stride, int64_t position, void* stream) {
  IXK_API_RANGE("ixk_kv_append");
  clear_error();
  if (dtype != IXK_BF16 && dtype != IXK_F16) return fail(IXK_UNIMPLEMENTED, "kv_append: dtype must be BF16 or F16");
  if (batch < 0 || heads <= 0 || head_dim <= 0 || position < 0 ||
      (batch > 0 && (k_new == nullptr || v_new == nullptr || k_cache == nullptr || v_cache == nullptr)))
    return fail(IXK_INVALID_ARGUMENT, "kv_append: null or negative argument");
  if (head_dim % glue::kVecElems || new_batch_stride % glue::kVecElems || new_head_stride % glue::kVecElems ||
      cache_batch_stride % glue::kVecElems || cache_token_stride % glue::kVecElems || cache_head_stride % glue::kVecElems ||
      new_head_stride < head_dim || cache_head_stride < head_dim || !glue::aligned16(k_new) || !glue::aligned16(v_new) ||
      !glue::aligned16(k_cache) || !glue::aligned16(v_cache))
    return fail(IXK_INVALID_ARGUMENT, "kv_append: head_dim and strides must be multiples of 8 elements, pointers 16-byte aligned");
  DeviceInfo info;
  if (int st = get_device_info(&info)) return st;
  const int vph = static_cast<int>(head_dim / glue::kVecElems);
  const int64_t total = batch * heads * vph;
  if (total == 0) return IXK_OK;
  const int grid = glue::elementwise_grid(2 * total, 256, info.sm_count);
  glue::kv_append_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new), static_cast<uint4*>(k_cache),
      static_cast<uint4*>(v_cache), total, vph, static_cast<int>(heads), new_batch_stride / glue::kVecElems,
      new_head_stride / glue::kVecElems, cache_batch_stride / glue::kVecElems, cache_head_stride / glue::kVecElems,
      position * (cache_token_stride / glue::kVecElems));
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

int ixk_residual_add(int dtype, int64_t rows, int64_t cols, const void* x, const void* partial, const void* bias,
                     void* out, void* stream) {
  IXK_API_RANGE("ixk_residual_add");
  clear_error();
  if (dtype != IXK_BF16 && dtype != IXK_F16) return fail(IXK_UNIMPLEMENTED, "residual_add: dtype must be BF16 or F16");
  if (rows < 0 || cols <= 0 || (rows > 0 && (x == nullptr || partial == nullptr || out == nullptr)))
    return fail(IXK_INVALID_ARGUMENT, "residual_add: null or negative argument");
  if (cols % glue::kVecElems || !glue::aligned16(x) || !glue::aligned16(partial) || !glue::aligned16(out) ||
      (bias != nullptr && !glue::aligned16(bias)))
    return fail(IXK_INVALID_ARGUMENT, "residual_add: cols must be a multiple of 8, pointers 16-byte aligned");
  DeviceInfo info;
  if (int st = get_device_info(&info)) return st;
  const int64_t total = rows * (cols / glue::kVecElems);
  if (total == 0) return IXK_OK;
  const int grid = glue::elementwise_grid(total, 256, info.sm_count);
  auto s = static_cast<cudaStream_t>(stream);
  const int vpr = static_cast<int>(cols / glue::kVecElems);
  if (dtype == IXK_BF16)
    glue::residual_add_kernel<true><<<grid, 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(partial),
                                                         static_cast<const uint4*>(bias), static_cast<uint4*>(out), total, vpr);
  else
    glue::residual_add_kernel<false><<<grid, 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(partial),
                                                          static_cast<const uint4*>(bias), static_cast<uint4*>(out), total, vpr);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

}  // extern "C"
