// Split-K for skinny GEMMs (M <= 128: decode-time projections, where the whole problem is one
// stream of the weight matrix through the chip).  With a single row of output tiles there are too
// few tiles to occupy 148 SMs, so the K range is cut into `splits` chunks that run as the batch
// dimension of the tensor-core kernel (each chunk writes an fp32 partial [M, N] into the caller's
// workspace), and this file's second kernel sums the partials and applies the epilogue once.
// The reference reaches the same end with shared-local-memory k-slicing inside a work-group
// (SLM_KS in xla/service/gpu/xetla/gemm/gemm_dispatch.h:183-214); here the slices are CTAs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace gemm {

namespace {

constexpr int kAssumedSms = 148;
constexpr int kSlabElems16 = 64;   // K elements per pipeline stage, 16-bit operands
constexpr int kMinChunk = 512;     // smallest K chunk worth a CTA

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * x * fmaf(0.044715f * x, x, 1.0f);
  const float e = ptx::ex2_approx(-2.885390081777927f * u);
  return __fdividef(x, 1.0f + e);
}
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dtype) {
  if (dtype == IXK_F32) return static_cast<const float*>(p)[i];
  const uint16_t h = static_cast<const uint16_t*>(p)[i];
  return dtype == IXK_BF16 ? __uint_as_float(static_cast<uint32_t>(h) << 16) : __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dtype, float v) {
  if (dtype == IXK_F32) {
    static_cast<float*>(p)[i] = v;
  } else if (dtype == IXK_BF16) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  } else {
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  }
}

struct ReduceArgs {
  const float* partial;  // [splits][M][N]
  int splits, M, N;
  const void* bias;
  const void* c;
  void* d;
  int64_t ldc, ldd;
  int out_dtype, bias_dtype, act;
  float beta;
  int geglu;   // the N columns are [gate | up] halves: out[m, n] = round(gelu(gate)) * round(up), N / 2 columns
};

__device__ __forceinline__ void reduce_epilogue_store(const ReduceArgs& a, int m, int n, float v) {
  if (a.bias != nullptr) v += load_as_f32(a.bias, n, a.bias_dtype);
  if (a.c != nullptr) v = fmaf(a.beta, load_as_f32(a.c, static_cast<int64_t>(m) * a.ldc + n, a.out_dtype), v);
  if (a.act == kActRelu) v = fmaxf(v, 0.0f);
  if (a.act == kActGelu) v = gelu_tanh_f(v);
  store_from_f32(a.d, static_cast<int64_t>(m) * a.ldd + n, a.out_dtype, v);
}

// A thread sums four consecutive columns of one row over the chunks, in chunk order, with the
// loads of all chunks in flight together (kVec: N is a multiple of 4, so the partial planes can be
// read 16 bytes at a time); otherwise one element per thread.
__device__ __forceinline__ float round_to(float v, int dtype) {
  if (dtype == IXK_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dtype == IXK_F16) return __half2float(__float2half_rn(v));
  return v;
}

// GeGLU over the two halves of a [M, 2 N'] product: thread = four consecutive output columns; the
// gate is activated and rounded, the up half rounded, then multiplied (the values a gate GEMM with
// a GELU epilogue, an up GEMM and an elementwise product would have produced one after the other).
__global__ void splitk_reduce_geglu_kernel(const ReduceArgs a) {
  const int half = a.N / 2, h4 = half / 4;
  const int64_t plane4 = static_cast<int64_t>(a.M) * a.N / 4;
  const int64_t total = static_cast<int64_t>(a.M) * h4;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / h4);
    const int n = static_cast<int>(i - static_cast<int64_t>(m) * h4) * 4;
    const float4* gsrc = reinterpret_cast<const float4*>(a.partial) + (static_cast<int64_t>(m) * a.N + n) / 4;
    const float4* usrc = gsrc + h4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
#pragma unroll 4
    for (int s = 0; s < a.splits; ++s) {
      const float4 gv = __ldg(gsrc + s * plane4), uv = __ldg(usrc + s * plane4);
      g.x += gv.x; g.y += gv.y; g.z += gv.z; g.w += gv.w;
      u.x += uv.x; u.y += uv.y; u.z += uv.z; u.w += uv.w;
    }
    const float gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      store_from_f32(a.d, static_cast<int64_t>(m) * a.ldd + n + e, a.out_dtype,
                     round_to(gelu_tanh_f(gs[e]), a.out_dtype) * round_to(us[e], a.out_dtype));
  }
}

template <bool kVec>
__global__ void splitk_reduce_kernel(const ReduceArgs a) {
  const int64_t plane = static_cast<int64_t>(a.M) * a.N;
  if constexpr (kVec) {
    const int64_t total = plane / 4;
    const int n4 = a.N / 4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int m = static_cast<int>(i / n4);
      const int n = static_cast<int>(i - static_cast<int64_t>(m) * n4) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4* src = reinterpret_cast<const float4*>(a.partial) + i;
#pragma unroll 4
      for (int s = 0; s < a.splits; ++s) {
        const float4 v = __ldg(src + s * (plane / 4));
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      reduce_epilogue_store(a, m, n, acc.x);
      reduce_epilogue_store(a, m, n + 1, acc.y);
      reduce_epilogue_store(a, m, n + 2, acc.z);
      reduce_epilogue_store(a, m, n + 3, acc.w);
    }
  } else {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < plane;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
      const int m = static_cast<int>(i / a.N);
      const int n = static_cast<int>(i - static_cast<int64_t>(m) * a.N);
      float v = 0.0f;
      for (int s = 0; s < a.splits; ++s) v += a.partial[s * plane + i];
      reduce_epilogue_store(a, m, n, v);
    }
  }
}

}  // namespace

int split_k_factor(int64_t M, int64_t N, int64_t K, int64_t batch, bool fp8) {
  if (batch != 1 || M > 128 || fp8) return 1;
  const int64_t tiles = (N + 127) / 128;  // one row of 128 x 128 tiles
  if (K % kSlabElems16 != 0) return 1;
  // One CTA per SM at this kernel's shared-memory size, so tiles x chunks run in waves of the SM
  // count: pick the chunk count whose last wave is fullest, charging every further wave for the
  // CTAs' fixed part (set-up, pipeline fill, epilogue).  Every chunk is a whole number of pipeline
  // slabs (no chunk reads into the next) of at least kMinChunk elements; at most four waves.
  auto score = [&](int64_t ctas) {
    const int64_t waves = (ctas + kAssumedSms - 1) / kAssumedSms;
    return static_cast<double>(ctas) / static_cast<double>(waves * kAssumedSms) - 0.04 * static_cast<double>(waves - 1);
  };
  int best = 1;
  double best_score = score(tiles);
  for (int s = 2; s <= 16; ++s) {
    if (K % (static_cast<int64_t>(s) * kSlabElems16) != 0 || K / s < kMinChunk) continue;
    const int64_t ctas = tiles * s;
    if ((ctas + kAssumedSms - 1) / kAssumedSms > 4) continue;
    if (score(ctas) >= best_score - 1e-9) {
      best = s;
      best_score = score(ctas);
    }
  }
  return best;
}

size_t split_k_workspace_bytes(int64_t M, int64_t N, int splits) {
  return splits <= 1 ? 0 : static_cast<size_t>(splits) * M * N * sizeof(float);
}

int launch_split_k(const Problem& p, int splits, void* workspace, const DeviceInfo& dev, cudaStream_t stream, bool geglu) {
  const int64_t chunk = p.K / splits;
  Problem part = p;
  part.K = chunk;
  part.batch = splits;
  part.a_batch_stride = p.a_mn_major ? chunk * p.lda : chunk;
  part.b_batch_stride = p.b_mn_major ? chunk * p.ldb : chunk;
  part.c = nullptr;
  part.bias = nullptr;
  part.beta = 0.0f;
  part.act = kActNone;
  part.d = workspace;
  part.out_dtype = IXK_F32;
  part.ldd = p.N;
  part.d_batch_stride = p.M * p.N;
  part.force_block_n = 128;
  int rc = launch(part, dev, stream);
  if (rc != IXK_OK) return rc;

  ReduceArgs r{};
  r.partial = static_cast<const float*>(workspace);
  r.splits = splits;
  r.M = static_cast<int>(p.M);
  r.N = static_cast<int>(p.N);
  r.bias = p.bias;
  r.c = p.beta != 0.0f ? p.c : nullptr;
  r.d = p.d;
  r.ldc = p.ldc;
  r.ldd = p.ldd;
  r.out_dtype = p.out_dtype;
  r.bias_dtype = p.bias_dtype;
  r.act = p.act;
  r.beta = p.beta;
  r.geglu = geglu ? 1 : 0;
  if (geglu) {
    const int64_t total = p.M * (p.N / 8);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 8 * dev.sm_count) blocks = 8 * dev.sm_count;
    splitk_reduce_geglu_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(r);
    IXK_CUDA_OK(cudaGetLastError());
    count_launch();
    return IXK_OK;
  }
  const bool vec = p.N % 4 == 0 && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0;
  const int64_t total = vec ? p.M * p.N / 4 : p.M * p.N;
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 8 * dev.sm_count) blocks = 8 * dev.sm_count;
  if (vec) splitk_reduce_kernel<true><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(r);
  else splitk_reduce_kernel<false><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(r);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

}  // namespace gemm
}  // namespace ixk
