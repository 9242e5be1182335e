// Attention backward for head sizes above 128 (the reference's fmha_bwd_policy_64x128x256,
// xla/service/gpu/xetla/sdp/fmha_policy.h:107-116, dispatched at fmha_backward.h:931-938).
//
// With 256-wide heads the dK and dV accumulators of a 128-key block alone fill the 512 columns of
// tensor memory, so the single-kernel scheme of fmha_bwd_sm100.cu (S^T, dP^T, dK, dV resident
// together) does not fit.  This path evaluates the same formulas (fmha_backward.h:489-700) as a
// chain over a group of heads at a time, with the score-sized intermediates in the caller's
// workspace and every matrix product on the library's tcgen05 GEMM kernel (heads = GEMM batches):
//   S   = Q.K^T                                   fp32  [g, F, T]
//   P   = exp(head_scale*S + bias - lse), masked  16-bit (P is a matmul operand from here on)
//   dV  = P^T.dO
//   dP  = dO.V^T                                  fp32, over S
//   dS  = P * (dP - D)                            16-bit, over P
//   dK  = head_scale * dS^T.Q,   dQ = head_scale * dS.K
// Rounding is the fused kernel's: P and dS rounded to the element type, all sums in fp32, each
// gradient rounded once.  Not a flash kernel: the scores make a round trip through HBM (about
// 12 bytes per score element) and a causal mask skips no work; it exists so that 256-wide heads
// (both decoder-layer configurations) have a backward at all.  D and -lse*log2(e) come from the
// shared prepare kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "fmha_sm100.h"
#include "gemm_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace fmha {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr size_t kChunkBudget = static_cast<size_t>(192) << 20;   // score-sized scratch per group of heads

struct ScoreArgs {
  int g, F, T, t_pad, f_pad;   // heads in this group, queries, keys, score row pitch, row pitch of the per-row arrays
  int causal, is_bf16;
  float scale_log2;
  const float* s32;            // [g, F, t_pad]  S, later dP
  uint16_t* p16;               // [g, F, t_pad]  P, later dS
  const float* neg_lse2;       // rows of this group's first head: [g, f_pad]
  const float* delta;
  const uint16_t* bias;        // at this (batch, first head); nullptr = none
  int64_t bias_head_stride, bias_row_stride;
};

__device__ __forceinline__ float bits_to_f32(uint16_t h, int is_bf16) {
  return is_bf16 ? __uint_as_float(static_cast<uint32_t>(h) << 16) : __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint16_t f32_to_bits(float x, int is_bf16) {
  return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
}

// One thread per 4 consecutive keys of one (head, query) row: 16 bytes of scores in, 8 bytes out.
template <bool kSecond>
__global__ void score_kernel(const ScoreArgs a) {
  const int quads = a.t_pad / 4;
  const int64_t total = static_cast<int64_t>(a.g) * a.F * quads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int tq = static_cast<int>(i % quads);
    const int64_t row = i / quads;                 // head * F + f
    const int f = static_cast<int>(row % a.F);
    const int h = static_cast<int>(row / a.F);
    const int t0 = tq * 4;
    const float4 s = *reinterpret_cast<const float4*>(a.s32 + row * a.t_pad + t0);
    const float sv[4] = {s.x, s.y, s.z, s.w};
    uint16_t* prow = a.p16 + row * a.t_pad + t0;
    uint16_t o[4];
    if (!kSecond) {
      // P = exp2(S*scale*log2e + bias*log2e - lse*log2e); 0 where masked or past the last key
      const float nl = a.neg_lse2[static_cast<int64_t>(h) * a.f_pad + f];
      const uint16_t* brow = a.bias == nullptr ? nullptr : a.bias + h * a.bias_head_stride + f * a.bias_row_stride;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + j;
        float x = fmaf(sv[j], a.scale_log2, nl);
        if (brow != nullptr && t < a.T) x = fmaf(bits_to_f32(brow[t], a.is_bf16), kLog2e, x);
        const bool keep = t < a.T && !(a.causal && t > f);
        o[j] = f32_to_bits(keep ? ptx::ex2_approx(x) : 0.0f, a.is_bf16);
      }
    } else {
      // dS = P * (dP - D)
      const float d = a.delta[static_cast<int64_t>(h) * a.f_pad + f];
      const uint2 pw = *reinterpret_cast<const uint2*>(prow);
      const uint16_t pv[4] = {static_cast<uint16_t>(pw.x & 0xffffu), static_cast<uint16_t>(pw.x >> 16),
                              static_cast<uint16_t>(pw.y & 0xffffu), static_cast<uint16_t>(pw.y >> 16)};
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = f32_to_bits(bits_to_f32(pv[j], a.is_bf16) * (sv[j] - d), a.is_bf16);
    }
    uint2 w;
    w.x = static_cast<uint32_t>(o[0]) | (static_cast<uint32_t>(o[1]) << 16);
    w.y = static_cast<uint32_t>(o[2]) | (static_cast<uint32_t>(o[3]) << 16);
    *reinterpret_cast<uint2*>(prow) = w;
  }
}

int t_pad_of(int T) { return (T + 7) / 8 * 8; }

}  // namespace

int bwd_wide_heads_per_group(const Problem& p) {
  const size_t per_head = static_cast<size_t>(p.F) * t_pad_of(p.T) * 6;   // fp32 + 16-bit per score
  if (per_head == 0) return 1;
  const size_t fit = kChunkBudget / per_head;
  return static_cast<int>(std::min<size_t>(std::max<size_t>(fit, 1), static_cast<size_t>(std::max(p.N, 1))));
}

size_t bwd_wide_scratch_bytes(const Problem& p) {
  const size_t scores = static_cast<size_t>(bwd_wide_heads_per_group(p)) * p.F * t_pad_of(p.T);
  return (scores * 4 + 255) / 256 * 256 + (scores * 2 + 255) / 256 * 256;
}

int launch_bwd_wide(const BwdProblem& bp, const DeviceInfo& dev, const float* neg_lse2, const float* delta, int f_pad,
                    void* scratch, cudaStream_t stream) {
  const Problem& p = bp.fwd;
  const int g_max = bwd_wide_heads_per_group(p);
  const int t_pad = t_pad_of(p.T);
  const size_t scores = static_cast<size_t>(g_max) * p.F * t_pad;
  float* s32 = static_cast<float*>(scratch);
  uint16_t* p16 = reinterpret_cast<uint16_t*>(static_cast<unsigned char*>(scratch) + (scores * 4 + 255) / 256 * 256);
  const uint32_t fmt = p.dtype == IXK_BF16 ? 1u : 0u;

  auto ptr16 = [](const void* base, int64_t elems) { return static_cast<const void*>(static_cast<const uint16_t*>(base) + elems); };
  auto out16 = [](void* base, int64_t elems) { return static_cast<void*>(static_cast<uint16_t*>(base) + elems); };
  // One batched product.  a: [M,K] with K contiguous (a_t = false) or M contiguous (a_t = true);
  // b: [K,N] with N contiguous (b_n = true) or K contiguous (b_n = false).
  auto product = [&](int64_t M, int64_t N, int64_t K, int g, const void* a, bool a_t, int64_t lda, int64_t a_bs, const void* b,
                     bool b_n, int64_t ldb, int64_t b_bs, void* d, int64_t ldd, int64_t d_bs, int out_dtype, float scale) {
    gemm::Problem q;
    q.M = M; q.N = N; q.K = K; q.batch = g;
    q.kind = gemm::kKindF16;
    q.ab_dtype = p.dtype;
    q.a_fmt = q.b_fmt = fmt;
    q.a = a; q.a_mn_major = a_t; q.lda = lda; q.a_batch_stride = a_bs;
    q.b = b; q.b_mn_major = b_n; q.ldb = ldb; q.b_batch_stride = b_bs;
    q.d = d; q.ldd = ldd; q.d_batch_stride = d_bs; q.ldc = ldd; q.c_batch_stride = d_bs;
    q.out_dtype = out_dtype;
    q.bias_dtype = p.dtype;
    q.acc_scale = scale;
    return gemm::launch(q, dev, stream);
  };
  const int64_t score_bs = static_cast<int64_t>(p.F) * t_pad;
  int rc;
  for (int b = 0; b < p.B; ++b) {
    for (int n0 = 0; n0 < p.N; n0 += g_max) {
      const int g = std::min(g_max, p.N - n0);
      const void* q = ptr16(p.q, b * p.q_strides[0] + n0 * p.q_strides[1]);
      const void* k = ptr16(p.k, b * p.k_strides[0] + n0 * p.k_strides[1]);
      const void* v = ptr16(p.v, b * p.v_strides[0] + n0 * p.v_strides[1]);
      const void* dO = ptr16(bp.grad_out, b * bp.do_strides[0] + n0 * bp.do_strides[1]);
      // S = Q.K^T
      if ((rc = product(p.F, p.T, p.H, g, q, false, p.q_strides[2], p.q_strides[1], k, false, p.k_strides[2], p.k_strides[1],
                        s32, t_pad, score_bs, IXK_F32, 1.0f)) != IXK_OK) return rc;
      ScoreArgs sa{};
      sa.g = g; sa.F = p.F; sa.T = p.T; sa.t_pad = t_pad; sa.f_pad = f_pad;
      sa.causal = p.causal ? 1 : 0;
      sa.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
      sa.scale_log2 = p.head_scale * kLog2e;
      sa.s32 = s32;
      sa.p16 = p16;
      sa.neg_lse2 = neg_lse2 + (static_cast<int64_t>(b) * p.N + n0) * f_pad;
      sa.delta = delta + (static_cast<int64_t>(b) * p.N + n0) * f_pad;
      sa.bias = p.bias == nullptr ? nullptr
                                  : static_cast<const uint16_t*>(p.bias) + b * p.bias_strides[0] + n0 * p.bias_strides[1];
      sa.bias_head_stride = p.bias_strides[1];
      sa.bias_row_stride = p.bias_strides[2];
      const int64_t work = static_cast<int64_t>(g) * p.F * (t_pad / 4);
      const int grid = static_cast<int>(std::min<int64_t>((work + 255) / 256, static_cast<int64_t>(dev.sm_count) * 16));
      score_kernel<false><<<grid, 256, 0, stream>>>(sa);
      IXK_CUDA_OK(cudaGetLastError());
      count_launch();
      // dV = P^T.dO
      if ((rc = product(p.T, p.H, p.F, g, p16, true, t_pad, score_bs, dO, true, bp.do_strides[2], bp.do_strides[1],
                        out16(bp.dv, b * bp.dv_strides[0] + n0 * bp.dv_strides[1]), bp.dv_strides[2], bp.dv_strides[1],
                        p.dtype, 1.0f)) != IXK_OK) return rc;
      // dP = dO.V^T (over S)
      if ((rc = product(p.F, p.T, p.H, g, dO, false, bp.do_strides[2], bp.do_strides[1], v, false, p.v_strides[2], p.v_strides[1],
                        s32, t_pad, score_bs, IXK_F32, 1.0f)) != IXK_OK) return rc;
      score_kernel<true><<<grid, 256, 0, stream>>>(sa);
      IXK_CUDA_OK(cudaGetLastError());
      count_launch();
      // dK = head_scale * dS^T.Q
      if ((rc = product(p.T, p.H, p.F, g, p16, true, t_pad, score_bs, q, true, p.q_strides[2], p.q_strides[1],
                        out16(bp.dk, b * bp.dk_strides[0] + n0 * bp.dk_strides[1]), bp.dk_strides[2], bp.dk_strides[1],
                        p.dtype, p.head_scale)) != IXK_OK) return rc;
      // dQ = head_scale * dS.K
      if ((rc = product(p.F, p.H, p.T, g, p16, false, t_pad, score_bs, k, true, p.k_strides[2], p.k_strides[1],
                        out16(bp.dq, b * bp.dq_strides[0] + n0 * bp.dq_strides[1]), bp.dq_strides[2], bp.dq_strides[1],
                        p.dtype, p.head_scale)) != IXK_OK) return rc;
    }
  }
  return IXK_OK;
}

}  // namespace fmha
}  // namespace ixk
