// Bandwidth-bound attention for a handful of query rows against a long key/value cache
// (decode).  The reference launches its 64-row prefill tile even for one query row
// (xla/service/gpu/xetla/sdp/fmha_policy.h:35-83 via fmha_forward.h:621-646); here the step is
// what it is on the hardware: a stream of K and V through the SMs at HBM speed.
//
//   grid  (splits * ceil(F / rows), N, B)   one (batch, head, pair of queries, key-split) per CTA, 8 warps
//   lane  owns 8 consecutive head-dim elements: one 128-bit load per key for K, one for V
//   score dot product finished with warp-shuffle reductions over the lanes sharing a key
//   softmax online (running max / sum in fp32, exp2 with head_scale*log2(e) folded in)
//
// Each split writes an unnormalised partial (O, max, sum) to scratch; a second small kernel
// merges the splits.  With one split the CTA normalises and stores directly.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fmha_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace fmha {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kUnroll = 4;      // keys in flight per lane group
constexpr int kMinKeysPerSplit = 256;
constexpr int kTargetCtas = 16 * 148;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeArgs {
  int B, N, H, F, T;
  int causal, is_bf16;
  int splits, keys_per_split;
  float scale_log2;
  const uint16_t* q;
  const uint16_t* k;
  const uint16_t* v;
  const uint16_t* bias;
  uint16_t* out;
  float* lse;
  float* partial;  // [B*N*F*splits][H + 2]
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3], bias_strides[3];
};

__device__ __forceinline__ float to_f32(uint16_t h, bool bf16) {
  return bf16 ? __uint_as_float(static_cast<uint32_t>(h) << 16) : __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ void unpack8(const uint4& w, bool bf16, float (&f)[8]) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bf16) {
      f[2 * i] = __uint_as_float(ww[i] << 16);
      f[2 * i + 1] = __uint_as_float(ww[i] & 0xffff0000u);
    } else {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}
__device__ __forceinline__ uint16_t from_f32(float x, bool bf16) {
  return bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
}
// 128-bit streaming load that does not pollute L1 (each K/V byte is used once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// kLanesPerKey lanes cooperate on one key (kLanesPerKey * 8 >= head size).  A CTA serves kQ
// consecutive query rows: every K and V vector is loaded once and used for all of them, so a
// step with a few query rows per sequence (2 <= F <= 16) streams the cache ceil(F / kQ) times,
// not F times.
template <int kLanesPerKey, int kQ>
__global__ void __launch_bounds__(kThreads, 2)
fmha_decode_kernel(const DecodeArgs a) {
  constexpr int kGroups = 32 / kLanesPerKey;  // keys handled side by side in one warp
  constexpr int kHPad = kLanesPerKey * 8;
  __shared__ float sm_acc[kWarps][kQ][kHPad];
  __shared__ float sm_m[kWarps][kQ];
  __shared__ float sm_l[kWarps][kQ];

  const bool bf16 = a.is_bf16 != 0;
  const int split = blockIdx.x % a.splits;
  const int f0 = (blockIdx.x / a.splits) * kQ;  // first query row of this CTA
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = lane / kLanesPerKey;
  const int sub = lane % kLanesPerKey;
  const int d0 = sub * 8;
  const bool dim_ok = d0 < a.H;  // H is a multiple of 8

  int t_begin = split * a.keys_per_split;
  int t_end = min(a.T, t_begin + a.keys_per_split);
  // keys t <= f are visible to row f (top-left anchored): the CTA streams up to its last row's limit
  if (a.causal) t_end = min(t_end, min(f0 + kQ, a.F));

  float qf[kQ][8];
  const uint16_t* bias_row[kQ];
#pragma unroll
  for (int r = 0; r < kQ; ++r) {
    const int f = f0 + r;
    uint4 w = make_uint4(0, 0, 0, 0);
    if (dim_ok && f < a.F)
      w = *reinterpret_cast<const uint4*>(a.q + batch * a.q_strides[0] + head * a.q_strides[1] +
                                          static_cast<int64_t>(f) * a.q_strides[2] + d0);
    unpack8(w, bf16, qf[r]);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[r][i] *= a.scale_log2;
    bias_row[r] = nullptr;
    if (a.bias != nullptr && f < a.F)
      bias_row[r] = a.bias + batch * a.bias_strides[0] + head * a.bias_strides[1] + static_cast<int64_t>(f) * a.bias_strides[2];
  }
  const uint16_t* kbase = a.k + batch * a.k_strides[0] + head * a.k_strides[1] + d0;
  const uint16_t* vbase = a.v + batch * a.v_strides[0] + head * a.v_strides[1] + d0;

  float m_run[kQ], l_run[kQ];
  float acc[kQ][8];
#pragma unroll
  for (int r = 0; r < kQ; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
  }

  // Key index of this lane group: warps interleave, groups inside a warp interleave.  The loop
  // bound is warp-uniform (the shuffles below need every lane); `ok` masks the ragged end.
  constexpr int kStride = kWarps * kGroups;
  for (int base = t_begin + warp * kGroups; base < t_end; base += kStride * kUnroll) {
    const int t0 = base + group;
    uint4 kw[kUnroll], vw[kUnroll];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 + u * kStride;
      ok[u] = t < t_end;
      kw[u] = make_uint4(0, 0, 0, 0);
      vw[u] = make_uint4(0, 0, 0, 0);
      if (ok[u] && dim_ok) {
        kw[u] = ld_stream(kbase + static_cast<int64_t>(t) * a.k_strides[2]);
        vw[u] = ld_stream(vbase + static_cast<int64_t>(t) * a.v_strides[2]);
      }
    }
    float x[kQ][kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float kf[8];
      unpack8(kw[u], bf16, kf);
      const int t = t0 + u * kStride;
#pragma unroll
      for (int r = 0; r < kQ; ++r) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(qf[r][i], kf[i], s);
#pragma unroll
        for (int off = kLanesPerKey / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const bool seen = ok[u] && (kQ == 1 || !a.causal || t <= f0 + r);
        if (seen && bias_row[r] != nullptr) s = fmaf(to_f32(__ldg(bias_row[r] + t), bf16), kLog2e, s);
        x[r][u] = seen ? s : -INFINITY;
      }
    }
    float vf[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) unpack8(vw[u], bf16, vf[u]);
#pragma unroll
    for (int r = 0; r < kQ; ++r) {
      float mx = x[r][0];
#pragma unroll
      for (int u = 1; u < kUnroll; ++u) mx = fmaxf(mx, x[r][u]);
      if (mx > m_run[r]) {
        const float corr = ptx::ex2_approx(m_run[r] - mx);  // 0 when m_run = -inf
        l_run[r] *= corr;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] *= corr;
        m_run[r] = mx;
      }
      if (m_run[r] != -INFINITY) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const float p = ptx::ex2_approx(x[r][u] - m_run[r]);  // 0 for masked / absent keys
          l_run[r] += p;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(p, vf[u][i], acc[r][i]);
        }
      }
    }
  }

  // Merge the lane groups of the warp (butterfly over the group index).
#pragma unroll
  for (int r = 0; r < kQ; ++r) {
#pragma unroll
    for (int off = kLanesPerKey; off < 32; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run[r], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run[r], off);
      const float m_new = fmaxf(m_run[r], m_o);
      const float c_s = (m_run[r] == -INFINITY) ? 0.0f : ptx::ex2_approx(m_run[r] - m_new);
      const float c_o = (m_o == -INFINITY) ? 0.0f : ptx::ex2_approx(m_o - m_new);
      l_run[r] = l_run[r] * c_s + l_o * c_o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[r][i], off);
        acc[r][i] = acc[r][i] * c_s + a_o * c_o;
      }
      m_run[r] = m_new;
    }
    if (group == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[warp][r][d0 + i] = acc[r][i];
      if (sub == 0) {
        sm_m[warp][r] = m_run[r];
        sm_l[warp][r] = l_run[r];
      }
    }
  }
  __syncthreads();

  // Merge the warps; thread d owns head-dim element d.
  const int d = threadIdx.x;
#pragma unroll
  for (int r = 0; r < kQ; ++r) {
    const int f = f0 + r;
    if (f >= a.F) break;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m_all = fmaxf(m_all, sm_m[w][r]);
    float l_all = 0.0f;
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float c = (sm_m[w][r] == -INFINITY) ? 0.0f : ptx::ex2_approx(sm_m[w][r] - m_all);
      l_all += sm_l[w][r] * c;
      if (d < kHPad) o += sm_acc[w][r][d] * c;
    }
    const int64_t row = (static_cast<int64_t>(batch) * a.N + head) * a.F + f;
    if (a.splits == 1) {
      if (d < a.H)
        a.out[batch * a.o_strides[0] + head * a.o_strides[1] + static_cast<int64_t>(f) * a.o_strides[2] + d] =
            from_f32(o / l_all, bf16);
      if (d == 0 && a.lse != nullptr) a.lse[row] = (m_all + log2f(l_all)) * kLn2;
    } else {
      float* part = a.partial + (row * a.splits + split) * (a.H + 2);
      if (d < a.H) part[d] = o;
      if (d == 0) {
        part[a.H] = m_all;
        part[a.H + 1] = l_all;
      }
    }
  }
}

// One CTA per (batch, head, query): merges the key splits.
__global__ void fmha_decode_combine_kernel(const DecodeArgs a) {
  const int64_t row = blockIdx.x;
  const int f = static_cast<int>(row % a.F);
  const int head = static_cast<int>((row / a.F) % a.N);
  const int batch = static_cast<int>(row / (static_cast<int64_t>(a.F) * a.N));
  const bool bf16 = a.is_bf16 != 0;
  const float* part = a.partial + row * a.splits * (a.H + 2);
  float m_all = -INFINITY;
  for (int s = 0; s < a.splits; ++s) m_all = fmaxf(m_all, part[s * (a.H + 2) + a.H]);
  float l_all = 0.0f;
  for (int s = 0; s < a.splits; ++s) {
    const float m_s = part[s * (a.H + 2) + a.H];
    const float c = (m_s == -INFINITY) ? 0.0f : ptx::ex2_approx(m_s - m_all);
    l_all += part[s * (a.H + 2) + a.H + 1] * c;
  }
  for (int d = threadIdx.x; d < a.H; d += blockDim.x) {
    float o = 0.0f;
    for (int s = 0; s < a.splits; ++s) {
      const float m_s = part[s * (a.H + 2) + a.H];
      const float c = (m_s == -INFINITY) ? 0.0f : ptx::ex2_approx(m_s - m_all);
      o += part[s * (a.H + 2) + d] * c;
    }
    a.out[batch * a.o_strides[0] + head * a.o_strides[1] + static_cast<int64_t>(f) * a.o_strides[2] + d] =
        from_f32(o / l_all, bf16);
  }
  if (threadIdx.x == 0 && a.lse != nullptr) a.lse[row] = (m_all + log2f(l_all)) * kLn2;
}

}  // namespace

// Query rows one CTA serves.  Two rows share every K and V load; with four the kernel is bound by
// instruction issue (the per-row dot products and their shuffle reductions) and by the registers
// of four accumulators (one CTA per SM), and ran slower than two passes of two rows.
int decode_rows_per_cta(int F) { return F >= 2 ? 2 : 1; }

int decode_splits(const Problem& p, int /*sm_count*/) {
  const int rows = decode_rows_per_cta(p.F);
  const int64_t base = static_cast<int64_t>(p.B) * p.N * ((p.F + rows - 1) / rows);
  int64_t want = (kTargetCtas + base - 1) / base;
  const int64_t max_splits = (p.T + kMinKeysPerSplit - 1) / kMinKeysPerSplit;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  return static_cast<int>(want);
}

size_t decode_workspace_bytes(const Problem& p, int splits) {
  if (splits <= 1) return 0;
  return static_cast<size_t>(splits) * p.B * p.N * p.F * (p.H + 2) * sizeof(float);
}

int launch_decode(const Problem& p, const DeviceInfo& dev, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream) {
  const int splits = decode_splits(p, dev.sm_count);
  const size_t need = decode_workspace_bytes(p, splits);
  if (need > 0) {
    if (workspace == nullptr || workspace_bytes < need)
      return fail(IXK_WORKSPACE_TOO_SMALL, "attention workspace: need " + std::to_string(need) + " bytes, got " +
                                               std::to_string(workspace_bytes));
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0)
      return fail(IXK_INVALID_ARGUMENT, "attention workspace must be 16-byte aligned");
  }
  if (static_cast<int64_t>(splits) * p.F > 0x7fffffff || p.N > 65535 || p.B > 65535)
    return fail(IXK_UNIMPLEMENTED, "grid too large for the decode kernel");
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  bool vec_ok = aligned(p.q) && aligned(p.k) && aligned(p.v);
  for (int i = 0; i < 3; ++i)
    vec_ok = vec_ok && p.q_strides[i] % 8 == 0 && p.k_strides[i] % 8 == 0 && p.v_strides[i] % 8 == 0;
  if (!vec_ok)
    return fail(IXK_UNIMPLEMENTED, "decode attention needs 16-byte aligned q/k/v and strides that are multiples of 8 elements");

  DecodeArgs a{};
  a.B = p.B;
  a.N = p.N;
  a.H = p.H;
  a.F = p.F;
  a.T = p.T;
  a.causal = p.causal ? 1 : 0;
  a.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
  a.splits = splits;
  a.keys_per_split = (p.T + splits - 1) / splits;
  a.scale_log2 = p.head_scale * kLog2e;
  a.q = static_cast<const uint16_t*>(p.q);
  a.k = static_cast<const uint16_t*>(p.k);
  a.v = static_cast<const uint16_t*>(p.v);
  a.bias = static_cast<const uint16_t*>(p.bias);
  a.out = static_cast<uint16_t*>(p.out);
  a.lse = p.lse;
  a.partial = static_cast<float*>(workspace);
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = p.q_strides[i];
    a.k_strides[i] = p.k_strides[i];
    a.v_strides[i] = p.v_strides[i];
    a.o_strides[i] = p.o_strides[i];
    a.bias_strides[i] = p.bias_strides[i];
  }
  const int rows_per_cta = decode_rows_per_cta(p.F);
  dim3 grid(splits * ((p.F + rows_per_cta - 1) / rows_per_cta), p.N, p.B);
  auto launch_lanes = [&](auto lanes_tag) {
    constexpr int kLanes = decltype(lanes_tag)::value;
    if (rows_per_cta == 1) fmha_decode_kernel<kLanes, 1><<<grid, kThreads, 0, stream>>>(a);
    else fmha_decode_kernel<kLanes, 2><<<grid, kThreads, 0, stream>>>(a);
  };
  if (p.H <= 64) launch_lanes(std::integral_constant<int, 8>{});
  else if (p.H <= 128) launch_lanes(std::integral_constant<int, 16>{});
  else launch_lanes(std::integral_constant<int, 32>{});
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  if (splits > 1) {
    const int64_t rows = static_cast<int64_t>(p.B) * p.N * p.F;
    fmha_decode_combine_kernel<<<static_cast<unsigned>(rows), 128, 0, stream>>>(a);
    IXK_CUDA_OK(cudaGetLastError());
    count_launch();
  }
  return IXK_OK;
}

}  // namespace fmha
}  // namespace ixk
