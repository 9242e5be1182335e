// Interface between the attention entry point and the two attention kernels.
#pragma once

#include "host_common.h"

namespace ixk {
namespace fmha {

// Validated attention problem; strides in elements, innermost (head_size) stride 1.
struct Problem {
  int dtype = IXK_BF16;
  bool causal = false;
  int B = 0, N = 0, H = 0, F = 0, T = 0;
  float head_scale = 1.0f;
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  const void* bias = nullptr;
  void* out = nullptr;
  float* lse = nullptr;
  int64_t q_strides[3] = {0, 0, 0};
  int64_t k_strides[3] = {0, 0, 0};
  int64_t v_strides[3] = {0, 0, 0};
  int64_t o_strides[3] = {0, 0, 0};
  int64_t bias_strides[3] = {0, 0, 0};
};

// Queries-per-(batch,head) at or below which the bandwidth-bound split-key kernel is used.
constexpr int kDecodeMaxQueries = 16;

// ---- tcgen05 prefill kernel (fmha_prefill_sm100.cu)
int launch_prefill(const Problem& p, const DeviceInfo& dev, cudaStream_t stream);

// ---- split-key decode kernel (fmha_decode_sm100.cu)
// Number of key splits chosen for a problem, and the scratch it needs:
// splits * B*N*F * (H + 2) floats (partial O, running max, running sum).
int decode_splits(const Problem& p, int sm_count);
size_t decode_workspace_bytes(const Problem& p, int splits);
int launch_decode(const Problem& p, const DeviceInfo& dev, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream);

// ---- tcgen05 backward kernels (fmha_bwd_sm100.cu)
// `fwd` carries q, k, v, bias, the forward's output (`out`, read only) and row statistic (`lse`).
struct BwdProblem {
  Problem fwd;
  const void* grad_out = nullptr;
  void* dq = nullptr;
  void* dk = nullptr;
  void* dv = nullptr;
  int64_t do_strides[3] = {0, 0, 0};
  int64_t dq_strides[3] = {0, 0, 0};
  int64_t dk_strides[3] = {0, 0, 0};
  int64_t dv_strides[3] = {0, 0, 0};
};
// fp32 scratch: -lse*log2e and rowsum(dO*O) per padded query row, and the dQ accumulator.
size_t bwd_workspace_bytes(const Problem& p);
int launch_bwd(const BwdProblem& p, const DeviceInfo& dev, void* workspace, size_t workspace_bytes,
               cudaStream_t stream);

// ---- head sizes above 128 (fmha_bwd_wide.cu): the same gradients as a chain of batched GEMMs
// over a group of heads at a time, with the score-sized intermediates in `scratch`
// (bwd_wide_scratch_bytes); neg_lse2 / delta are the prepare kernel's per-row arrays [B*N, f_pad].
size_t bwd_wide_scratch_bytes(const Problem& p);
int launch_bwd_wide(const BwdProblem& p, const DeviceInfo& dev, const float* neg_lse2, const float* delta, int f_pad,
                    void* scratch, cudaStream_t stream);

}  // namespace fmha
}  // namespace ixk
