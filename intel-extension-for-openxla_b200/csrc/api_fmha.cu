// Attention entry point: the host logic of RunFusedMHA
// (xla/service/gpu/xetla_gpu_fused_mha_runner.cc:45-149) — dropout rejection, stride checks,
// dimension derivation — in front of the two kernels.
#include <cmath>

#include "fmha_sm100.h"

namespace ixk {
namespace {

int make_problem(const ixk_fmha_desc* d, const void* q, const void* k, const void* v, const void* bias,
                 void* out, float* lse, fmha::Problem* p, bool need_pointers) {
  if (d == nullptr) return fail(IXK_INVALID_ARGUMENT, "desc is NULL");
  if (d->reserved != 0) return fail(IXK_INVALID_ARGUMENT, "desc.reserved must be 0");
  if (d->dtype != IXK_BF16 && d->dtype != IXK_F16)
    return fail(IXK_UNIMPLEMENTED, "Invalid MHA datatype: BF16 and F16 only");  // runner.cc:145, :209-217
  if (d->dropout_prob != 0.0f) return fail(IXK_UNIMPLEMENTED, "Unimplemented dropout");  // runner.cc:59-61
  if (d->num_batches < 0 || d->num_heads < 0 || d->num_queries < 0 || d->num_keys < 0 || d->head_size < 0)
    return fail(IXK_INVALID_ARGUMENT, "negative dimension");
  if (d->head_size > 256)
    return fail(IXK_UNIMPLEMENTED, "head_size > 256 is not supported");  // fmha_forward.h:642 CHECK(false)
  if (d->head_size % 8 != 0)
    return fail(IXK_UNIMPLEMENTED, "head_size must be a multiple of 8 (16-byte rows)");
  if (!std::isfinite(d->head_scale)) return fail(IXK_INVALID_ARGUMENT, "head_scale is not finite");
  p->dtype = d->dtype;
  p->causal = d->causal != 0;
  p->B = d->num_batches;
  p->N = d->num_heads;
  p->H = d->head_size;
  p->F = d->num_queries;
  p->T = d->num_keys;
  p->head_scale = d->head_scale;
  p->q = q;
  p->k = k;
  p->v = v;
  p->bias = bias;
  p->out = out;
  p->lse = lse;
  for (int i = 0; i < 3; ++i) {
    p->q_strides[i] = d->q_strides[i];
    p->k_strides[i] = d->k_strides[i];
    p->v_strides[i] = d->v_strides[i];
    p->o_strides[i] = d->o_strides[i];
    p->bias_strides[i] = bias != nullptr || !need_pointers ? d->bias_strides[i] : 0;
    if (d->q_strides[i] < 0 || d->k_strides[i] < 0 || d->v_strides[i] < 0 || d->o_strides[i] < 0 ||
        d->bias_strides[i] < 0)
      return fail(IXK_INVALID_ARGUMENT, "negative stride");
  }
  // Stride 0 on a dimension with more than one entry means "one tensor for all of them".  That is
  // a broadcast READ for K and V over heads and batches (multi-query attention) and for the bias
  // (ixk.h); anywhere else it would alias rows of a tensor that is read row by row, or make the
  // writes of different (batch, head, row) triples land on one address.  (The workspace queries
  // pass descriptors whose strides may be unset: they are not checked there.)
  if (need_pointers) {
    const int64_t ext_q[3] = {p->B, p->N, p->F};
    const int64_t ext_k[3] = {p->B, p->N, p->T};
    for (int i = 0; i < 3; ++i) {
      if (ext_q[i] > 1 && d->o_strides[i] == 0)
        return fail(IXK_INVALID_ARGUMENT, "out: stride 0 on a dimension with more than one entry (rows would overwrite each other)");
      if (ext_q[i] > 1 && d->q_strides[i] == 0)
        return fail(IXK_UNIMPLEMENTED, "q: stride 0 (broadcast) is only supported for k, v and bias");
    }
    if (ext_k[2] > 1 && (d->k_strides[2] == 0 || d->v_strides[2] == 0))
      return fail(IXK_UNIMPLEMENTED, "k/v: stride 0 on the key dimension");
  }
  if (need_pointers) {
    if (p->B == 0 || p->N == 0 || p->F == 0) return IXK_OK;
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr)
      return fail(IXK_INVALID_ARGUMENT, "q, k, v and out must be non-NULL");
    if (p->T == 0 || p->H == 0) return fail(IXK_INVALID_ARGUMENT, "num_keys and head_size must be positive");
  }
  return IXK_OK;
}

bool use_decode(const fmha::Problem& p) { return p.F <= fmha::kDecodeMaxQueries; }

}  // namespace
}  // namespace ixk

extern "C" {

size_t ixk_fmha_fwd_workspace_bytes(const ixk_fmha_desc* desc) {
  ixk::fmha::Problem p;
  if (ixk::make_problem(desc, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &p, false) != IXK_OK) return 0;
  if (p.B == 0 || p.N == 0 || p.F == 0 || p.T == 0) return 0;
  if (!ixk::use_decode(p)) return 0;
  return ixk::fmha::decode_workspace_bytes(p, ixk::fmha::decode_splits(p, 148));
}

int ixk_fmha_fwd(const ixk_fmha_desc* desc, const void* q, const void* k, const void* v, const void* bias,
                 void* out, float* lse, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  IXK_API_RANGE("ixk_fmha_fwd");
  ixk::clear_error();
  ixk::fmha::Problem p;
  int rc = ixk::make_problem(desc, q, k, v, bias, out, lse, &p, true);
  if (rc != IXK_OK) return rc;
  if (p.B == 0 || p.N == 0 || p.F == 0) return IXK_OK;
  auto aligned16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
  if (!aligned16(q) || !aligned16(k) || !aligned16(v))
    return ixk::fail(IXK_INVALID_ARGUMENT, "q, k and v must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(out) & 1u) != 0) return ixk::fail(IXK_INVALID_ARGUMENT, "out is misaligned");
  for (int i = 0; i < 3; ++i) {
    if (p.q_strides[i] % 8 != 0 || p.k_strides[i] % 8 != 0 || p.v_strides[i] % 8 != 0)
      return ixk::fail(IXK_UNIMPLEMENTED, "q/k/v strides must be multiples of 8 elements (16 bytes)");
  }
  ixk::DeviceInfo dev;
  if ((rc = ixk::get_device_info(&dev)) != IXK_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (ixk::use_decode(p)) return ixk::fmha::launch_decode(p, dev, workspace, workspace_bytes, stream);
  return ixk::fmha::launch_prefill(p, dev, stream);
}

size_t ixk_fmha_bwd_workspace_bytes(const ixk_fmha_bwd_desc* desc) {
  if (desc == nullptr) return 0;
  ixk::fmha::Problem p;
  if (ixk::make_problem(&desc->fwd, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &p, false) != IXK_OK) return 0;
  return ixk::fmha::bwd_workspace_bytes(p);
}

int ixk_fmha_bwd(const ixk_fmha_bwd_desc* desc, const void* q, const void* k, const void* v, const void* out,
                 const void* bias, const void* grad_out, const float* lse, void* dq, void* dk, void* dv,
                 void* workspace, size_t workspace_bytes, void* cuda_stream) {
  IXK_API_RANGE("ixk_fmha_bwd");
  ixk::clear_error();
  if (desc == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "desc is NULL");
  ixk::fmha::BwdProblem bp;
  int rc = ixk::make_problem(&desc->fwd, q, k, v, bias, const_cast<void*>(out), const_cast<float*>(lse), &bp.fwd, true);
  if (rc != IXK_OK) return rc;
  const ixk::fmha::Problem& p = bp.fwd;
  if (p.B == 0 || p.N == 0 || (p.F == 0 && p.T == 0)) return IXK_OK;
  if (p.F == 0 || p.T == 0)
    return ixk::fail(IXK_UNIMPLEMENTED, "attention backward with an empty query or key axis");
  if (grad_out == nullptr || lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr)
    return ixk::fail(IXK_INVALID_ARGUMENT, "grad_out, lse, dq, dk and dv must be non-NULL");
  auto aligned16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(grad_out) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return ixk::fail(IXK_INVALID_ARGUMENT, "q, k, v, out, grad_out, dq, dk and dv must be 16-byte aligned");
  for (int i = 0; i < 3; ++i) {
    bp.do_strides[i] = desc->do_strides[i];
    bp.dq_strides[i] = desc->dq_strides[i];
    bp.dk_strides[i] = desc->dk_strides[i];
    bp.dv_strides[i] = desc->dv_strides[i];
    if (bp.do_strides[i] < 0 || bp.dq_strides[i] < 0 || bp.dk_strides[i] < 0 || bp.dv_strides[i] < 0)
      return ixk::fail(IXK_INVALID_ARGUMENT, "negative stride");
    {
      // The gradients are written once per (batch, head, row): no zero strides.  K and V shared
      // between heads (stride 0) would need dK / dV summed over those heads, which this kernel
      // does not do.
      const int64_t ext_q = i == 0 ? p.B : (i == 1 ? p.N : p.F);
      const int64_t ext_k = i == 2 ? p.T : ext_q;
      if ((ext_q > 1 && bp.dq_strides[i] == 0) || (ext_k > 1 && (bp.dk_strides[i] == 0 || bp.dv_strides[i] == 0)))
        return ixk::fail(IXK_INVALID_ARGUMENT, "dq/dk/dv: stride 0 on a dimension with more than one entry");
      if ((ext_q > 1 && bp.do_strides[i] == 0) || (ext_k > 1 && (p.k_strides[i] == 0 || p.v_strides[i] == 0)))
        return ixk::fail(IXK_UNIMPLEMENTED, "attention backward with a broadcast (stride 0) k, v or grad_out");
    }
    if (p.q_strides[i] % 8 != 0 || p.k_strides[i] % 8 != 0 || p.v_strides[i] % 8 != 0 || p.o_strides[i] % 8 != 0 ||
        bp.do_strides[i] % 8 != 0 ||
        bp.dq_strides[i] % 8 != 0 || bp.dk_strides[i] % 8 != 0 || bp.dv_strides[i] % 8 != 0)
      return ixk::fail(IXK_UNIMPLEMENTED, "q/k/v/out/grad_out/dq/dk/dv strides must be multiples of 8 elements (16 bytes)");
  }
  bp.grad_out = grad_out;
  bp.dq = dq;
  bp.dk = dk;
  bp.dv = dv;
  ixk::DeviceInfo dev;
  if ((rc = ixk::get_device_info(&dev)) != IXK_OK) return rc;
  return ixk::fmha::launch_bwd(bp, dev, workspace, workspace_bytes, static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
