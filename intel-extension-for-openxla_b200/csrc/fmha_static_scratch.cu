// ixk_fmha_fwd_static_scratch: the attention forward for callers that have no way to hand
// over scratch memory and must not allocate any.
//
// Who that is: a custom-call handler that XLA runs with a fixed buffer assignment and no
// scratch allocator wired to it; a serving loop whose framework has already claimed nearly all
// of HBM for its own pool, so that a cudaMalloc from a library fails or stalls the device; code
// that runs where an allocation is simply not allowed to happen (an allocation synchronises the
// device and can fail, neither of which such a caller can absorb mid-step).
//
// The split-key decode path needs scratch for the per-split partial results.  Here that scratch
// is a fixed array that lives in the library's device image: every GPU that loads libixk.so
// carries IXK_STATIC_SCRATCH_BYTES of it until the process exits.  The entry point forwards to
// the ordinary ixk_fmha_fwd with that array as the workspace, so results are identical to a
// call that passes its own workspace.
#include <mutex>

#include "host_common.h"

namespace {

constexpr size_t kScratchBytes = IXK_STATIC_SCRATCH_BYTES;

// Device-resident scratch.  In host code this name is only a handle for the symbol — it is
// not a device address and must never be passed to a kernel; the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices];  // per device ordinal; nullptr until that device's first call

// Looks up (once per device, with that device current) where the array lives on the current device.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return ixk::fail(IXK_NO_DEVICE, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  }
  if (dev < 0 || dev >= kMaxDevices) return ixk::fail(IXK_NO_DEVICE, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return ixk::fail(IXK_CUDA_ERROR,
                       std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return IXK_OK;
}

}  // namespace

extern "C" {

int ixk_fmha_fwd_static_scratch(const ixk_fmha_desc* desc, const void* q, const void* k, const void* v,
                                const void* bias, void* out, float* lse, void* cuda_stream) {
  IXK_API_RANGE("ixk_fmha_fwd_static_scratch");
  ixk::clear_error();
  if (desc == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "desc is NULL");
  const size_t need = ixk_fmha_fwd_workspace_bytes(desc);
  if (need > kScratchBytes)
    return ixk::fail(IXK_WORKSPACE_TOO_SMALL,
                     "this problem needs " + std::to_string(need) + " bytes of scratch but the built-in scratch holds " +
                         std::to_string(kScratchBytes) + "; call ixk_fmha_fwd with a workspace of your own");
  void* scratch = nullptr;
  if (need > 0) {
    const int rc = scratch_for_current_device(&scratch);
    if (rc != IXK_OK) return rc;
  }
  // Every partial the combine step reads is written by the split kernel of the same call, so
  // nothing in the array has to start at zero and nothing is cleared.
  return ixk_fmha_fwd(desc, q, k, v, bias, out, lse, scratch, need > 0 ? kScratchBytes : 0, cuda_stream);
}

}  // extern "C"
