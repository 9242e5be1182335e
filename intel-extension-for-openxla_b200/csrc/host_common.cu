#include "host_common.h"

#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

namespace ixk {

namespace {
thread_local std::string tl_last_error;
std::atomic<uint64_t> g_launches{0};

// Written by a kernel whose bounded wait gave up; one per device (a module-scope
// device variable exists once in every device that loads this library).
__device__ int g_status_word;

constexpr int kMaxDevices = 64;
std::mutex g_dev_mu;
DeviceInfo g_dev[kMaxDevices];
bool g_dev_ready[kMaxDevices];

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::once_flag g_encode_once;
EncodeFn g_encode = nullptr;

void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = reinterpret_cast<EncodeFn>(fn);
  (void)cudaGetLastError();
}
}  // namespace

int fail(int code, const std::string& msg) {
  tl_last_error = msg;
  return code;
}
void clear_error() { tl_last_error.clear(); }
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {
bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("IXK_NVTX");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}
}  // namespace
ApiRange::ApiRange(const char* name) : on(nvtx_enabled()) {
  if (on) nvtxRangePushA(name);
}
ApiRange::~ApiRange() {
  if (on) nvtxRangePop();
}

int get_device_info(DeviceInfo* info) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(IXK_NO_DEVICE, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  }
  if (dev < 0 || dev >= kMaxDevices) return fail(IXK_NO_DEVICE, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_dev_mu);
  if (!g_dev_ready[dev]) {
    DeviceInfo d;
    d.device = dev;
    IXK_CUDA_OK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    IXK_CUDA_OK(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    IXK_CUDA_OK(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (d.cc_major != 10)
      return fail(IXK_NO_DEVICE, "libixk needs a compute-capability 10.x (B200) device; found " +
                                     std::to_string(d.cc_major) + "." + std::to_string(d.cc_minor));
    void* p = nullptr;
    IXK_CUDA_OK(cudaGetSymbolAddress(&p, g_status_word));
    d.status_word = static_cast<int*>(p);
    IXK_CUDA_OK(cudaMemset(d.status_word, 0, sizeof(int)));
    g_dev[dev] = d;
    g_dev_ready[dev] = true;
  }
  *info = g_dev[dev];
  return IXK_OK;
}

int encode_tmap(CUtensorMap* out, const void* base, const TmapSpec& s) {
  std::call_once(g_encode_once, resolve_encode);
  if (g_encode == nullptr)
    return fail(IXK_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the installed driver");
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  cuuint32_t estr[4];
  for (uint32_t i = 0; i < s.rank; ++i) {
    dims[i] = s.dims[i];
    box[i] = s.box[i];
    estr[i] = 1;
    if (i + 1 < s.rank) strides[i] = s.strides_bytes[i];
  }
  CUresult r = g_encode(out, s.dtype, s.rank, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        !s.swizzle128 ? CU_TENSOR_MAP_SWIZZLE_NONE
                        : s.swizzle_atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::string m = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)) + " (rank " +
                    std::to_string(s.rank) + ", dims";
    for (uint32_t i = 0; i < s.rank; ++i) m += " " + std::to_string(s.dims[i]);
    m += ", box";
    for (uint32_t i = 0; i < s.rank; ++i) m += " " + std::to_string(s.box[i]);
    m += ", strides";
    for (uint32_t i = 0; i + 1 < s.rank; ++i) m += " " + std::to_string(s.strides_bytes[i]);
    m += ")";
    return fail(IXK_INVALID_ARGUMENT, m);
  }
  return IXK_OK;
}

}  // namespace ixk

// ------------------------------------------------------------------ C ABI
extern "C" {

const char* ixk_status_string(int status) {
  switch (status) {
    case IXK_OK: return "OK";
    case IXK_INVALID_ARGUMENT: return "INVALID_ARGUMENT";
    case IXK_UNIMPLEMENTED: return "UNIMPLEMENTED";
    case IXK_WORKSPACE_TOO_SMALL: return "WORKSPACE_TOO_SMALL";
    case IXK_CUDA_ERROR: return "CUDA_ERROR";
    case IXK_NO_DEVICE: return "NO_DEVICE";
    case IXK_DEVICE_TIMEOUT: return "DEVICE_TIMEOUT";
    default: return "UNKNOWN";
  }
}

const char* ixk_last_error(void) { return ixk::tl_last_error.c_str(); }

const char* ixk_version(void) { return "0.1.0"; }

int ixk_device_status(int* status_word) {
  IXK_API_RANGE("ixk_device_status");
  ixk::clear_error();
  if (status_word == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "status_word is NULL");
  ixk::DeviceInfo dev;
  int rc = ixk::get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  IXK_CUDA_OK(cudaDeviceSynchronize());
  int w = 0;
  IXK_CUDA_OK(cudaMemcpy(&w, dev.status_word, sizeof(int), cudaMemcpyDeviceToHost));
  if (w != 0) IXK_CUDA_OK(cudaMemset(dev.status_word, 0, sizeof(int)));
  *status_word = w;
  if (w != 0)
    return ixk::fail(IXK_DEVICE_TIMEOUT, "a device-side wait gave up, site code " + std::to_string(w));
  return IXK_OK;
}

uint64_t ixk_launch_count(void) { return ixk::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
