// Host-side plumbing shared by the entry points: error reporting, the per-device
// status word, TMA tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda, so the library loads on a machine without a driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "ixk.h"

namespace ixk {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const std::string& msg);
void clear_error();

#define IXK_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ::ixk::fail(IXK_CUDA_ERROR, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// What the kernels need to know about the current device.
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  int* status_word = nullptr;  // device memory, one int, zero when clean
};
// Fills `info` for the current device (cached per device, thread-safe).  Returns
// IXK_NO_DEVICE unless the device is compute capability 10.x.
int get_device_info(DeviceInfo* info);

void count_launch(uint64_t n = 1);

// A named NVTX range around an entry point, for timelines of a host program that calls the library
// (the reference marks its thunks through its profiler plug-in instead).  Off unless the
// environment has IXK_NVTX=1 when the library is first used; costs one branch when off.
struct ApiRange {
  explicit ApiRange(const char* name);
  ~ApiRange();
  ApiRange(const ApiRange&) = delete;
  ApiRange& operator=(const ApiRange&) = delete;
  bool on;
};
#define IXK_API_RANGE(name) ::ixk::ApiRange ixk_api_range_(name)

// 2-D .. 4-D tiled tensor map with 128-byte swizzle (or none when box_inner_bytes < 128 is
// impossible to swizzle).  dims/strides innermost first; strides[0] is implied (= elem size),
// strides_bytes[i] is the pitch of dimension i+1.
struct TmapSpec {
  CUtensorMapDataType dtype;
  uint32_t rank;
  uint64_t dims[4];
  uint64_t strides_bytes[3];
  uint32_t box[4];
  bool swizzle128;
  bool swizzle_atom32 = false;  // with swizzle128: exchange 32-byte pieces (by row modulo 4) instead of 16-byte ones
};
int encode_tmap(CUtensorMap* out, const void* base, const TmapSpec& spec);

namespace comm {
// Where a rank's scattered output goes: dest[o] = slot `rank` of the `world` slots ([rows / world]
// rows of row_bytes each) that start at slots_offset in rank o's exchange buffer.  Checks that the
// slots fit and that the communicator is connected and belongs to the current device.
int scatter_targets(ixk_comm* c, size_t slots_offset, long long rows, size_t row_bytes, void** dest, int* world);
}  // namespace comm

}  // namespace ixk
