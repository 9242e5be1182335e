// Self-test of the bounded device-side wait that every tensor-core kernel of this library uses.
//
// One CTA of two warps: warp 0 waits on an mbarrier phase that nothing will ever complete, with a
// cycle budget given by the caller; warp 1 waits on a second barrier that warp 0 was meant to
// complete.  The first wait must run out, record its site code in the device status word and
// raise the CTA's abort flag; the second must then leave through the abort flag instead of
// running out its own budget; the kernel must return.  Nothing here faults or hangs: giving up
// IS the behaviour under test.
#include "host_common.h"
#include "ptx.cuh"

namespace ixk {
namespace {

enum : int { kSiteSelfTestFirst = 901, kSiteSelfTestSecond = 902 };

__global__ void __launch_bounds__(64, 1) bounded_wait_kernel(long long limit, int* status_word, long long* cycles_out) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bars[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&bars[1]), 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  ptx::AbortCtl ctl{&abort_flag, status_word};
  const long long t0 = clock64();
  if (lane == 0) {
    if (warp == 0) {
      // nobody arrives on bars[0]
      if (ptx::mbar_wait_limit(ptx::smem_u32(&bars[0]), 0, ctl, kSiteSelfTestFirst, limit))
        ptx::mbar_arrive(ptx::smem_u32(&bars[1]));
    } else {
      // a far larger budget: this wait ends because warp 0 raised the abort flag
      (void)ptx::mbar_wait_limit(ptx::smem_u32(&bars[1]), 0, ctl, kSiteSelfTestSecond, limit * 1000);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && cycles_out != nullptr) *cycles_out = clock64() - t0;
}

}  // namespace
}  // namespace ixk

extern "C" int ixk_selftest_bounded_wait(long long limit_cycles, long long* cycles_out_device, void* cuda_stream) {
  ixk::clear_error();
  if (limit_cycles <= 0 || limit_cycles > 100000000LL)
    return ixk::fail(IXK_INVALID_ARGUMENT, "limit_cycles must be in (0, 1e8]: the self-test is meant to give up within milliseconds");
  ixk::DeviceInfo dev;
  int rc = ixk::get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  ixk::bounded_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(limit_cycles, dev.status_word,
                                                                                cycles_out_device);
  IXK_CUDA_OK(cudaGetLastError());
  ixk::count_launch();
  return IXK_OK;
}
