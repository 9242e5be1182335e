// All-reduce over NVLink peer memory for the row-parallel projections of a tensor-parallel layer.
//
// Replaces the reference's in-process collective (xla/service/gpu/ccl_ops.cc: allreduce_dpcpp
// :98-246, dispatched by sycl_allreduce :604-789).  The idea is the reference's: every rank can
// address every other rank's buffer, so rank r reduces slice r of all send buffers with plain
// loads and writes the result into all receive buffers with plain stores; 16-bit floats are
// summed in fp32 (:674-676).  What differs is everything around it.  The reference meets its
// participants on the host (a mutex, a condition variable and two stream waits per call); here
// the ranks are separate processes, one per GPU, and they meet on the device: every CTA trades a
// generation number with the same CTA of every peer through flags in the peers' memory, before
// it reads (the peers' partial sums are complete) and before it exits (the peers are done with
// this rank's memory).  No host work per call, so a layer step with its all-reduces inside
// replays as one CUDA graph.
//
// Two algorithms:
//   one-shot  every rank reads all `world` buffers in full and keeps the sum: world x the bytes
//             over NVLink but a single exchange, for latency-bound messages (the 393 KB partials
//             of a decode step); the residual add that follows a row-parallel projection can be
//             fused in, so that exchange + add are one launch;
//   two-shot  the reference's scheme (reduce a slice, broadcast it): 2 x the bytes, for
//             bandwidth-bound messages (the 67 MB partial of a prefill layer).
// Only plain ld.global / st.global touch peer memory: no TMA, no multicast.
// Every flag wait is bounded: a wait that runs out records a site code in the device status
// word (ixk_device_status) and the kernel returns; the communicator is then unusable.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "host_common.h"

namespace ixk {
namespace comm {

constexpr int kMaxRanks = IXK_COMM_MAX_RANKS;
constexpr int kMaxBlocks = 64;   // CTAs of one all-reduce launch = flag slots per rank
constexpr int kThreads = 512;
constexpr size_t kHeaderBytes = 8192;
constexpr long long kDefaultWaitCycles = 2000000000LL;  // about one second
enum : int { kSiteStart = 301, kSiteEnd = 302 };

// At the start of every rank's allocation.  sig[phase][b][r] is written by CTA b of rank r:
// phase 0 before the data is read, phase 1 before the kernel exits.
enum : int { kPhaseStart = 0, kPhaseDone = 1 };
struct Flags {
  uint32_t sig[2][kMaxBlocks][kMaxRanks];
  uint32_t counter[kMaxBlocks];  // local: the generation CTA slot b used last
};
static_assert(sizeof(Flags) <= kHeaderBytes, "flag header");

struct Args {
  Flags* flags[kMaxRanks];
  const void* in[kMaxRanks];
  void* out[kMaxRanks];  // two-shot: every rank's output; one-shot: out[0] is this rank's output
  const void* x;         // epilogue: out = x + round(round(sum) [+ bias[col]]); nullptr = plain sum
  const void* bias;
  long long cols;
  size_t count;          // elements
  int rank, world, kind;
  int skip_end;          // one-shot only: leave without waiting for the peers (see ixk_comm_set_alternating)
  long long wait_limit;
  int* status_word;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Thread r < world tells CTA blockIdx.x of rank r that this CTA has reached generation `gen`, and
// waits until that CTA has said the same.  The release / acquire pair at system scope orders this
// CTA's earlier writes (made visible to the signalling threads by the __syncthreads before)
// ahead of the peer's later reads.  Returns false in every thread of the CTA if a wait ran out.
__device__ __forceinline__ bool exchange(const Args& a, int phase, uint32_t gen, int site, int* abort_smem) {
  __syncthreads();
  if (threadIdx.x < a.world && static_cast<int>(threadIdx.x) != a.rank) {
    const int peer = threadIdx.x;
    st_release_sys(&a.flags[peer]->sig[phase][blockIdx.x][a.rank], gen);
    const uint32_t* mine = &a.flags[a.rank]->sig[phase][blockIdx.x][peer];
    const long long t0 = clock64();
    uint32_t spins = 0;
    // (>=, wrap-safe: a peer that left without the second meeting may already have announced the
    // next generation here)
    while (static_cast<int32_t>(ld_acquire_sys(mine) - gen) < 0) {
      if ((++spins & 63u) == 0 && clock64() - t0 > a.wait_limit) {
        atomicCAS(a.status_word, 0, site);
        *abort_smem = 1;
        break;
      }
    }
  }
  __syncthreads();
  return *reinterpret_cast<volatile int*>(abort_smem) == 0;
}

template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const void* p, size_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ void store1(void* p, size_t i, float f) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(f);
  }
  static __device__ __forceinline__ float round1(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
};
template <>
struct Vec<__half> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const void* p, size_t i) {
    return __half2float(static_cast<const __half*>(p)[i]);
  }
  static __device__ __forceinline__ void store1(void* p, size_t i, float f) {
    static_cast<__half*>(p)[i] = __float2half_rn(f);
  }
  static __device__ __forceinline__ float round1(float f) { return __half2float(__float2half_rn(f)); }
};
template <>
struct Vec<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float load1(const void* p, size_t i) { return static_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, size_t i, float f) { static_cast<float*>(p)[i] = f; }
  static __device__ __forceinline__ float round1(float f) { return f; }
};

__device__ __forceinline__ float combine(float a, float b, int kind) {
  switch (kind) {
    case IXK_REDUCE_PRODUCT: return a * b;
    case IXK_REDUCE_MIN: return fminf(a, b);
    case IXK_REDUCE_MAX: return fmaxf(a, b);
    default: return a + b;
  }
}

enum : int { kOneShot = 0, kTwoShotMode = 1, kReduceScatter = 2, kAllGather = 3 };

// kWorld > 0: the rank loop is unrolled and all loads of a vector are in flight together;
// kWorld == 0: any world size up to kMaxRanks.  Ranks are always combined in the order
// 0, 1, ..., world - 1, so every rank computes the same bits.
// kMode: one-shot all-reduce (every rank reads everything), two-shot all-reduce (reduce a slice,
// write it to all ranks), reduce-scatter (the first half of the two-shot: rank r keeps the sum of
// slice r; reducescatter_dpcpp, ccl_ops.cc:518-559) and all-gather (the second half: rank r's
// piece goes to slot r of every rank's buffer; ccl_ops.cc:268-294).
template <typename T, int kWorld, int kMode>
__global__ void __launch_bounds__(kThreads) all_reduce_kernel(const Args a) {
  constexpr bool kTwoShot = kMode == kTwoShotMode;
  using V = Vec<T>;
  constexpr int E = V::kElems;
  __shared__ int abort_smem;
  if (threadIdx.x == 0) abort_smem = 0;
  const int world = kWorld > 0 ? kWorld : a.world;
  const uint32_t gen = a.flags[a.rank]->counter[blockIdx.x] + 1;
  if (world > 1 && !exchange(a, kPhaseStart, gen, kSiteStart, &abort_smem)) return;

  const size_t vecs = a.count / E;
  size_t v_begin = 0, v_end = vecs;
  if (kTwoShot) {  // this rank's slice; the last rank also takes what does not divide (ccl_ops.cc:109-114)
    const size_t per = vecs / world;
    v_begin = per * a.rank;
    v_end = a.rank == world - 1 ? vecs : v_begin + per;
  }
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  if (kMode == kAllGather) {
    // a.count = elements per rank (whole vectors); in[0] is this rank's piece, out[r] every rank's gathered buffer
    for (size_t v = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; v < vecs; v += stride) {
      const uint4 piece = static_cast<const uint4*>(a.in[0])[v];
      for (int r = 0; r < world; ++r) static_cast<uint4*>(a.out[r])[static_cast<size_t>(a.rank) * vecs + v] = piece;
    }
    if (world > 1 && !exchange(a, kPhaseDone, gen, kSiteEnd, &abort_smem)) return;
    if (threadIdx.x == 0) a.flags[a.rank]->counter[blockIdx.x] = gen;
    return;
  }
  if (kMode == kReduceScatter) {  // a.count = elements per rank: slice r of every contribution is [r * count, (r + 1) * count)
    v_begin = static_cast<size_t>(a.rank) * vecs;
    v_end = v_begin + vecs;
  }
  for (size_t v = v_begin + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; v < v_end; v += stride) {
    float acc[E];
    if (kWorld > 0) {
      uint4 d[kWorld > 0 ? kWorld : 1];
#pragma unroll
      for (int r = 0; r < kWorld; ++r) d[r] = ld_peer(static_cast<const uint4*>(a.in[r]) + v);
      V::unpack(d[0], acc);
#pragma unroll
      for (int r = 1; r < kWorld; ++r) {
        float f[E];
        V::unpack(d[r], f);
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = combine(acc[i], f[i], a.kind);
      }
    } else {
      V::unpack(ld_peer(static_cast<const uint4*>(a.in[0]) + v), acc);
      for (int r = 1; r < world; ++r) {
        float f[E];
        V::unpack(ld_peer(static_cast<const uint4*>(a.in[r]) + v), f);
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = combine(acc[i], f[i], a.kind);
      }
    }
    if (kMode != kReduceScatter && a.x != nullptr) {
      // out = x + round(round(sum) + bias): every intermediate is rounded to the storage type, so
      // that the result has the bits of an all-reduce followed by the separate residual add
      float xf[E];
      V::unpack(static_cast<const uint4*>(a.x)[v], xf);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = V::round1(acc[i]);
      if (a.bias != nullptr) {
        float bf[E];
        V::unpack(static_cast<const uint4*>(a.bias)[(v * E % a.cols) / E], bf);
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] = V::round1(acc[i] + bf[i]);
      }
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] += xf[i];
    }
    if (kTwoShot) {
      const uint4 packed = V::pack(acc);
      for (int r = 0; r < world; ++r) static_cast<uint4*>(a.out[r])[v] = packed;
    } else if (kMode == kReduceScatter) {
      static_cast<uint4*>(a.out[0])[v - v_begin] = V::pack(acc);
    } else {
      static_cast<uint4*>(a.out[0])[v] = V::pack(acc);
    }
  }
  // elements behind the last whole 16-byte vector (one thread of the rank that owns the tail)
  if (kMode != kReduceScatter && blockIdx.x == 0 && threadIdx.x == 0 && (!kTwoShot || a.rank == world - 1)) {
    for (size_t i = vecs * E; i < a.count; ++i) {
      float s = V::load1(a.in[0], i);
      for (int r = 1; r < world; ++r) s = combine(s, V::load1(a.in[r], i), a.kind);
      if (kTwoShot) {
        for (int r = 0; r < world; ++r) V::store1(a.out[r], i, s);
      } else {
        if (a.x != nullptr) {
          s = V::round1(s);
          if (a.bias != nullptr) s = V::round1(s + V::load1(a.bias, i % a.cols));
          s += V::load1(a.x, i);
        }
        V::store1(a.out[0], i, s);
      }
    }
  }
  if (world > 1 && !(kMode == kOneShot && a.skip_end) && !exchange(a, kPhaseDone, gen, kSiteEnd, &abort_smem)) return;
  if (threadIdx.x == 0) a.flags[a.rank]->counter[blockIdx.x] = gen;
}

}  // namespace comm
}  // namespace ixk

// ------------------------------------------------------------------ communicator (host)

struct ixk_comm {
  int rank = 0, world = 1, device = -1;
  size_t data_bytes = 0;
  unsigned char* base = nullptr;                       // this rank's allocation: header + data
  unsigned char* peer[IXK_COMM_MAX_RANKS] = {};        // every rank's allocation as mapped here (peer[rank] == base)
  bool ipc_opened[IXK_COMM_MAX_RANKS] = {};
  bool connected = false;
  long long wait_limit = ixk::comm::kDefaultWaitCycles;
  int force_algo = 0;                                   // 0 = by size, 1 = one-shot, 2 = two-shot
  bool alternating = false;                             // the caller never reuses a contribution range in consecutive calls
};

namespace ixk {
namespace comm {
namespace {

size_t elem_size(int dtype) { return dtype == IXK_F32 ? 4 : 2; }

int grid_for(size_t vecs) {
  const size_t per_cta = static_cast<size_t>(kThreads) * 2;
  size_t g = (vecs + per_cta - 1) / per_cta;
  if (g < 1) g = 1;
  if (g > static_cast<size_t>(kMaxBlocks)) g = kMaxBlocks;
  return static_cast<int>(g);
}

template <typename T, int kMode>
void launch_world(const Args& a, int grid, cudaStream_t stream) {
  if (kMode == kAllGather) {  // no arithmetic: one instantiation serves every world size
    all_reduce_kernel<T, 0, kMode><<<grid, kThreads, 0, stream>>>(a);
    return;
  }
  switch (a.world) {
    case 2: all_reduce_kernel<T, 2, kMode><<<grid, kThreads, 0, stream>>>(a); break;
    case 4: all_reduce_kernel<T, 4, kMode><<<grid, kThreads, 0, stream>>>(a); break;
    case 8: all_reduce_kernel<T, 8, kMode><<<grid, kThreads, 0, stream>>>(a); break;
    default: all_reduce_kernel<T, 0, kMode><<<grid, kThreads, 0, stream>>>(a); break;
  }
}

template <int kMode>
void launch_dtype(int dtype, const Args& a, int grid, cudaStream_t stream) {
  if (kMode == kAllGather) {  // bytes are bytes
    launch_world<float, kMode>(a, grid, stream);
    return;
  }
  if (dtype == IXK_BF16) launch_world<__nv_bfloat16, kMode>(a, grid, stream);
  else if (dtype == IXK_F16) launch_world<__half, kMode>(a, grid, stream);
  else launch_world<float, kMode>(a, grid, stream);
}

int run(ixk_comm* c, int dtype, int kind, size_t in_offset, const void* x, const void* bias, long long cols, void* out,
        size_t count, cudaStream_t stream) {
  if (c == nullptr) return fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  if (dtype != IXK_BF16 && dtype != IXK_F16 && dtype != IXK_F32)
    return fail(IXK_UNIMPLEMENTED, "all-reduce: BF16, F16 and F32 only");
  if (kind < IXK_REDUCE_SUM || kind > IXK_REDUCE_MAX) return fail(IXK_INVALID_ARGUMENT, "unknown reduction kind");
  if (count == 0) return IXK_OK;
  if (out == nullptr) return fail(IXK_INVALID_ARGUMENT, "out is NULL");
  if (!c->connected) return fail(IXK_INVALID_ARGUMENT, "the communicator has not been connected to its peers");
  const size_t bytes = count * elem_size(dtype);
  if (in_offset % 16 != 0 || in_offset > c->data_bytes || bytes > c->data_bytes - in_offset)
    return fail(IXK_INVALID_ARGUMENT, "the contribution [in_offset, in_offset + bytes) must lie inside the "
                                      "communicator's buffer and start on a 16-byte boundary");
  if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(bias) & 15u) != 0)
    return fail(IXK_INVALID_ARGUMENT, "out, x and bias must be 16-byte aligned");
  if (bias != nullptr && (cols <= 0 || cols % (16 / static_cast<long long>(elem_size(dtype))) != 0 ||
                          count % static_cast<size_t>(cols) != 0))
    return fail(IXK_INVALID_ARGUMENT, "bias needs cols to be a multiple of one 16-byte vector and to divide count");
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  if (dev.device != c->device) return fail(IXK_INVALID_ARGUMENT, "the communicator belongs to another device");

  unsigned char* data = c->base + kHeaderBytes;
  unsigned char* o = static_cast<unsigned char*>(out);
  const bool out_in_comm = o >= data && o + bytes <= data + c->data_bytes;
  unsigned char* in_here = data + in_offset;
  const bool in_place = o == in_here;
  if (!in_place && o < in_here + bytes && in_here < o + bytes)
    return fail(IXK_INVALID_ARGUMENT, "out overlaps the contribution without being the same range");
  if (in_place && x != nullptr)
    return fail(IXK_INVALID_ARGUMENT, "the fused residual form cannot write over the contribution (peers still read it)");
  // Two-shot needs the output at the same offset in every rank's buffer (peers write into it) and
  // pays off once the message is bandwidth-bound.  In place it is the only safe scheme: a rank
  // then overwrites only the slice that it alone reads, whereas a one-shot rank would overwrite
  // a contribution that its peers may still be reading.
  bool two_shot = c->world > 1 && x == nullptr && (in_place || (out_in_comm && bytes >= (static_cast<size_t>(1) << 20)));
  if (c->force_algo == 1 && !in_place) two_shot = false;
  if (c->force_algo == 2) {
    if (!out_in_comm || x != nullptr)
      return fail(IXK_INVALID_ARGUMENT, "two-shot all-reduce needs `out` inside the communicator's buffer and no epilogue");
    two_shot = c->world > 1;
  }
  Args a{};
  for (int r = 0; r < c->world; ++r) {
    a.flags[r] = reinterpret_cast<Flags*>(c->peer[r]);
    a.in[r] = c->peer[r] + kHeaderBytes + in_offset;
    a.out[r] = two_shot ? c->peer[r] + kHeaderBytes + (o - data) : nullptr;
  }
  if (!two_shot) a.out[0] = out;
  a.x = x;
  a.bias = bias;
  a.cols = cols;
  a.count = count;
  a.rank = c->rank;
  a.world = c->world;
  a.kind = kind;
  a.skip_end = (c->alternating && !two_shot) ? 1 : 0;
  a.wait_limit = c->wait_limit;
  a.status_word = dev.status_word;
  const size_t vecs = bytes / 16;
  const int grid = grid_for(two_shot ? vecs / c->world : vecs);
  if (two_shot) launch_dtype<kTwoShotMode>(dtype, a, grid, stream);
  else launch_dtype<kOneShot>(dtype, a, grid, stream);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

// The two halves of the two-shot all-reduce as calls of their own.  `count` = elements per rank, a
// whole number of 16-byte vectors.
int run_half(ixk_comm* c, int dtype, int kind, bool gather, size_t comm_offset, void* local, size_t count,
             cudaStream_t stream) {
  if (c == nullptr) return fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  if (dtype != IXK_BF16 && dtype != IXK_F16 && dtype != IXK_F32)
    return fail(IXK_UNIMPLEMENTED, "reduce-scatter / all-gather: BF16, F16 and F32 only");
  if (!gather && (kind < IXK_REDUCE_SUM || kind > IXK_REDUCE_MAX)) return fail(IXK_INVALID_ARGUMENT, "unknown reduction kind");
  if (count == 0) return IXK_OK;
  if (local == nullptr) return fail(IXK_INVALID_ARGUMENT, "the local buffer is NULL");
  if (!c->connected) return fail(IXK_INVALID_ARGUMENT, "the communicator has not been connected to its peers");
  const size_t piece = count * elem_size(dtype);
  if (piece % 16 != 0) return fail(IXK_UNIMPLEMENTED, "the per-rank piece must be a whole number of 16-byte vectors");
  const size_t total = piece * static_cast<size_t>(c->world);
  if (comm_offset % 16 != 0 || comm_offset > c->data_bytes || total > c->data_bytes - comm_offset)
    return fail(IXK_INVALID_ARGUMENT, "[offset, offset + world * piece) must lie inside the communicator's buffer, 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(local) & 15u) != 0) return fail(IXK_INVALID_ARGUMENT, "the local buffer must be 16-byte aligned");
  unsigned char* data = c->base + kHeaderBytes;
  unsigned char* l = static_cast<unsigned char*>(local);
  if (l < data + comm_offset + total && data + comm_offset < l + piece)
    return fail(IXK_INVALID_ARGUMENT, "the local buffer overlaps the exchanged range");
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  if (dev.device != c->device) return fail(IXK_INVALID_ARGUMENT, "the communicator belongs to another device");
  Args a{};
  for (int r = 0; r < c->world; ++r) {
    a.flags[r] = reinterpret_cast<Flags*>(c->peer[r]);
    a.in[r] = gather ? nullptr : c->peer[r] + kHeaderBytes + comm_offset;
    a.out[r] = gather ? c->peer[r] + kHeaderBytes + comm_offset : nullptr;
  }
  if (gather) a.in[0] = local; else a.out[0] = local;
  a.count = gather ? piece / 4 : count;   // the gather kernel is instantiated for 4-byte words whatever the type
  a.rank = c->rank;
  a.world = c->world;
  a.kind = kind;
  a.wait_limit = c->wait_limit;
  a.status_word = dev.status_word;
  const int grid = grid_for(piece / 16);
  if (gather) launch_dtype<kAllGather>(dtype, a, grid, stream);
  else launch_dtype<kReduceScatter>(dtype, a, grid, stream);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

// Second half of a projection whose output was scattered (gemm::Problem::scatter_*): slot s of
// this rank's `world` slots holds rank s's partial sums of the rows this rank owns.  The two-shot
// kernel does the rest: its "contributions" are the local slots (addressed so that the kernel's
// slice index lands inside them), its outputs every rank's result buffer.
int run_scattered(ixk_comm* c, int dtype, size_t slots_offset, const void* x, const void* bias, size_t out_offset,
                  long long rows, long long cols, cudaStream_t stream) {
  if (c == nullptr) return fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  if (dtype != IXK_BF16 && dtype != IXK_F16) return fail(IXK_UNIMPLEMENTED, "scattered all-reduce: BF16 and F16 only");
  if (rows < 0 || cols < 0) return fail(IXK_INVALID_ARGUMENT, "negative size");
  if (rows == 0 || cols == 0) return IXK_OK;
  if (!c->connected) return fail(IXK_INVALID_ARGUMENT, "the communicator has not been connected to its peers");
  if (rows % c->world != 0 || cols % 8 != 0)
    return fail(IXK_UNIMPLEMENTED, "rows must divide among the ranks and cols be a multiple of 8");
  const size_t bytes = static_cast<size_t>(rows) * cols * 2;
  const size_t slot_bytes = bytes / c->world;
  auto inside = [&](size_t off) { return off % 16 == 0 && off <= c->data_bytes && bytes <= c->data_bytes - off; };
  if (!inside(slots_offset) || !inside(out_offset))
    return fail(IXK_INVALID_ARGUMENT, "slots and result must lie inside the communicator's buffer, 16-byte aligned");
  if (slots_offset < out_offset + bytes && out_offset < slots_offset + bytes)
    return fail(IXK_INVALID_ARGUMENT, "the result overlaps the slots");
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(bias) & 15u) != 0)
    return fail(IXK_INVALID_ARGUMENT, "x and bias must be 16-byte aligned");
  if (bias != nullptr && x == nullptr) return fail(IXK_INVALID_ARGUMENT, "bias comes with the residual x only");
  DeviceInfo dev;
  int rc = get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  if (dev.device != c->device) return fail(IXK_INVALID_ARGUMENT, "the communicator belongs to another device");
  Args a{};
  const uintptr_t slots = reinterpret_cast<uintptr_t>(c->base + kHeaderBytes + slots_offset);
  for (int r = 0; r < c->world; ++r) {
    a.flags[r] = reinterpret_cast<Flags*>(c->peer[r]);
    // the kernel reads in[s] + (this rank's slice begin + i): make that slot s, element i
    a.in[r] = reinterpret_cast<const void*>(slots + static_cast<uintptr_t>(r) * slot_bytes -
                                            static_cast<uintptr_t>(c->rank) * slot_bytes);
    a.out[r] = c->peer[r] + kHeaderBytes + out_offset;
  }
  a.x = x;
  a.bias = bias;
  a.cols = cols;
  a.count = static_cast<size_t>(rows) * cols;
  a.rank = c->rank;
  a.world = c->world;
  a.kind = IXK_REDUCE_SUM;
  a.wait_limit = c->wait_limit;
  a.status_word = dev.status_word;
  const int grid = grid_for(slot_bytes / 16);
  launch_dtype<kTwoShotMode>(dtype, a, grid, stream);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

}  // namespace

int scatter_targets(ixk_comm* c, size_t slots_offset, long long rows, size_t row_bytes, void** dest, int* world) {
  if (c == nullptr) return fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  if (!c->connected) return fail(IXK_INVALID_ARGUMENT, "the communicator has not been connected to its peers");
  if (rows <= 0 || rows % c->world != 0) return fail(IXK_UNIMPLEMENTED, "the rows must divide among the ranks");
  const size_t slot_bytes = static_cast<size_t>(rows / c->world) * row_bytes;
  const size_t total = slot_bytes * c->world;
  if (slots_offset % 16 != 0 || slot_bytes % 16 != 0 || slots_offset > c->data_bytes || total > c->data_bytes - slots_offset)
    return fail(IXK_INVALID_ARGUMENT, "the slots must lie inside the communicator's buffer, 16-byte aligned");
  int device = -1;
  IXK_CUDA_OK(cudaGetDevice(&device));
  if (device != c->device) return fail(IXK_INVALID_ARGUMENT, "the communicator belongs to another device");
  for (int o = 0; o < c->world; ++o)
    dest[o] = c->peer[o] + kHeaderBytes + slots_offset + static_cast<size_t>(c->rank) * slot_bytes;
  *world = c->world;
  return IXK_OK;
}

}  // namespace comm
}  // namespace ixk

extern "C" {

int ixk_all_reduce_scattered(ixk_comm* c, int dtype, size_t slots_offset, const void* x, const void* bias,
                             size_t out_offset, int64_t rows, int64_t cols, void* cuda_stream) {
  IXK_API_RANGE("ixk_all_reduce_scattered");
  ixk::clear_error();
  return ixk::comm::run_scattered(c, dtype, slots_offset, x, bias, out_offset, rows, cols, static_cast<cudaStream_t>(cuda_stream));
}

int ixk_reduce_scatter(ixk_comm* c, int dtype, int kind, size_t in_offset, void* out, size_t count_per_rank, void* cuda_stream) {
  IXK_API_RANGE("ixk_reduce_scatter");
  ixk::clear_error();
  return ixk::comm::run_half(c, dtype, kind, false, in_offset, out, count_per_rank, static_cast<cudaStream_t>(cuda_stream));
}

int ixk_all_gather(ixk_comm* c, int dtype, const void* in, size_t out_offset, size_t count_per_rank, void* cuda_stream) {
  IXK_API_RANGE("ixk_all_gather");
  ixk::clear_error();
  return ixk::comm::run_half(c, dtype, IXK_REDUCE_SUM, true, out_offset, const_cast<void*>(in), count_per_rank,
                             static_cast<cudaStream_t>(cuda_stream));
}

int ixk_comm_create(int rank, int world, size_t buffer_bytes, ixk_comm** comm, void* handle_out) {
  IXK_API_RANGE("ixk_comm_create");
  ixk::clear_error();
  if (comm == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  *comm = nullptr;
  if (world < 1 || world > IXK_COMM_MAX_RANKS || rank < 0 || rank >= world)
    return ixk::fail(IXK_INVALID_ARGUMENT, "need 0 <= rank < world <= " + std::to_string(IXK_COMM_MAX_RANKS));
  if (buffer_bytes == 0 || buffer_bytes % 16 != 0)
    return ixk::fail(IXK_INVALID_ARGUMENT, "buffer_bytes must be a positive multiple of 16");
  ixk::DeviceInfo dev;
  int rc = ixk::get_device_info(&dev);
  if (rc != IXK_OK) return rc;
  ixk_comm* c = new ixk_comm();
  c->rank = rank;
  c->world = world;
  c->device = dev.device;
  c->data_bytes = buffer_bytes;
  if (const char* e = std::getenv("IXK_ALLREDUCE_ALGO")) c->force_algo = std::atoi(e);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, ixk::comm::kHeaderBytes + buffer_bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, ixk::comm::kHeaderBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && handle_out != nullptr) {
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == IXK_COMM_HANDLE_BYTES, "IPC handle size");
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) std::memcpy(handle_out, &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (p != nullptr) cudaFree(p);
    delete c;
    return ixk::fail(IXK_CUDA_ERROR, std::string("ixk_comm_create: ") + cudaGetErrorString(e));
  }
  c->base = static_cast<unsigned char*>(p);
  c->peer[rank] = c->base;
  c->connected = world == 1;
  *comm = c;
  return IXK_OK;
}

int ixk_comm_connect_ipc(ixk_comm* c, const void* handles) {
  IXK_API_RANGE("ixk_comm_connect_ipc");
  ixk::clear_error();
  if (c == nullptr || handles == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "comm or handles is NULL");
  if (c->connected) return ixk::fail(IXK_INVALID_ARGUMENT, "already connected");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const unsigned char*>(handles) + static_cast<size_t>(r) * IXK_COMM_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return ixk::fail(IXK_CUDA_ERROR, "cudaIpcOpenMemHandle(rank " + std::to_string(r) + "): " + cudaGetErrorString(e));
    }
    c->peer[r] = static_cast<unsigned char*>(p);
    c->ipc_opened[r] = true;
  }
  c->connected = true;
  return IXK_OK;
}

int ixk_comm_connect_pointers(ixk_comm* c, void* const* peer_bases) {
  IXK_API_RANGE("ixk_comm_connect_pointers");
  ixk::clear_error();
  if (c == nullptr || peer_bases == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "comm or peer_bases is NULL");
  if (c->connected) return ixk::fail(IXK_INVALID_ARGUMENT, "already connected");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (peer_bases[r] == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "peer_bases[" + std::to_string(r) + "] is NULL");
    c->peer[r] = static_cast<unsigned char*>(peer_bases[r]);
  }
  c->connected = true;
  return IXK_OK;
}

void* ixk_comm_base(ixk_comm* c) { return c == nullptr ? nullptr : c->base; }
void* ixk_comm_buffer(ixk_comm* c) { return c == nullptr ? nullptr : c->base + ixk::comm::kHeaderBytes; }
size_t ixk_comm_buffer_bytes(ixk_comm* c) { return c == nullptr ? 0 : c->data_bytes; }

int ixk_comm_set_wait_limit(ixk_comm* c, long long cycles) {
  ixk::clear_error();
  if (c == nullptr || cycles <= 0) return ixk::fail(IXK_INVALID_ARGUMENT, "comm is NULL or cycles <= 0");
  c->wait_limit = cycles;
  return IXK_OK;
}

int ixk_comm_set_alternating(ixk_comm* c, int on) {
  ixk::clear_error();
  if (c == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  c->alternating = on != 0;
  return IXK_OK;
}

int ixk_comm_destroy(ixk_comm* c) {
  IXK_API_RANGE("ixk_comm_destroy");
  ixk::clear_error();
  if (c == nullptr) return IXK_OK;
  cudaError_t first = cudaSuccess;
  for (int r = 0; r < c->world; ++r) {
    if (c->ipc_opened[r]) {
      cudaError_t e = cudaIpcCloseMemHandle(c->peer[r]);
      if (first == cudaSuccess) first = e;
    }
  }
  if (c->base != nullptr) {
    cudaError_t e = cudaFree(c->base);
    if (first == cudaSuccess) first = e;
  }
  delete c;
  if (first != cudaSuccess) {
    (void)cudaGetLastError();
    return ixk::fail(IXK_CUDA_ERROR, std::string("ixk_comm_destroy: ") + cudaGetErrorString(first));
  }
  return IXK_OK;
}

int ixk_all_reduce(ixk_comm* c, int dtype, int kind, size_t in_offset, void* out, size_t count, void* cuda_stream) {
  IXK_API_RANGE("ixk_all_reduce");
  ixk::clear_error();
  return ixk::comm::run(c, dtype, kind, in_offset, nullptr, nullptr, 0, out, count, static_cast<cudaStream_t>(cuda_stream));
}

int ixk_all_reduce_residual(ixk_comm* c, int dtype, size_t in_offset, const void* x, const void* bias, void* out,
                            int64_t rows, int64_t cols, void* cuda_stream) {
  IXK_API_RANGE("ixk_all_reduce_residual");
  ixk::clear_error();
  if (x == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "x is NULL");
  if (rows < 0 || cols < 0) return ixk::fail(IXK_INVALID_ARGUMENT, "negative size");
  return ixk::comm::run(c, dtype, IXK_REDUCE_SUM, in_offset, x, bias, cols, out, static_cast<size_t>(rows) * cols,
                        static_cast<cudaStream_t>(cuda_stream));
}

// Slice of a `count`-element message that rank `rank` of `world` reduces and broadcasts in the
// two-shot scheme, in elements: whole 16-byte vectors split evenly, the last rank also takes the
// remainder (ccl_ops.cc:103-114).  Host arithmetic only.
int ixk_all_reduce_slice(int dtype, size_t count, int rank, int world, size_t* begin, size_t* end) {
  ixk::clear_error();
  if (begin == nullptr || end == nullptr || world < 1 || rank < 0 || rank >= world)
    return ixk::fail(IXK_INVALID_ARGUMENT, "bad rank / world or NULL result pointer");
  const size_t e = 16 / ixk::comm::elem_size(dtype);
  const size_t vecs = count / e;
  const size_t per = vecs / world;
  *begin = per * rank * e;
  *end = rank == world - 1 ? count : (per * (rank + 1)) * e;
  return IXK_OK;
}

}  // extern "C"
