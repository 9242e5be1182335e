// Attention backward for sm_100a: dQ, dK, dV from Q, K, V, O, dO and the forward's row statistic.
// Replaces fmha_backward_kernel_{bf16,fp16} (xla/service/gpu/xetla/sdp/sdp_backward.h) and follows
// its three-kernel split (fmha_backward.h:854-918):
//   1. bwd_prepare_kernel : D = rowsum(dO * O), -lse * log2(e) in padded rows, zero the fp32 dQ
//                           accumulator                                   (fmha_backward.h:182-222)
//   2. fmha_bwd_kernel    : one CTA per (batch, head, block of 128 keys) loops over the blocks of
//                           128 queries that see those keys; dK and dV accumulate in tensor memory
//                           for the whole loop, dQ contributions are added to the fp32 accumulator
//                           by bulk reductions                             (fmha_backward.h:489-700)
//   3. bwd_convert_kernel : dQ = head_scale * accumulator, rounded once    (fmha_backward.h:836-850)
//
// The main kernel works on TRANSPOSED score tiles, keys along the 128 TMEM lanes and queries along
// the columns, so that P^T and dS^T are produced in the orientation the dV and dK products want:
//   S^T  = K   . Q^T      (SS, both K-major)                 -> TMEM, fp32
//   dP^T = V   . dO^T     (SS, both K-major)                 -> TMEM, fp32
//   P^T  = exp2(S^T * scale*log2e + bias*log2e - lse*log2e)  -> TMEM, 16-bit, over S^T
//   dS^T = P^T * (dP^T - D)                                  -> shared memory, 16-bit, swizzled
//   dV  += P^T  . dO      (TS: A from TMEM, B = dO with the head dim contiguous)
//   dK  += dS^T . Q       (SS: A K-major, B = Q with the head dim contiguous)
//   dQ^T = K^T  . dS^T    (SS: A = the K tile read with the head dim as M, B = dS^T read with the
//                          queries as N) -> TMEM with the head dim along the lanes
// Tensor memory (512 columns) at head size 128: S^T/P^T 128, dP^T 128 (reused for dQ^T once dS^T
// is out), dV 128, dK 128.  Shared memory (224 KB at head size 128): K, V, two Q tiles, one dO
// tile, dS^T, four 8 KB staging pieces for dQ.
// Warps 0-7 compute P^T and dS^T (one key row per thread, each warpgroup half of the step's
// queries); warps 8-11 drain dQ^T into registers, transpose it through the staging pieces and hand
// each piece (16 query rows, contiguous in the accumulator) to a bulk reduction; warp 12 loads K,
// V, Q and the row statistics, warp 14 the dO tiles; warp 13 issues the MMAs with all lanes and an
// elected lane per instruction, in the order dV(i), S^T(i+1), dQ^T(i), dK(i), dP^T(i+1), so that
// the next scores are ready when the compute warps finish dS^T and dQ^T leaves the columns it
// shares with dP^T while dK runs.  CTAs of one (batch, head) are neighbours in launch order: its
// Q, dO and accumulator slice stay in L2.  Every wait is bounded.
// Tried and dropped: two CTAs of a cluster on neighbouring key blocks that exchange halves of their
// dQ^T partials through distributed shared memory before one bulk reduction each (half the L2
// traffic).  Correct, but 1.13 ms against 0.85 ms: 64 remote 4-byte stores per thread took 2500
// cycles per step, the local add 1070 and the 32 KB reduction still 2370.
// What bounds it: the additions to the dQ accumulator.  Each step adds 64 KB; the memory system
// sustained about 3 TB/s of fp32 reductions over the whole GPU whether they were issued as bulk
// reductions, as per-lane vector reductions or as warp-coalesced scalar ones, which is about
// 3600 cycles per step against 2560 cycles of MMA work.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <type_traits>

#include "fmha_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace fmha {

namespace {

constexpr int kBlk = 128;                       // keys per CTA = queries per step = TMEM lanes
constexpr int kChunkElems = 64;                 // 16-bit elements per 128-byte swizzle row
constexpr int kChunkBytes = kBlk * 128;         // one 128-row x 128-byte box
constexpr int kBwdThreads = 512;                // warp 15 only takes part in the register re-partitioning
constexpr int kComputeThreads = 256;            // two warpgroups, each takes half of a step's query columns
constexpr int kReduceWarp = 8;                  // first warp of the dQ warpgroup
constexpr int kBwdProducerWarp = 12;
constexpr int kBwdMmaWarp = 13;
constexpr int kStages = 2;                      // Q tiles in flight
constexpr int kDoWarp = 14;                     // loads the dO tiles
// per-thread register budgets after re-partitioning: 384 x 152 + 128 x 56 = 65536
constexpr int kWorkRegs = 152;
constexpr int kCtrlRegs = 56;
constexpr float kLog2e = 1.4426950408889634f;

// wait sites reported in the device status word
constexpr int kSiteBwdKv = 0x41, kSiteBwdQdoFull = 0x42, kSiteBwdQdoEmpty = 0x43, kSiteBwdS = 0x44,
              kSiteBwdP = 0x45, kSiteBwdDqFull = 0x46, kSiteBwdDqFree = 0x47, kSiteBwdFinal = 0x48,
              kSiteBwdAlign = 0x49, kSiteBwdDp = 0x4a, kSiteBwdDs = 0x4b;

template <int kHeadDim>
struct BwdCfg {
  static_assert(kHeadDim == 64 || kHeadDim == 128, "head size bucket");
  static constexpr int kChunks = kHeadDim / kChunkElems;
  static constexpr int kTileBytes = kChunks * kChunkBytes;          // a 128-row Q, dO, K or V tile
  static constexpr int kDsBytes = 2 * kChunkBytes;                  // dS^T: 128 keys x 128 queries, 16-bit
  static constexpr int kRowBytes = kBlk * 4;                        // 128 fp32 row values
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTileBytes;
  static constexpr int kOffQ = 2 * kTileBytes;                      // kStages Q tiles
  static constexpr int kOffDo = kOffQ + kStages * kTileBytes;       // one dO tile: it lives from dP^T to the next dV
  static constexpr int kOffDs = kOffDo + kTileBytes;
  static constexpr int kPieceRows = 16;                              // query rows per bulk reduction of dQ
  static constexpr int kPieceBytes = kPieceRows * kHeadDim * 4;
  static constexpr int kPieceBufs = 64 / kPieceRows;                // staging buffers: 64 query rows in all
  static constexpr int kOffDqStage = kOffDs + kDsBytes;
  static constexpr int kOffRows = kOffDqStage + kPieceBufs * kPieceBytes;   // per stage: -lse*log2e row, D row
  static constexpr int kOffBars = kOffRows + kStages * 2 * kRowBytes;
  static constexpr int kSmemBytes = kOffBars + 256;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  // tensor memory columns
  static constexpr int kTmemS = 0;
  static constexpr int kTmemDP = 128;
  static constexpr int kTmemDV = 256;
  static constexpr int kTmemDK = 256 + kHeadDim;
  static constexpr int kTmemDQ = kHeadDim == 128 ? kTmemDP : 256 + 2 * kHeadDim;
};

struct BwdArgs {
  int B, N, H, F, T;
  int f_pad;                 // F rounded up to a multiple of 128: row pitch of the fp32 scratch arrays
  int num_kblocks, num_qblocks;
  int causal, is_bf16;
  float scale_log2, head_scale;
  const uint16_t* bias;
  int64_t bias_strides[3];
  const float* neg_lse2;     // [B*N, f_pad]  -lse * log2(e); -inf in the padding
  const float* delta;        // [B*N, f_pad]  rowsum(dO * O); 0 in the padding
  float* dq_acc;             // [B*N, f_pad, kHeadDim] fp32
  uint16_t* dk;
  uint16_t* dv;
  int64_t dk_strides[3], dv_strides[3];
  int* status_word;
};

struct PrepArgs {
  int B, N, H, F, f_pad, head_pad, is_bf16;
  const uint16_t* out;
  const uint16_t* grad_out;
  const float* lse;
  int64_t o_strides[3], do_strides[3];
  float* neg_lse2;
  float* delta;
  float* dq_acc;
};

__device__ __forceinline__ float to_f32(uint16_t h, int is_bf16) {
  return is_bf16 ? __uint_as_float(static_cast<uint32_t>(h) << 16) : __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack16(uint32_t w, int is_bf16) {
  if (is_bf16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// One warp per group of four consecutive padded query rows of one (batch, head) (the padded row
// count is a multiple of 128, so a group never straddles two heads): a lane takes 8 head elements
// (16 bytes) of O and dO and one float4 per 128 floats of each accumulator row.  The row -> (batch,
// head, query) arithmetic is done once per group: with one 64-bit division chain per ROW the
// kernel was bound by instruction issue (about 400 instructions per row) at 2.5 TB/s.
__global__ void bwd_prepare_kernel(const PrepArgs a) {
  constexpr int kRows = 4;
  const int lane = threadIdx.x & 31;
  const int64_t groups = static_cast<int64_t>(a.B) * a.N * (a.f_pad / kRows);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int groups_per_head = a.f_pad / kRows;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); g < groups; g += warps) {
    const int64_t bn = g / groups_per_head;
    const int f0 = static_cast<int>(g - bn * groups_per_head) * kRows;
    const int n = static_cast<int>(bn % a.N), b = static_cast<int>(bn / a.N);
    const int64_t row0 = bn * a.f_pad + f0;
    const uint16_t* o_base = a.out + b * a.o_strides[0] + n * a.o_strides[1] + lane * 8;
    const uint16_t* g_base = a.grad_out + b * a.do_strides[0] + n * a.do_strides[1] + lane * 8;
    uint4 ow[kRows], gw[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      ow[r] = gw[r] = make_uint4(0u, 0u, 0u, 0u);
      if (f0 + r < a.F && lane * 8 < a.H) {      // head sizes up to 256 fit one 16-byte load per lane
        ow[r] = *reinterpret_cast<const uint4*>(o_base + static_cast<int64_t>(f0 + r) * a.o_strides[2]);
        gw[r] = *reinterpret_cast<const uint4*>(g_base + static_cast<int64_t>(f0 + r) * a.do_strides[2]);
      }
    }
    // the group's accumulator rows are contiguous: kRows * head_pad floats
    float* acc = a.dq_acc + row0 * a.head_pad;
    for (int h = lane * 4; h < kRows * a.head_pad; h += 128) *reinterpret_cast<float4*>(acc + h) = make_float4(0.f, 0.f, 0.f, 0.f);
    float sums[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const uint32_t ov[4] = {ow[r].x, ow[r].y, ow[r].z, ow[r].w}, gv[4] = {gw[r].x, gw[r].y, gw[r].z, gw[r].w};
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = unpack16(ov[j], a.is_bf16), y = unpack16(gv[j], a.is_bf16);
        sum = fmaf(x.x, y.x, sum);
        sum = fmaf(x.y, y.y, sum);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      sums[r] = sum;
    }
    if (lane < kRows) {
      float mine = sums[0];
#pragma unroll
      for (int r = 1; r < kRows; ++r) mine = lane == r ? sums[r] : mine;
      const int f = f0 + lane;
      a.delta[row0 + lane] = mine;
      a.neg_lse2[row0 + lane] = f < a.F ? -a.lse[bn * a.F + f] * kLog2e : -INFINITY;
    }
  }
}

struct ConvertArgs {
  int B, N, H, F, f_pad, head_pad, is_bf16;
  float head_scale;
  const float* dq_acc;
  uint16_t* dq;
  int64_t dq_strides[3];
};

// One thread per 8 head elements: two float4 in, 16 bytes out.
__global__ void bwd_convert_kernel(const ConvertArgs a) {
  const int groups = a.H / 8;
  const int64_t total = static_cast<int64_t>(a.B) * a.N * a.F * groups;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int hg = static_cast<int>(i % groups);
    const int64_t r = i / groups;
    const int f = static_cast<int>(r % a.F);
    const int64_t bn = r / a.F;
    const int n = static_cast<int>(bn % a.N), b = static_cast<int>(bn / a.N);
    const float4* src = reinterpret_cast<const float4*>(a.dq_acc + (bn * a.f_pad + f) * a.head_pad + 8 * hg);
    const float4 lo = src[0], hi = src[1];
    uint4 w;
    w.x = pack16(lo.x * a.head_scale, lo.y * a.head_scale, a.is_bf16);
    w.y = pack16(lo.z * a.head_scale, lo.w * a.head_scale, a.is_bf16);
    w.z = pack16(hi.x * a.head_scale, hi.y * a.head_scale, a.is_bf16);
    w.w = pack16(hi.z * a.head_scale, hi.w * a.head_scale, a.is_bf16);
    *reinterpret_cast<uint4*>(a.dq + b * a.dq_strides[0] + n * a.dq_strides[1] + f * a.dq_strides[2] + 8 * hg) = w;
  }
}

__device__ __forceinline__ void bwd_mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      ".reg .b64 da, db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      ".reg .b64 db;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int kHeadDim, bool kBias, bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1)
fmha_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const BwdArgs args) {
  using C = BwdCfg<kHeadDim>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = ptx::smem_u32(smem_raw);
  if ((smem_base & 1023u) != 0) {   // the swizzled tiles need 1024-byte alignment; never seen, but checked
    if (threadIdx.x == 0) atomicCAS(args.status_word, 0, kSiteBwdAlign);
    return;
  }
  const uint32_t k_smem = smem_base + C::kOffK;
  const uint32_t v_smem = smem_base + C::kOffV;
  const uint32_t ds_smem = smem_base + C::kOffDs;
  auto stage_q = [&](uint32_t st) { return smem_base + C::kOffQ + st * C::kTileBytes; };
  const uint32_t do_smem = smem_base + C::kOffDo;
  const uint32_t dq_stage = smem_base + C::kOffDqStage;
  auto rows_off = [&](uint32_t st) { return static_cast<uint32_t>(C::kOffRows) + st * 2 * C::kRowBytes; };
  const uint32_t bar_base = smem_base + C::kOffBars;
  const uint32_t kv_full = bar_base;
  auto q_full = [&](uint32_t st) { return bar_base + 8u * (1 + st); };
  auto q_empty = [&](uint32_t st) { return bar_base + 8u * (3 + st); };
  const uint32_t s_full = bar_base + 8u * 5, p_ready = bar_base + 8u * 6, dq_full = bar_base + 8u * 7,
                 dq_free = bar_base + 8u * 8, final_bar = bar_base + 8u * 9, dp_full = bar_base + 8u * 10,
                 ds_ready = bar_base + 8u * 11, do_full = bar_base + 8u * 12, do_empty = bar_base + 8u * 13;
  uint8_t* tail = smem_raw + C::kOffBars + 8 * 14;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ptx::AbortCtl ctl{abort_flag, args.status_word};

  // work item: the key blocks of one (batch, head) are neighbours in launch order, so that its Q, dO
  // and slice of the dQ accumulator (1 MB at 2048 queries) stay in L2 while they are shared;
  // within a head the heaviest key block comes first (under the causal mask block 0 is seen by
  // every query block).  A causal launch runs in two passes over the heads, the heavy half of the
  // key blocks first and the light half after it, so that the last CTAs to start are short ones.
  int kb, bn;
  {
    const int heads = args.B * args.N;
    const int first = args.causal ? (args.num_kblocks + 1) / 2 : args.num_kblocks;   // key blocks in pass 0
    const int pass0 = heads * first;
    if (static_cast<int>(blockIdx.x) < pass0) {
      kb = blockIdx.x % first;
      bn = blockIdx.x / first;
    } else {
      const int rest = args.num_kblocks - first;
      const int idx = blockIdx.x - pass0;
      kb = first + idx % rest;
      bn = idx / rest;
    }
  }
  const int n = bn % args.N, b = bn / args.N;
  const int i0 = args.causal ? kb : 0;
  const int n_steps = args.num_qblocks > i0 ? args.num_qblocks - i0 : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(kv_full, 1);
    for (uint32_t st = 0; st < kStages; ++st) {
      ptx::mbar_init(q_full(st), 1);
      ptx::mbar_init(q_empty(st), 1);
    }
    ptx::mbar_init(do_full, 1);
    ptx::mbar_init(do_empty, 1);
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(dp_full, 1);
    ptx::mbar_init(p_ready, kComputeThreads);
    ptx::mbar_init(ds_ready, kComputeThreads);
    ptx::mbar_init(dq_full, 1);
    ptx::mbar_init(dq_free, 128);
    ptx::mbar_init(final_bar, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
    ptx::prefetch_tmap(&tmap_do);
  }
  if (warp == kBwdMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kBwdProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    ptx::setmaxnreg_dec<kCtrlRegs>();
    if (lane == 0 && n_steps > 0) {
      ptx::mbar_expect_tx(kv_full, 2 * C::kTileBytes);
      for (int c = 0; c < C::kChunks; ++c) {
        ptx::tma_load_4d(k_smem + c * kChunkBytes, &tmap_k, kv_full, c * kChunkElems, kb * kBlk, n, b);
        ptx::tma_load_4d(v_smem + c * kChunkBytes, &tmap_v, kv_full, c * kChunkElems, kb * kBlk, n, b);
      }
      for (int it = 0; it < n_steps; ++it) {
        const uint32_t st = it & 1;
        if (it >= kStages && !ptx::mbar_wait(q_empty(st), ((it >> 1) - 1) & 1, ctl, kSiteBwdQdoEmpty)) break;
        const int q0 = (i0 + it) * kBlk;
        ptx::mbar_expect_tx(q_full(st), C::kTileBytes + 2 * C::kRowBytes);
        for (int c = 0; c < C::kChunks; ++c)
          ptx::tma_load_4d(stage_q(st) + c * kChunkBytes, &tmap_q, q_full(st), c * kChunkElems, q0, n, b);
        const int64_t row0 = static_cast<int64_t>(bn) * args.f_pad + q0;
        ptx::bulk_load_1d(smem_base + rows_off(st), args.neg_lse2 + row0, C::kRowBytes, q_full(st));
        ptx::bulk_load_1d(smem_base + rows_off(st) + C::kRowBytes, args.delta + row0, C::kRowBytes, q_full(st));
      }
    }
  } else if (warp == kDoWarp) {
    // ------------------------------------------------------------------ dO loads (one buffer)
    ptx::setmaxnreg_dec<kCtrlRegs>();
    if (lane == 0) {
      for (int it = 0; it < n_steps; ++it) {
        if (it >= 1 && !ptx::mbar_wait(do_empty, (it - 1) & 1, ctl, kSiteBwdQdoEmpty)) break;
        ptx::mbar_expect_tx(do_full, C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c)
          ptx::tma_load_4d(do_smem + c * kChunkBytes, &tmap_do, do_full, c * kChunkElems, (i0 + it) * kBlk, n, b);
      }
    }
  } else if (warp == kBwdMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (all 32 lanes)
    ptx::setmaxnreg_dec<kCtrlRegs>();
    if (n_steps > 0) {
      const uint32_t fmt = kBf16 ? 1u : 0u;
      const uint32_t idesc_t = ptx::umma_idesc(fmt, fmt, 0, 0, kBlk, kBlk);         // S^T, dP^T
      const uint32_t idesc_kv = ptx::umma_idesc(fmt, fmt, 0, 1, kBlk, kHeadDim);    // dV (A in TMEM), dK
      // dQ^T = K^T.dS^T: head dim along the lanes (M = 128; at head size 64 the upper 64 lanes
      // multiply whatever follows the K tile in shared memory and are never read), queries along
      // the columns, both operands read with their M / N dimension contiguous
      const uint32_t idesc_dq = ptx::umma_idesc(fmt, fmt, 1, 1, kBlk, kBlk);
      // descriptor address field: 16-byte units of the offset inside this CTA's window (were the
      // kernel launched in a cluster, the shared addresses of every CTA but the first would carry
      // the rank in their upper bits: measured 0x01000400 for the second CTA of a pair)
      auto da = [](uint32_t addr) { return (addr & 0x3ffffu) >> 4; };
      const uint64_t kmajor = ptx::umma_smem_desc(0, 16, 1024);
      const uint64_t mnmajor = ptx::umma_smem_desc(0, kChunkBytes, 1024);
      const uint32_t k_lo = static_cast<uint32_t>(kmajor), k_hi = static_cast<uint32_t>(kmajor >> 32);
      const uint32_t m_lo = static_cast<uint32_t>(mnmajor), m_hi = static_cast<uint32_t>(mnmajor >> 32);
      auto issue_s = [&](uint32_t q_addr) {        // S^T = K.Q^T
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
          bwd_mma_ss(tmem_base + C::kTmemS, k_lo + da(k_smem) + off, k_hi, k_lo + da(q_addr) + off, k_hi,
                     idesc_t, ks != 0 ? 1u : 0u);
        }
        ptx::umma_commit_elect(s_full);
      };
      auto issue_dp = [&](uint32_t do_addr) {      // dP^T = V.dO^T
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
          bwd_mma_ss(tmem_base + C::kTmemDP, k_lo + da(v_smem) + off, k_hi, k_lo + da(do_addr) + off, k_hi,
                     idesc_t, ks != 0 ? 1u : 0u);
        }
        ptx::umma_commit_elect(dp_full);
      };
      // Order per step: dV(i), S^T(i+1), dQ^T(i), dK(i), dP^T(i+1).  S^T of the next step runs
      // while the compute warps still turn dP^T into dS^T; dQ^T comes before dK so that it is
      // drained from the columns it shares with dP^T while dK runs.
      bool alive = ptx::mbar_wait(kv_full, 0, ctl, kSiteBwdKv) && ptx::mbar_wait(q_full(0), 0, ctl, kSiteBwdQdoFull) &&
                   ptx::mbar_wait(do_full, 0, ctl, kSiteBwdQdoFull);
      if (alive) {
        ptx::tc_fence_after_sync();
        issue_s(stage_q(0));
        issue_dp(do_smem);
      }
      for (int it = 0; it < n_steps && alive; ++it) {
        const uint32_t st = it & 1;
        const uint32_t q_addr = stage_q(st), do_addr = do_smem;
        const bool more = it + 1 < n_steps;
        if (!ptx::mbar_wait(p_ready, it & 1, ctl, kSiteBwdP)) break;
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kBlk / 16; ++ks)     // dV += P^T.dO over 16 queries at a time
          bwd_mma_ts(tmem_base + C::kTmemDV, tmem_base + C::kTmemS + (ks >> 2) * 64 + (ks & 3) * 8,
                     m_lo + da(do_addr) + ((ks * 2048) >> 4), m_hi, idesc_kv, (it > 0 || ks > 0) ? 1u : 0u);
        ptx::umma_commit_elect(do_empty);          // dO(i) has no reader after dV(i)
        if (more) {
          if (!ptx::mbar_wait(q_full(st ^ 1), ((it + 1) >> 1) & 1, ctl, kSiteBwdQdoFull)) break;
          ptx::tc_fence_after_sync();
          issue_s(stage_q(st ^ 1));
        }
        if (!ptx::mbar_wait(ds_ready, it & 1, ctl, kSiteBwdDs)) break;
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kBlk / 16; ++ks)     // dQ^T = K^T.dS^T over 16 keys at a time
          bwd_mma_ss(tmem_base + C::kTmemDQ, m_lo + da(k_smem) + ((ks * 2048) >> 4), m_hi,
                     m_lo + da(ds_smem) + ((ks * 2048) >> 4), m_hi, idesc_dq, ks != 0 ? 1u : 0u);
        ptx::umma_commit_elect(dq_full);
#pragma unroll
        for (int ks = 0; ks < kBlk / 16; ++ks) {   // dK += dS^T.Q
          const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
          bwd_mma_ss(tmem_base + C::kTmemDK, k_lo + da(ds_smem) + off, k_hi, m_lo + da(q_addr) + ((ks * 2048) >> 4),
                     m_hi, idesc_kv, (it > 0 || ks > 0) ? 1u : 0u);
        }
        ptx::umma_commit_elect(q_empty(st));
        if (more) {
          // dP^T shares its columns with dQ^T at head size 128
          if (!ptx::mbar_wait(dq_free, it & 1, ctl, kSiteBwdDqFree)) break;
          if (!ptx::mbar_wait(do_full, (it + 1) & 1, ctl, kSiteBwdQdoFull)) break;
          ptx::tc_fence_after_sync();
          issue_dp(do_smem);
        }
      }
      ptx::umma_commit_elect(final_bar);
    }
  } else if (warp < kReduceWarp) {
    // ------------------------------------------------------------------ P^T and dS^T (one key row per thread,
    // warpgroup 0 on query columns 0-63 of the step, warpgroup 1 on 64-127)
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const int key = kb * kBlk + r;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool key_ok = key < args.T;
    ptx::setmaxnreg_inc<kWorkRegs>();
    bool alive = true;
    for (int it = 0; it < n_steps && alive; ++it) {
      const uint32_t st = it & 1;
      if (!ptx::mbar_wait(q_full(st), (it >> 1) & 1, ctl, kSiteBwdQdoFull)) { alive = false; break; }
      if (!ptx::mbar_wait(s_full, it & 1, ctl, kSiteBwdS)) { alive = false; break; }
      ptx::tc_fence_after_sync();
      const int q0 = (i0 + it) * kBlk;
      const float* nl = reinterpret_cast<const float*>(smem_raw + rows_off(st)) + 64 * half;
      const float* dl = nl + kBlk;
      const bool diag = args.causal && (i0 + it) == kb;
      // bias column of this key (clamped to the last valid key: the mask zeroes what lies beyond)
      [[maybe_unused]] const uint16_t* bias_col = nullptr;
      if constexpr (kBias)
        bias_col = args.bias + b * args.bias_strides[0] + n * args.bias_strides[1] + (key_ok ? key : args.T - 1);
      // phase A: P^T = exp2(S^T * scale*log2e + bias*log2e - lse*log2e) for this warpgroup's 64 queries.
      // Only the diagonal block of a causal problem and a ragged last key block need the mask.
      // (with a bias, a ragged last query block takes the same path: it clamps the bias row index)
      const bool need_mask = diag || (kb + 1) * kBlk > args.T || (kBias && q0 + kBlk > args.F);
      const uint64_t scale2 = ptx::f32x2(args.scale_log2, args.scale_log2);
      uint64_t p2[32];     // P as fp32 pairs (queries 2j, 2j+1 of this warpgroup's half)
      auto phase_a = [&](auto masked) {
        constexpr bool kMasked = decltype(masked)::value;
        uint32_t s[2][32];
        ptx::tmem_ld_32x32(tmem_base + lane_addr + C::kTmemS + 64 * half, s[0]);
        ptx::tmem_ld_32x32(tmem_base + lane_addr + C::kTmemS + 64 * half + 32, s[1]);
        // bias values of this thread's key for 32 queries: no branch per element (row indices past
        // the last query are clamped; those columns come out as zero through -inf in the lse row)
        [[maybe_unused]] uint16_t bv[32];
        [[maybe_unused]] auto load_bias = [&](int c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            int q = q0 + 64 * half + 32 * c + j;
            if constexpr (kMasked) q = min(q, args.F - 1);
            bv[j] = bias_col[static_cast<int64_t>(q) * args.bias_strides[2]];
          }
        };
        if constexpr (kBias) load_bias(0);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pw[16];
          if constexpr (kBias) {
            if (c == 1) load_bias(1);
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 nl4 = *reinterpret_cast<const float4*>(nl + 32 * c + 4 * j4);
            uint64_t x[2] = {ptx::fma2(ptx::f32x2(__uint_as_float(s[c][4 * j4]), __uint_as_float(s[c][4 * j4 + 1])), scale2,
                                       ptx::f32x2(nl4.x, nl4.y)),
                             ptx::fma2(ptx::f32x2(__uint_as_float(s[c][4 * j4 + 2]), __uint_as_float(s[c][4 * j4 + 3])), scale2,
                                       ptx::f32x2(nl4.z, nl4.w))};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float x0, x1;
              ptx::f32x2_split(x[e], x0, x1);
              const int col = 32 * c + 4 * j4 + 2 * e;
              if constexpr (kBias) {
                x0 = fmaf(to_f32(bv[4 * j4 + 2 * e], kBf16), kLog2e, x0);
                x1 = fmaf(to_f32(bv[4 * j4 + 2 * e + 1], kBf16), kLog2e, x1);
              }
              float e0 = ptx::ex2_approx(x0), e1 = ptx::ex2_approx(x1);
              if constexpr (kMasked) {
                const int lim = diag ? key - (q0 + 64 * half + col) : 0;   // masked when key > query
                e0 = (!key_ok || lim > 0) ? 0.0f : e0;
                e1 = (!key_ok || lim > 1) ? 0.0f : e1;
              }
              p2[16 * c + 2 * j4 + e] = ptx::f32x2(e0, e1);
              pw[2 * j4 + e] = pack16(e0, e1, kBf16);
            }
          }
          // P^T goes over the S^T columns this warpgroup has already read: queries 0-63 at columns
          // 0-31, queries 64-127 at columns 64-95
          ptx::tmem_st_32x16(tmem_base + lane_addr + C::kTmemS + 64 * half + 16 * c, pw);
        }
      };
      if (need_mask) phase_a(std::true_type{}); else phase_a(std::false_type{});
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(p_ready);
      // phase B: dS^T = P^T * (dP^T - D)
      if (!ptx::mbar_wait(dp_full, it & 1, ctl, kSiteBwdDp)) { alive = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t dp[2][32];
      ptx::tmem_ld_32x32(tmem_base + lane_addr + C::kTmemDP + 64 * half, dp[0]);
      ptx::tmem_ld_32x32(tmem_base + lane_addr + C::kTmemDP + 64 * half + 32, dp[1]);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dw[16];
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          const float4 dl4 = *reinterpret_cast<const float4*>(dl + 32 * c + 4 * j4);
          const uint64_t d0 = ptx::mul2(p2[16 * c + 2 * j4],
                                        ptx::sub2(ptx::f32x2(__uint_as_float(dp[c][4 * j4]), __uint_as_float(dp[c][4 * j4 + 1])),
                                                  ptx::f32x2(dl4.x, dl4.y)));
          const uint64_t d1 = ptx::mul2(p2[16 * c + 2 * j4 + 1],
                                        ptx::sub2(ptx::f32x2(__uint_as_float(dp[c][4 * j4 + 2]), __uint_as_float(dp[c][4 * j4 + 3])),
                                                  ptx::f32x2(dl4.z, dl4.w)));
          float a0, a1, b0, b1;
          ptx::f32x2_split(d0, a0, a1);
          ptx::f32x2_split(d1, b0, b1);
          dw[2 * j4] = pack16(a0, a1, kBf16);
          dw[2 * j4 + 1] = pack16(b0, b1, kBf16);
        }
        const uint32_t row_addr = ds_smem + half * kChunkBytes + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t grp = static_cast<uint32_t>(c * 4 + g) ^ static_cast<uint32_t>(r & 7);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (grp << 4)), "r"(dw[4 * g]),
                       "r"(dw[4 * g + 1]), "r"(dw[4 * g + 2]), "r"(dw[4 * g + 3])
                       : "memory");
        }
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(ds_ready);
    }
    // epilogue: this thread's row of dV and dK
    const bool have = n_steps > 0 && alive && ptx::mbar_wait(final_bar, 0, ctl, kSiteBwdFinal);
    if (n_steps == 0 || have) {
      ptx::tc_fence_after_sync();
      uint16_t* dv_row = args.dv + b * args.dv_strides[0] + n * args.dv_strides[1] + static_cast<int64_t>(key) * args.dv_strides[2];
      uint16_t* dk_row = args.dk + b * args.dk_strides[0] + n * args.dk_strides[1] + static_cast<int64_t>(key) * args.dk_strides[2];
      {
        const int which = half;      // warpgroup 0 stores dV, warpgroup 1 dK
        uint16_t* dst = which == 0 ? dv_row : dk_row;
        const uint32_t col0 = which == 0 ? C::kTmemDV : C::kTmemDK;
        const float mul = which == 0 ? 1.0f : args.head_scale;
#pragma unroll 1
        for (int c = 0; c < kHeadDim / 32; ++c) {
          uint32_t acc[32];
          if (n_steps > 0) {
            ptx::tmem_ld_32x32(tmem_base + lane_addr + col0 + 32 * c, acc);
            ptx::tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0u;
          }
          if (key_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int h = 32 * c + 8 * g;
              if (h < args.H) {
                uint4 w;
                w.x = pack16(__uint_as_float(acc[8 * g]) * mul, __uint_as_float(acc[8 * g + 1]) * mul, kBf16);
                w.y = pack16(__uint_as_float(acc[8 * g + 2]) * mul, __uint_as_float(acc[8 * g + 3]) * mul, kBf16);
                w.z = pack16(__uint_as_float(acc[8 * g + 4]) * mul, __uint_as_float(acc[8 * g + 5]) * mul, kBf16);
                w.w = pack16(__uint_as_float(acc[8 * g + 6]) * mul, __uint_as_float(acc[8 * g + 7]) * mul, kBf16);
                *reinterpret_cast<uint4*>(dst + h) = w;
              }
            }
          }
        }
      }
    }
  } else if (warp < kBwdProducerWarp) {
    // ------------------------------------------------------------------ dQ^T: TMEM -> fp32 accumulator
    // One head-dim element per thread: the 32 lanes of a warp add to 32 consecutive floats of one
    // query row of the accumulator, a full 128-byte line per instruction.
    ptx::setmaxnreg_inc<kWorkRegs>();
    const int d = threadIdx.x - kReduceWarp * 32;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t piece = 0;      // running count of staged pieces: buffer = piece & 1
    for (int it = 0; it < n_steps; ++it) {
      if (!ptx::mbar_wait(dq_full, it & 1, ctl, kSiteBwdDqFull)) break;
      ptx::tc_fence_after_sync();
      const int q0 = (i0 + it) * kBlk;
      float* dst = args.dq_acc + (static_cast<int64_t>(bn) * args.f_pad + q0) * kHeadDim;
      uint32_t acc[4][32];
      if (d < kHeadDim) {
#pragma unroll
        for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(tmem_base + lane_addr + C::kTmemDQ + 32 * c, acc[c]);
        ptx::tmem_ld_wait();
      }
      // the columns are free once they sit in registers
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(dq_free);
      // Pieces of 16 query rows in four staging buffers: transpose through shared memory into the accumulator's
      // [query][head dim] order (conflict-free: a warp writes 32 consecutive floats of one row),
      // then one bulk reduction per piece adds the contiguous block to global memory.
#pragma unroll
      for (int c = 0; c < kBlk / C::kPieceRows; ++c, ++piece) {
        const uint32_t buf = dq_stage + (piece % C::kPieceBufs) * C::kPieceBytes;
        if (d < kHeadDim) {
#pragma unroll
          for (int j = 0; j < C::kPieceRows; ++j) {
            const int row = c * C::kPieceRows + j;
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(buf + (j * kHeadDim + d) * 4), "r"(acc[row >> 5][row & 31]) : "memory");
          }
        }
        ptx::fence_proxy_async_smem();
        // the reduction that last read the NEXT piece's buffer has finished before anyone passes
        // this barrier
        if (threadIdx.x == kReduceWarp * 32) ptx::bulk_wait_group_read<C::kPieceBufs - 2>();
        ptx::named_barrier_sync(1, 128);
        if (threadIdx.x == kReduceWarp * 32) {
          ptx::bulk_reduce_add_f32(dst + c * C::kPieceRows * kHeadDim, buf, C::kPieceBytes);
          ptx::bulk_commit_group();
        }
      }
    }
    if (threadIdx.x == kReduceWarp * 32) ptx::bulk_wait_group<0>();   // all additions performed before the CTA exits
  } else {
    ptx::setmaxnreg_dec<kCtrlRegs>();     // warp 15: nothing else to do
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == kBwdMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <int kHeadDim, bool kBias, bool kBf16>
int launch_bwd_cfg(const BwdProblem& bp, const DeviceInfo& dev, float* neg_lse2, float* delta, float* dq_acc,
                   int f_pad, cudaStream_t stream) {
  using C = BwdCfg<kHeadDim>;
  const Problem& p = bp.fwd;
  const CUtensorMapDataType dt = p.dtype == IXK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  auto make_map = [&](CUtensorMap* out, const void* base, const int64_t* strides, int rows) -> int {
    TmapSpec s{};
    s.dtype = dt;
    s.rank = 4;
    s.swizzle128 = true;
    s.dims[0] = p.H;
    s.dims[1] = rows;
    s.dims[2] = p.N;
    s.dims[3] = p.B;
    auto stride_bytes = [&](int64_t st, uint64_t fallback) -> uint64_t {
      return st > 0 ? static_cast<uint64_t>(st) * 2 : fallback;   // size-1 dimensions still need a legal stride
    };
    const uint64_t row_pitch = stride_bytes(strides[2], static_cast<uint64_t>(p.H) * 2);
    s.strides_bytes[0] = row_pitch;
    s.strides_bytes[1] = stride_bytes(strides[1], row_pitch * rows);
    s.strides_bytes[2] = stride_bytes(strides[0], row_pitch * rows * p.N);
    s.box[0] = kChunkElems;
    s.box[1] = kBlk;
    s.box[2] = 1;
    s.box[3] = 1;
    return encode_tmap(out, base, s);
  };
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map(&tq, p.q, p.q_strides, p.F)) != IXK_OK) return rc;
  if ((rc = make_map(&tk, p.k, p.k_strides, p.T)) != IXK_OK) return rc;
  if ((rc = make_map(&tv, p.v, p.v_strides, p.T)) != IXK_OK) return rc;
  if ((rc = make_map(&tdo, bp.grad_out, bp.do_strides, p.F)) != IXK_OK) return rc;

  BwdArgs a{};
  a.B = p.B; a.N = p.N; a.H = p.H; a.F = p.F; a.T = p.T;
  a.f_pad = f_pad;
  a.num_kblocks = (p.T + kBlk - 1) / kBlk;
  a.num_qblocks = (p.F + kBlk - 1) / kBlk;
  a.causal = p.causal ? 1 : 0;
  a.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
  a.scale_log2 = p.head_scale * kLog2e;
  a.head_scale = p.head_scale;
  a.bias = static_cast<const uint16_t*>(p.bias);
  a.neg_lse2 = neg_lse2;
  a.delta = delta;
  a.dq_acc = dq_acc;
  a.dk = static_cast<uint16_t*>(bp.dk);
  a.dv = static_cast<uint16_t*>(bp.dv);
  for (int i = 0; i < 3; ++i) {
    a.bias_strides[i] = p.bias_strides[i];
    a.dk_strides[i] = bp.dk_strides[i];
    a.dv_strides[i] = bp.dv_strides[i];
  }
  a.status_word = dev.status_word;

  auto* fn = &fmha_bwd_kernel<kHeadDim, kBias, kBf16>;
  static thread_local int configured_device = -1;
  if (configured_device != dev.device) {
    IXK_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured_device = dev.device;
  }
  const int64_t ctas = static_cast<int64_t>(a.num_kblocks) * p.N * p.B;
  if (ctas > 0x7fffffff) return fail(IXK_UNIMPLEMENTED, "too many (batch, head, key block) work items");
  fn<<<static_cast<unsigned>(ctas), kBwdThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, a);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

template <int kHeadDim>
int launch_bwd_dtype(const BwdProblem& bp, const DeviceInfo& dev, float* neg_lse2, float* delta, float* dq_acc, int f_pad,
                     cudaStream_t stream, bool bias) {
  if (bp.fwd.dtype == IXK_BF16)
    return bias ? launch_bwd_cfg<kHeadDim, true, true>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream)
                : launch_bwd_cfg<kHeadDim, false, true>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream);
  return bias ? launch_bwd_cfg<kHeadDim, true, false>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream)
              : launch_bwd_cfg<kHeadDim, false, false>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream);
}

int head_pad_of(int H) { return H <= 64 ? 64 : 128; }
int f_pad_of(int F) { return (F + kBlk - 1) / kBlk * kBlk; }

}  // namespace

size_t bwd_workspace_bytes(const Problem& p) {
  if (p.B == 0 || p.N == 0 || p.F == 0) return 0;
  if (p.H > 128) {  // the two per-row arrays (256-byte aligned end) + the score-sized scratch of one group of heads
    const size_t rows = (static_cast<size_t>(p.B) * p.N * f_pad_of(p.F) * 2 * sizeof(float) + 255) / 256 * 256;
    return rows + bwd_wide_scratch_bytes(p);
  }
  return static_cast<size_t>(p.B) * p.N * f_pad_of(p.F) * (head_pad_of(p.H) + 2) * sizeof(float);
}

int launch_bwd(const BwdProblem& bp, const DeviceInfo& dev, void* workspace, size_t workspace_bytes,
               cudaStream_t stream) {
  const Problem& p = bp.fwd;
  const size_t need = bwd_workspace_bytes(p);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(IXK_WORKSPACE_TOO_SMALL, "attention backward needs ixk_fmha_bwd_workspace_bytes(desc) bytes of workspace");
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(IXK_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
  const bool wide = p.H > 128;
  const int f_pad = f_pad_of(p.F), head_pad = wide ? 0 : head_pad_of(p.H);   // (no fp32 dQ accumulator on the wide path)
  const int64_t rows = static_cast<int64_t>(p.B) * p.N * f_pad;
  float* neg_lse2 = static_cast<float*>(workspace);
  float* delta = neg_lse2 + rows;
  float* dq_acc = delta + rows;

  PrepArgs pa{};
  pa.B = p.B; pa.N = p.N; pa.H = p.H; pa.F = p.F; pa.f_pad = f_pad; pa.head_pad = head_pad;
  pa.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
  pa.out = static_cast<const uint16_t*>(p.out);
  pa.grad_out = static_cast<const uint16_t*>(bp.grad_out);
  pa.lse = p.lse;
  for (int i = 0; i < 3; ++i) {
    pa.o_strides[i] = p.o_strides[i];
    pa.do_strides[i] = bp.do_strides[i];
  }
  pa.neg_lse2 = neg_lse2;
  pa.delta = delta;
  pa.dq_acc = dq_acc;
  const int prep_grid = static_cast<int>(std::min<int64_t>((rows / 4 + 7) / 8, static_cast<int64_t>(dev.sm_count) * 8));
  bwd_prepare_kernel<<<prep_grid, 256, 0, stream>>>(pa);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();

  if (wide) {
    unsigned char* scratch = static_cast<unsigned char*>(workspace) + (static_cast<size_t>(rows) * 2 * sizeof(float) + 255) / 256 * 256;
    return launch_bwd_wide(bp, dev, neg_lse2, delta, f_pad, scratch, stream);
  }
  int rc;
  const bool bias = p.bias != nullptr;
  if (head_pad == 64) {
    rc = launch_bwd_dtype<64>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream, bias);
  } else {
    rc = launch_bwd_dtype<128>(bp, dev, neg_lse2, delta, dq_acc, f_pad, stream, bias);
  }
  if (rc != IXK_OK) return rc;

  ConvertArgs ca{};
  ca.B = p.B; ca.N = p.N; ca.H = p.H; ca.F = p.F; ca.f_pad = f_pad; ca.head_pad = head_pad;
  ca.is_bf16 = pa.is_bf16;
  ca.head_scale = p.head_scale;
  ca.dq_acc = dq_acc;
  ca.dq = static_cast<uint16_t*>(bp.dq);
  for (int i = 0; i < 3; ++i) ca.dq_strides[i] = bp.dq_strides[i];
  const int64_t pairs = static_cast<int64_t>(p.B) * p.N * p.F * (p.H / 8);
  const int conv_grid = static_cast<int>(std::min<int64_t>((pairs + 255) / 256, static_cast<int64_t>(dev.sm_count) * 8));
  bwd_convert_kernel<<<conv_grid, 256, 0, stream>>>(ca);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}
}  // namespace fmha
}  // namespace ixk

