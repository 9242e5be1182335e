// Persistent, warp-specialised tcgen05 GEMM with a fused epilogue for sm_100a.
//
//   D[M,N] = act( acc_scale * (A[M,K] . B[K,N]) + bias[n] + beta * C[M,N] )
//
// Replaces the XeTLA hgemm_* kernels (xla/service/gpu/xetla/gemm/hgemm_impl.h:101-459)
// and the oneDNN matmul + post-ops call (xla/service/gpu/onednn_matmul_utils.cc:394-491).
//
// One CTA per SM, 192 threads:
//   warp 0      TMA producer: A/B k-slabs of 128 bytes into a 128B-swizzled shared-memory ring
//   warp 1      TMEM allocation + single-thread tcgen05.mma issue (128 x BLOCK_N x 32 bytes of K)
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator, bias/activation/residual in fp32,
//               one rounding, 16-byte global stores
// The accumulator is double-buffered in TMEM (2 x BLOCK_N columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  Either operand may be K-major or MN-major in global
// memory; the TMA box shape and the UMMA descriptors follow the operand's major-ness, so no
// transposed copy is ever made.  Operands are 16-bit (kind::f16) or 8-bit (kind::f8f6f4).
#include <type_traits>

#include "gemm_sm100.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "ptx.cuh"

namespace ixk {
namespace gemm {

namespace {

static_assert(int(kKindF16) == int(ptx::kKindF16) && int(kKindF8) == int(ptx::kKindF8) &&
              int(kKindTf32) == int(ptx::kKindTf32) && int(kKindI8) == int(ptx::kKindI8), "MMA kind codes");
constexpr int kBlockM = 128;
constexpr int kSlabBytes = 128;  // bytes of K per shared-memory row (one swizzle span)
constexpr int kThreads = 192;
constexpr int kATileBytes = kBlockM * kSlabBytes;  // 16 KiB

template <int kBlockN>
struct Cfg {
  static constexpr int kBTileBytes = kBlockN * kSlabBytes;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * kBlockN;
  static constexpr int kBarrierBytes = 256;
  // output staging: two boxes of 32 rows x 128 bytes per epilogue warp
  static constexpr int kStagingBytes = 4 * 2 * 32 * 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;  // + align slack
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Site codes written to the status word by a wait that gave up.
enum : int { kSiteProducer = 101, kSiteMmaFull = 102, kSiteMmaAcc = 103, kSiteEpilogue = 104 };

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) == x / (1 + exp(-2u)),  u = sqrt(2/pi) (x + 0.044715 x^3)
  const float u = 0.7978845608028654f * x * fmaf(0.044715f * x, x, 1.0f);
  const float e = ptx::ex2_approx(-2.885390081777927f * u);  // exp(-2u) = 2^(-2u log2 e)
  return __fdividef(x, 1.0f + e);
}

__device__ __forceinline__ void load_row16(const void* base, int64_t elem_off, int dtype, int count,
                                           bool vec_ok, float (&out)[32]) {
  // Reads `count` (<= 32) consecutive elements of type `dtype` starting at elem_off into out[].
  if (dtype == IXK_F32) {
    const float* p = static_cast<const float*>(base) + elem_off;
    if (vec_ok && count == 32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
        out[4 * i + 0] = v.x;
        out[4 * i + 1] = v.y;
        out[4 * i + 2] = v.z;
        out[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = i < count ? __ldg(p + i) : 0.0f;
    }
  } else {
    const uint16_t* p = static_cast<const uint16_t*>(base) + elem_off;
    uint32_t w[16];
    if (vec_ok && count == 32) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
        w[4 * i + 0] = v.x;
        w[4 * i + 1] = v.y;
        w[4 * i + 2] = v.z;
        w[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t lo = (2 * i) < count ? __ldg(p + 2 * i) : 0u;
        const uint32_t hi = (2 * i + 1) < count ? __ldg(p + 2 * i + 1) : 0u;
        w[i] = lo | (hi << 16);
      }
    }
    if (dtype == IXK_BF16) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
      }
    }
  }
}

// 32 fp32 values -> 16 words of 16-bit pairs, rounded once.
__device__ __forceinline__ void pack_row16(const float (&v)[32], int dtype, uint32_t* w) {
  if (dtype == IXK_BF16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
}

__device__ __forceinline__ void store_row(void* base, int64_t elem_off, int dtype, int count,
                                          bool vec_ok, const float (&v)[32]) {
  if (dtype == IXK_F32 || dtype == IXK_S32) {  // 32-bit words, copied bit for bit
    float* p = static_cast<float*>(base) + elem_off;
    if (vec_ok && count == 32) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < count) p[i] = v[i];
    }
  } else {
    uint32_t w[16];
    if (dtype == IXK_BF16) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    uint16_t* p = static_cast<uint16_t*>(base) + elem_off;
    if (vec_ok && count == 32) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        reinterpret_cast<uint4*>(p)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (2 * i < count) p[2 * i] = static_cast<uint16_t>(w[i] & 0xffffu);
        if (2 * i + 1 < count) p[2 * i + 1] = static_cast<uint16_t>(w[i] >> 16);
      }
    }
  }
}

// Grouped raster: consecutive tile ids walk down a band of `kGroupM` row-blocks before moving
// to the next column-block, so the CTAs running at the same time share A and B slabs in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& bz, int& bm,
                                            int& bn) {
  constexpr int kGroupM = 8;
  const int per_batch = tiles_m * tiles_n;
  bz = t / per_batch;
  t -= bz * per_batch;
  const int band = kGroupM * tiles_n;
  const int g = t / band;
  const int first_m = g * kGroupM;
  const int rows = min(tiles_m - first_m, kGroupM);
  const int r = t - g * band;
  bm = first_m + r % rows;
  bn = r / rows;
}

// One tile's epilogue for the calling warp (TMEM lanes [32 quarter, 32 quarter + 32) of the
// accumulator at tmem_acc): scale, bias, residual, activation, one rounding, store.
template <int kBlockN>
__device__ __forceinline__ void epilogue_tile(const KernelArgs& args, const CUtensorMap* tmap_d_ptr, uint32_t tmem_acc,
                                              uint32_t stage_smem, int bz, int bm, int bn, int quarter, int lane,
                                              uint32_t& n_store, int d_row_shift = 0) {
  const CUtensorMap& tmap_d = *tmap_d_ptr;
  if (bm * kBlockM >= args.M) return;  // a CTA pair's second half past the last row block
  const int row_in_tile = quarter * 32 + lane;
  const bool vec_d = args.d_vec_ok != 0;
  const bool vec_c = args.c_vec_ok != 0;
  const bool vec_bias = args.bias_vec_ok != 0;
      const int m = bm * kBlockM + row_in_tile;
    const bool row_ok = m < args.M;
    const int64_t d_row = bz * args.d_batch_stride + static_cast<int64_t>(m) * args.ldd;
    const int64_t c_row = bz * args.c_batch_stride + static_cast<int64_t>(m) * args.ldc;
    // 32 columns of this thread's row: accumulator -> scale, bias, residual, activation
    auto chunk = [&](int c0, int n, int count, float (&v)[32]) {
      uint32_t r[32];
      ptx::tmem_ld_32x32(tmem_acc + c0, r);
      ptx::tmem_ld_wait();
      if (args.out_dtype == IXK_S32) {  // integer accumulator (kind::i8): the bits go out as they are
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        return;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * args.acc_scale;
      if (args.bias != nullptr) {
        float b[32];
        load_row16(args.bias, bz * args.bias_batch_stride + n, args.bias_dtype, count, vec_bias, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += b[i];
      }
      if (args.c != nullptr && row_ok) {
        float cc[32];
        load_row16(args.c, c_row + n, args.out_dtype, count, vec_c, cc);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(args.beta, cc[i], v[i]);
      }
      if (args.aux != nullptr && row_ok)  // the value the activation is applied to, as a second output
        store_row(args.aux, bz * args.aux_batch_stride + static_cast<int64_t>(m) * args.ld_aux + n, args.out_dtype, count,
                  args.aux_vec_ok != 0, v);
      if (args.act == kActRelu) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
      } else if (args.act == kActGelu) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
      }
    };
    if (args.d_tma) {
      // 16-bit output through shared memory: each warp writes its 32 rows x 64 columns into a
      // 128-byte-swizzled box of its own (lane = row, conflict-free) and one lane hands the box
      // to a TMA store; two boxes per warp, so a box is only rewritten after the store issued
      // two passes earlier has read it.  Stored from registers, a warp's 16-byte stores land in
      // 32 different lines each; those requests queue in front of the producer's and the
      // issuer's barrier traffic and cost 8-11 % of the kernel.
#pragma unroll 1
      for (int c0 = 0; c0 < kBlockN; c0 += 64) {
        const int n = bn * kBlockN + c0;
        if (n >= args.N) break;  // warp-uniform
        uint32_t wv[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int nh = n + 32 * half;
          if (nh < args.N) {  // warp-uniform
            float v[32];
            chunk(c0 + 32 * half, nh, min(32, args.N - nh), v);
            pack_row16(v, args.out_dtype, &wv[16 * half]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) wv[16 * half + i] = 0u;
          }
        }
        const uint32_t box = stage_smem + static_cast<uint32_t>((quarter * 2 + (n_store & 1)) * 4096);
        if (lane == 0) ptx::bulk_wait_group_read<1>();
        __syncwarp();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t addr = box + static_cast<uint32_t>(lane * 128 + ((g ^ (lane & 7)) << 4));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(wv[4 * g]), "r"(wv[4 * g + 1]),
                       "r"(wv[4 * g + 2]), "r"(wv[4 * g + 3])
                       : "memory");
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_3d(&tmap_d, box, n, bm * kBlockM + quarter * 32 - d_row_shift, bz);
          ptx::bulk_commit_group();
        }
        ++n_store;
      }
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < kBlockN; c0 += 32) {
        const int n = bn * kBlockN + c0;
        if (n >= args.N) break;  // warp-uniform
        const int count = min(32, args.N - n);
        float v[32];
        chunk(c0, n, count, v);
        if (row_ok) store_row(args.d, d_row + n, args.out_dtype, count, vec_d, v);
      }
    }
}

template <int kBlockN, int kKind>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_d, const KernelArgs args) {
  using C = Cfg<kBlockN>;
  constexpr int kStages = C::kStages;
  constexpr int kElemBytes = kKind == ptx::kKindF16 ? 2 : (kKind == ptx::kKindTf32 ? 4 : 1);
  constexpr int kSlabElems = kSlabBytes / kElemBytes;  // K elements per pipeline stage
  constexpr int kUmmaK = 32 / kElemBytes;              // K elements per tcgen05.mma

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t stage_smem = smem_base + kStages * C::kStageBytes;  // output staging boxes
  const uint32_t bar_base = stage_smem + C::kStagingBytes;
  // barrier slots (8 bytes each): full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  uint8_t* tail = smem_gen + kStages * C::kStageBytes + C::kStagingBytes + 8 * (2 * kStages + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ptx::AbortCtl ctl{abort_flag, args.status_word};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(acc_full_bar(b), 1);
      ptx::mbar_init(acc_empty_bar(b), 128);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (args.d_tma) ptx::prefetch_tmap(&tmap_d);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (args.K + kSlabElems - 1) / kSlabElems;
  const int num_tiles = args.tiles_m * args.tiles_n * args.batch;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // (all 32 lanes walk the loop; an elected lane issues the copies)
    {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int bz, bm, bn;
        tile_coords(t, args.tiles_m, args.tiles_n, bz, bm, bn);
        const int m0 = bm * kBlockM;
        const int n0 = bn * kBlockN;
        const int az = args.a_broadcast ? 0 : bz;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, ctl, kSiteProducer)) {
            alive = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * C::kStageBytes;
          const uint32_t b_dst = a_dst + kATileBytes;
          const uint32_t bar = full_bar(stage);
          const int k0 = kb * kSlabElems;
          if (ptx::elect_one()) {
          ptx::mbar_expect_tx(bar, C::kStageBytes);
          if (args.a_mn_major) {
            // box = [kSlabElems k-rows][128 bytes of M]; one box per 128-byte column block
#pragma unroll
            for (int i = 0; i < kBlockM / kSlabElems; ++i)
              ptx::tma_load_3d(a_dst + i * (kSlabElems * kSlabBytes), &tmap_a, bar,
                               m0 + i * kSlabElems, k0, az);
          } else {
            ptx::tma_load_3d(a_dst, &tmap_a, bar, k0, m0, az);
          }
          if (args.b_mn_major) {
#pragma unroll
            for (int i = 0; i < kBlockN / kSlabElems; ++i)
              ptx::tma_load_3d(b_dst + i * (kSlabElems * kSlabBytes), &tmap_b, bar,
                               n0 + i * kSlabElems, k0, bz);
          } else {
            ptx::tma_load_3d(b_dst, &tmap_b, bar, k0, n0, bz);
          }
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // (all 32 lanes walk the loop; an elected lane issues each MMA and commit)
    {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      // K-major: 8-row groups are 1024 B apart, a k-step moves 32 B inside the swizzle span.
      // MN-major: 8-k groups are 1024 B apart, 128-byte column blocks are a whole slab apart,
      //           a k-step moves kUmmaK rows of 128 B.
      const uint32_t a_lbo = args.a_mn_major ? kSlabElems * kSlabBytes : 16;
      const uint32_t b_lbo = args.b_mn_major ? kSlabElems * kSlabBytes : 16;
      const uint32_t a_kstep = args.a_mn_major ? kUmmaK * kSlabBytes : 32;
      const uint32_t b_kstep = args.b_mn_major ? kUmmaK * kSlabBytes : 32;
      // 32-bit elements, MN-major: the 128-byte swizzle in 32-byte pieces, groups of 4 k rows
      const bool a_sw32 = kKind == ptx::kKindTf32 && args.a_mn_major, b_sw32 = kKind == ptx::kKindTf32 && args.b_mn_major;
      const uint32_t a_sbo = a_sw32 ? 512 : 1024, b_sbo = b_sw32 ? 512 : 1024;
      const uint32_t a_type = a_sw32 ? 1 : 2, b_type = b_sw32 ? 1 : 2;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        if (!ptx::mbar_wait(acc_empty_bar(buf), acc_phase ^ 1u, ctl, kSiteMmaAcc)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(full_bar(stage), phase, ctl, kSiteMmaFull)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_src = smem_base + stage * C::kStageBytes;
          const uint32_t b_src = a_src + kATileBytes;
#pragma unroll
          for (int ks = 0; ks < kSlabElems / kUmmaK; ++ks) {
            const uint64_t da = ptx::umma_smem_desc(a_src + ks * a_kstep, a_lbo, a_sbo, a_type);
            const uint64_t db = ptx::umma_smem_desc(b_src + ks * b_kstep, b_lbo, b_sbo, b_type);
            ptx::umma_ss_elect<kKind>(d_tmem, da, db, args.idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          ptx::umma_commit_elect(empty_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        ptx::umma_commit_elect(acc_full_bar(buf));
        buf ^= 1;
        if (buf == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    int buf = 0;
    uint32_t acc_phase = 0;
    uint32_t n_store = 0;  // TMA stores issued by this warp (alternating between its two boxes)
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int bz, bm, bn;
      tile_coords(t, args.tiles_m, args.tiles_n, bz, bm, bn);
      if (!ptx::mbar_wait(acc_full_bar(buf), acc_phase, ctl, kSiteEpilogue)) break;
      ptx::tc_fence_after_sync();
      epilogue_tile<kBlockN>(args, &tmap_d, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBlockN, stage_smem,
                             bz, bm, bn, quarter, lane, n_store);
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(acc_empty_bar(buf));
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1u;
    }
    // the staging boxes must outlive the stores that read them
    if (args.d_tma && lane == 0) ptx::bulk_wait_group<0>();
  }

  // Teardown.  On the abort path give copies still in flight time to land before the
  // shared memory they target is released.
  if (*abort_flag != 0) __nanosleep(2000000);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs works on a 256 x 256 tile (tcgen05 cta_group::2).  Each
// CTA loads its own 128 rows of A and its own 128 columns of B per k-slab, 32 KB instead of the
// 48 KB a lone CTA needs for 128 x 256, so the operand traffic out of L2 drops by a third; that
// traffic (17 TB/s for all SMs) is what bounds the single-CTA kernel.  The even CTA's MMA warp
// issues for both; its commits arrive on the barriers of both CTAs, and both CTAs' TMA copies are
// counted on the even CTA's full barrier.  Everything else is per CTA as above.
struct PairCfg {
  static constexpr int kBlockN = 256;                       // tile columns (128 per CTA as B rows)
  static constexpr int kStageBytes = 2 * kATileBytes;       // A 128 x 128 B + B half 128 x 128 B
  static constexpr int kStages = (192 * 1024) / kStageBytes;  // 6
  static constexpr int kTmemCols = 2 * kBlockN;
  static constexpr int kStagingBytes = 4 * 2 * 32 * 128;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};
enum : int { kSitePairFull = 111, kSitePairPeer = 112, kSitePairAcc = 113, kSitePairForward = 114 };

// The tensor maps of D: one, or one per destination of a scattered output (rows of D dealt out
// in equal blocks to up to kMaxScatter buffers, each a dense [M / kDests', N] matrix).
template <int kDests>
struct OutputMaps {
  CUtensorMap m[kDests];
};

template <int kKind, int kDests>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ OutputMaps<kDests> tmaps_d, const KernelArgs args) {
  using C = PairCfg;
  constexpr int kStages = C::kStages;
  constexpr int kBlockN = C::kBlockN;
  constexpr int kHalfN = kBlockN / 2;
  constexpr int kElemBytes = kKind == ptx::kKindF16 ? 2 : (kKind == ptx::kKindTf32 ? 4 : 1);
  constexpr int kSlabElems = kSlabBytes / kElemBytes;
  constexpr int kUmmaK = 32 / kElemBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t stage_smem = smem_base + kStages * C::kStageBytes;
  const uint32_t bar_base = stage_smem + C::kStagingBytes;
  // barrier slots: full[kStages], empty[kStages], peer_full[kStages] (even CTA), acc_full[2], acc_empty[2] (even CTA)
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto peer_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (3 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (3 * kStages + 2 + b); };
  uint8_t* tail = smem_gen + kStages * C::kStageBytes + C::kStagingBytes + 8 * (3 * kStages + 4);
  static_assert(8 * (3 * kStages + 4) + 8 <= C::kBarrierBytes, "barrier area");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0: issues the MMAs, 1: its partner
  ptx::AbortCtl ctl{abort_flag, args.status_word};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
      ptx::mbar_init(peer_full_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(acc_full_bar(b), 1);
      ptx::mbar_init(acc_empty_bar(b), 256);  // the epilogue threads of both CTAs
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (args.d_tma) ptx::prefetch_tmap(&tmaps_d.m[0]);
  }
  __syncthreads();
  ptx::cluster_sync_all();  // both CTAs' barriers exist before anyone arrives on them remotely
  // tcgen05.alloc / dealloc with cta_group::2 are collective over the pair: one warp of EACH CTA
  // executes them (with the even CTA alone the odd CTA's columns were never released, and the
  // next launch's allocation on that SM did not return).
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (args.K + kSlabElems - 1) / kSlabElems;
  const int tiles_m2 = (args.tiles_m + 1) / 2;  // pair tiles along M
  const int num_tiles = tiles_m2 * args.tiles_n * args.batch;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA: its A rows, its B columns)
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int t = pair_id; t < num_tiles && alive; t += num_pairs) {
      int bz, bm2, bn;
      tile_coords(t, tiles_m2, args.tiles_n, bz, bm2, bn);
      const int m0 = (bm2 * 2 + static_cast<int>(rank)) * kBlockM;
      const int n0 = bn * kBlockN + static_cast<int>(rank) * kHalfN;
      const int az = args.a_broadcast ? 0 : bz;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(empty_bar(stage), phase ^ 1u, ctl, kSiteProducer)) {
          alive = false;
          break;
        }
        const uint32_t a_dst = smem_base + stage * C::kStageBytes;
        const uint32_t b_dst = a_dst + kATileBytes;
        // both CTAs' copies are counted on the EVEN CTA's barrier, which its issuer waits on
        const uint32_t bar = ptx::map_to_cta(full_bar(stage), 0);
        const int k0 = kb * kSlabElems;
        if (ptx::elect_one()) {
          if (rank == 0) ptx::mbar_expect_tx(full_bar(stage), 2 * C::kStageBytes);
          if (args.a_mn_major) {
#pragma unroll
            for (int i = 0; i < kBlockM / kSlabElems; ++i)
              ptx::tma_load_3d_pair(a_dst + i * (kSlabElems * kSlabBytes), &tmap_a, bar, m0 + i * kSlabElems, k0, az);
          } else {
            ptx::tma_load_3d_pair(a_dst, &tmap_a, bar, k0, m0, az);
          }
          if (args.b_mn_major) {
#pragma unroll
            for (int i = 0; i < kHalfN / kSlabElems; ++i)
              ptx::tma_load_3d_pair(b_dst + i * (kSlabElems * kSlabBytes), &tmap_b, bar, n0 + i * kSlabElems, k0, bz);
          } else {
            ptx::tma_load_3d_pair(b_dst, &tmap_b, bar, k0, n0, bz);
          }
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && rank == 1) {
    // (the odd CTA's second warp only takes part in the TMEM allocation)
  } else if (warp == 1) {
    // ------------------------------------------------------------ even CTA: MMA issuer for the pair
    int stage = 0;
    uint32_t phase = 0;
    int buf = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    const uint32_t a_lbo = args.a_mn_major ? kSlabElems * kSlabBytes : 16;
    const uint32_t b_lbo = args.b_mn_major ? kSlabElems * kSlabBytes : 16;
    const uint32_t a_kstep = args.a_mn_major ? kUmmaK * kSlabBytes : 32;
    const uint32_t b_kstep = args.b_mn_major ? kUmmaK * kSlabBytes : 32;
    // 32-bit elements, MN-major: the 128-byte swizzle in 32-byte pieces, groups of 4 k rows
    const bool a_sw32 = kKind == ptx::kKindTf32 && args.a_mn_major, b_sw32 = kKind == ptx::kKindTf32 && args.b_mn_major;
    const uint32_t a_sbo = a_sw32 ? 512 : 1024, b_sbo = b_sw32 ? 512 : 1024;
    const uint32_t a_type = a_sw32 ? 1 : 2, b_type = b_sw32 ? 1 : 2;
    for (int t = pair_id; t < num_tiles && alive; t += num_pairs) {
      if (!ptx::mbar_wait(acc_empty_bar(buf), acc_phase ^ 1u, ctl, kSitePairAcc)) break;
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + buf * kBlockN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(full_bar(stage), phase, ctl, kSitePairFull)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t a_src = smem_base + stage * C::kStageBytes;
        const uint32_t b_src = a_src + kATileBytes;
#pragma unroll
        for (int ks = 0; ks < kSlabElems / kUmmaK; ++ks) {
          const uint64_t da = ptx::umma_smem_desc(a_src + ks * a_kstep, a_lbo, a_sbo, a_type);
          const uint64_t db = ptx::umma_smem_desc(b_src + ks * b_kstep, b_lbo, b_sbo, b_type);
          ptx::umma_ss_pair_elect<kKind>(d_tmem, da, db, args.idesc, (kb | ks) != 0 ? 1u : 0u);
        }
        ptx::umma_commit_pair_elect(empty_bar(stage));  // both CTAs' producers may refill the slot
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!alive) break;
      ptx::umma_commit_pair_elect(acc_full_bar(buf));  // both CTAs' epilogue warps
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------ epilogue (each CTA: its 128 rows)
    const int quarter = warp & 3;
    int buf = 0;
    uint32_t acc_phase = 0;
    uint32_t n_store = 0;
    for (int t = pair_id; t < num_tiles; t += num_pairs) {
      int bz, bm2, bn;
      tile_coords(t, tiles_m2, args.tiles_n, bz, bm2, bn);
      if (!ptx::mbar_wait(acc_full_bar(buf), acc_phase, ctl, kSiteEpilogue)) break;
      ptx::tc_fence_after_sync();
      const int bm = bm2 * 2 + static_cast<int>(rank);
      // scattered output: this row block's destination and the row that destination starts at
      const int dest = kDests > 1 ? (bm * kBlockM) / args.scatter_rows : 0;
      epilogue_tile<kBlockN>(args, &tmaps_d.m[dest], tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBlockN,
                             stage_smem, bz, bm, bn, quarter, lane, n_store, kDests > 1 ? dest * args.scatter_rows : 0);
      ptx::tc_fence_before_sync();
      if (rank == 0) {
        ptx::mbar_arrive(acc_empty_bar(buf));
      } else {
        ptx::mbar_arrive_cluster(acc_empty_bar(buf), 0);
      }
      buf ^= 1;
      if (buf == 0) acc_phase ^= 1u;
    }
    if (args.d_tma && lane == 0) {
      ptx::bulk_wait_group<0>();
      if (kDests > 1) {  // the stores went to other GPUs: complete at system scope before the kernel ends
        ptx::fence_proxy_async_all();
        __threadfence_system();
      }
    }
  }

  // Teardown: neither CTA may leave while its partner can still read its shared memory or arrive
  // on its barriers.
  if (*abort_flag != 0) __nanosleep(2000000);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
  ptx::cluster_sync_all();
}

template <int kBlockN, int kKind>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const KernelArgs& args,
               int grid, cudaStream_t stream) {
  using C = Cfg<kBlockN>;
  auto* fn = &gemm_kernel<kBlockN, kKind>;
  static thread_local int configured_device = -1;
  int dev = 0;
  IXK_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    IXK_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured_device = dev;
  }
  fn<<<grid, kThreads, C::kSmemBytes, stream>>>(ta, tb, td, args);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

template <int kKind, int kDests>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const OutputMaps<kDests>& td, const KernelArgs& args,
                int pairs, cudaStream_t stream) {
  auto* fn = &gemm_pair_kernel<kKind, kDests>;
  static thread_local int configured_device = -1;
  int dev = 0;
  IXK_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    IXK_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  IXK_CUDA_OK(cudaLaunchKernelEx(&cfg, fn, ta, tb, td, args));
  count_launch();
  return IXK_OK;
}

}  // namespace

int pick_block_n(int64_t M, int64_t N, int64_t batch, int sm_count) {
  // Largest N-tile that still gives every SM a tile; wide tiles halve the shared-memory
  // traffic per flop, narrow ones keep skinny (weight-streaming) problems spread over the chip.
  const int64_t tiles_m = (M + kBlockM - 1) / kBlockM;
  for (int bn : {256, 128}) {
    const int64_t tiles = tiles_m * ((N + bn - 1) / bn) * batch;
    if (tiles >= sm_count) return bn;
  }
  return 64;
}

int launch(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  const int es = p.kind == ptx::kKindF16 ? 2 : (p.kind == ptx::kKindTf32 ? 4 : 1);
  const int slab_elems = kSlabBytes / es;
  int bn = p.force_block_n > 0 ? p.force_block_n : pick_block_n(p.M, p.N, p.batch, dev.sm_count);
  if (bn != 64 && bn != 128 && bn != 256) return fail(IXK_INVALID_ARGUMENT, "block_n must be 64, 128 or 256");
  // An MN-major 8-bit B tile is loaded in 128-column boxes (one swizzle span), so it cannot be
  // narrower than 128 columns.
  if (es == 1 && p.b_mn_major && bn < 128) bn = 128;

  // Large problems run on CTA pairs (256 x 256 tiles): worth it once every pair of SMs has a tile.
  const int64_t tiles_m_all = (p.M + kBlockM - 1) / kBlockM;
  const int64_t pair_tiles = ((tiles_m_all + 1) / 2) * ((p.N + 255) / 256) * p.batch;
  bool pair = bn == 256 && tiles_m_all >= 2 && pair_tiles >= dev.sm_count / 2;
  if (const char* env = std::getenv("IXK_GEMM_PAIR")) pair = pair && std::atoi(env) != 0;
  const int b_box_rows = pair ? 128 : bn;
  if (p.scatter_world > 0) {
    // Only the kernel that large projections run on stores to several destinations, and only
    // whole row blocks of one CTA.
    if (p.scatter_world > kMaxScatter) return fail(IXK_INVALID_ARGUMENT, "too many destinations");
    if (!pair || p.kind != ptx::kKindF16 || p.batch != 1 || p.out_dtype == IXK_F32 || p.aux != nullptr ||
        p.M % (static_cast<int64_t>(p.scatter_world) * kBlockM) != 0 || p.N % 8 != 0)
      return fail(IXK_UNIMPLEMENTED,
                  "a scattered output needs a 16-bit, un-batched problem large enough for the CTA-pair kernel "
                  "(at least 74 tiles of 256 x 256), M a multiple of 128 x destinations and N a multiple of 8");
    for (int o = 0; o < p.scatter_world; ++o)
      if (p.scatter_dest[o] == nullptr || (reinterpret_cast<uintptr_t>(p.scatter_dest[o]) & 15u) != 0)
        return fail(IXK_INVALID_ARGUMENT, "a destination of the scattered output is NULL or not 16-byte aligned");
  }

  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : es == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                           : (p.ab_dtype == IXK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  // A is [M,K]: K-major when K is contiguous.  B is [K,N]: MN-major when N is contiguous.
  auto make_map = [&](CUtensorMap* out, const void* base, bool mn_major, int64_t mn, int64_t ld,
                      int64_t batch_stride, int block_mn, bool broadcast) -> int {
    TmapSpec s{};
    s.dtype = dt;
    s.rank = 3;
    s.swizzle128 = true;
    s.swizzle_atom32 = mn_major && es == 4;  // what an MN-major operand of 32-bit elements needs
    if (mn_major) {
      s.dims[0] = mn;
      s.dims[1] = p.K;
      s.box[0] = slab_elems;  // 128 bytes of M/N
      s.box[1] = slab_elems;  // k rows of one stage
    } else {
      s.dims[0] = p.K;
      s.dims[1] = mn;
      s.box[0] = slab_elems;
      s.box[1] = block_mn;
    }
    s.dims[2] = broadcast ? 1 : p.batch;
    s.box[2] = 1;
    s.strides_bytes[0] = static_cast<uint64_t>(ld) * es;
    // A batch of one still needs a legal (16-byte multiple, non-zero) stride.
    s.strides_bytes[1] = (p.batch > 1 && !broadcast) ? static_cast<uint64_t>(batch_stride) * es
                                                     : s.strides_bytes[0] * s.dims[1];
    return encode_tmap(out, base, s);
  };
  CUtensorMap ta, tb;
  int rc = make_map(&ta, p.a, p.a_mn_major, p.M, p.lda, p.a_batch_stride, kBlockM, p.a_broadcast);
  if (rc != IXK_OK) return rc;
  rc = make_map(&tb, p.b, p.b_mn_major, p.N, p.ldb, p.b_batch_stride, b_box_rows, false);
  if (rc != IXK_OK) return rc;

  KernelArgs k{};
  k.M = static_cast<int>(p.M);
  k.N = static_cast<int>(p.N);
  k.K = static_cast<int>(p.K);
  k.batch = static_cast<int>(p.batch);
  k.tiles_m = static_cast<int>((p.M + kBlockM - 1) / kBlockM);
  k.tiles_n = static_cast<int>((p.N + bn - 1) / bn);
  k.a_mn_major = p.a_mn_major;
  k.b_mn_major = p.b_mn_major;
  k.idesc = ptx::umma_idesc(p.a_fmt, p.b_fmt, p.a_mn_major ? 1 : 0, p.b_mn_major ? 1 : 0, pair ? 2 * kBlockM : kBlockM, bn,
                            p.kind == ptx::kKindI8 ? 2u : 1u);
  k.bias = p.bias;
  k.c = (p.beta != 0.0f) ? p.c : nullptr;
  k.d = p.d;
  k.ldd = p.ldd;
  k.ldc = p.ldc;
  k.d_batch_stride = p.d_batch_stride;
  k.c_batch_stride = p.c_batch_stride;
  k.out_dtype = p.out_dtype;
  k.bias_dtype = p.bias_dtype;
  k.act = p.act;
  k.acc_scale = p.acc_scale;
  k.beta = p.beta;
  k.status_word = dev.status_word;
  const int out_es = (p.out_dtype == IXK_F32 || p.out_dtype == IXK_S32) ? 4 : 2;
  const int bias_es = p.bias_dtype == IXK_F32 ? 4 : 2;
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  k.d_vec_ok = aligned16(p.d) && (p.ldd * out_es) % 16 == 0 && (p.d_batch_stride * out_es) % 16 == 0;
  k.c_vec_ok = k.c && aligned16(p.c) && (p.ldc * out_es) % 16 == 0 && (p.c_batch_stride * out_es) % 16 == 0;
  k.bias_vec_ok = p.bias && aligned16(p.bias) && (p.bias_batch_stride * bias_es) % 16 == 0;
  k.a_broadcast = p.a_broadcast ? 1 : 0;
  k.bias_batch_stride = p.bias_batch_stride;
  k.aux = p.aux;
  k.ld_aux = p.ld_aux;
  k.aux_batch_stride = p.aux_batch_stride;
  k.aux_vec_ok = p.aux && aligned16(p.aux) && (p.ld_aux * out_es) % 16 == 0 && (p.aux_batch_stride * out_es) % 16 == 0;
  (void)bias_es;
  // A 16-bit D whose rows start on 16-byte boundaries leaves through shared memory and TMA stores.
  CUtensorMap td = ta;  // placeholder unless D qualifies
  k.d_tma = (out_es == 2 && k.d_vec_ok) ? 1 : 0;
  if (k.d_tma) {
    TmapSpec s{};
    s.dtype = p.out_dtype == IXK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    s.rank = 3;
    s.swizzle128 = true;
    s.dims[0] = p.N;
    s.dims[1] = p.M;
    s.dims[2] = p.batch;
    s.box[0] = 64;
    s.box[1] = 32;
    s.box[2] = 1;
    s.strides_bytes[0] = static_cast<uint64_t>(p.ldd) * 2;
    s.strides_bytes[1] = p.batch > 1 ? static_cast<uint64_t>(p.d_batch_stride) * 2 : s.strides_bytes[0] * s.dims[1];
    if ((rc = encode_tmap(&td, p.d, s)) != IXK_OK) return rc;
  }
  OutputMaps<kMaxScatter> td_scatter;
  if (p.scatter_world > 0) {
    k.d_tma = 1;
    k.scatter_rows = static_cast<int>(p.M / p.scatter_world);
    TmapSpec s{};
    s.dtype = p.out_dtype == IXK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    s.rank = 3;
    s.swizzle128 = true;
    s.dims[0] = p.N;
    s.dims[1] = k.scatter_rows;
    s.dims[2] = 1;
    s.box[0] = 64;
    s.box[1] = 32;
    s.box[2] = 1;
    s.strides_bytes[0] = static_cast<uint64_t>(p.N) * 2;
    s.strides_bytes[1] = s.strides_bytes[0] * s.dims[1];
    for (int o = 0; o < kMaxScatter; ++o)
      if ((rc = encode_tmap(&td_scatter.m[o], p.scatter_dest[o < p.scatter_world ? o : 0], s)) != IXK_OK) return rc;
  }

  auto dispatch = [&](auto kind_tag) -> int {
    constexpr int kKind = decltype(kind_tag)::value;
    if (pair) {
      const int pairs = static_cast<int>(pair_tiles < dev.sm_count / 2 ? pair_tiles : dev.sm_count / 2);
      if (p.scatter_world > 0) {
        if constexpr (kKind == ptx::kKindF16) return launch_pair<kKind, kMaxScatter>(ta, tb, td_scatter, k, pairs, stream);
      }
      OutputMaps<1> one;
      one.m[0] = td;
      return launch_pair<kKind, 1>(ta, tb, one, k, pairs, stream);
    }
    const int64_t tiles = static_cast<int64_t>(k.tiles_m) * k.tiles_n * k.batch;
    const int grid = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
    if (bn == 256) return launch_one<256, kKind>(ta, tb, td, k, grid, stream);
    if (bn == 128) return launch_one<128, kKind>(ta, tb, td, k, grid, stream);
    return launch_one<64, kKind>(ta, tb, td, k, grid, stream);
  };
  switch (p.kind) {
    case ptx::kKindF8: return dispatch(std::integral_constant<int, ptx::kKindF8>{});
    case ptx::kKindTf32: return dispatch(std::integral_constant<int, ptx::kKindTf32>{});
    case ptx::kKindI8: return dispatch(std::integral_constant<int, ptx::kKindI8>{});
    default: return dispatch(std::integral_constant<int, ptx::kKindF16>{});
  }
}

}  // namespace gemm
}  // namespace ixk
