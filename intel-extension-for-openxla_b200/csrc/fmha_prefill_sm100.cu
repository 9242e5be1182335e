// Flash-attention forward for sm_100a on tcgen05 / TMEM.
//
//   O = softmax(head_scale * Q.K^T + bias, masked) . V        one (batch, head, query block) per CTA
//
// Replaces FmhaForwardKernel (xla/service/gpu/xetla/sdp/fmha_forward.h:526-612).  Where the
// XeTLA kernel keeps Q in shared local memory, re-normalises P on every key block and reduces
// rows across sub-groups through shared memory, this one is built on the Blackwell units:
//
//   warp 0        TMA producer: Q once, then K_0, V_0, K_1, V_1 ... through a shared-memory ring
//   warp 1        tcgen05.mma issuer:  S_t = Q_t.K_j^T  (A, B from shared memory, S in TMEM)
//                                      O_t += P_t.V_j   (A = P from TMEM, B = V from shared memory)
//   warps 4-7     softmax for query tile 0: one thread owns one row of S (a TMEM lane), so
//   warps 8-11    softmax for query tile 1  row max / row sum need no cross-thread traffic
//
// A CTA carries kQTiles tiles of 128 query rows; with two tiles the tensor core works on one
// tile's S / P.V while the other tile's softmax runs.  P overwrites S in place in TMEM as
// packed 16-bit pairs.  The running maximum is only raised when it moved by more than 2^8
// (exact: the same stale maximum scales P, the row sum and O), which keeps the O rescale off
// the common path.  exp is evaluated as exp2 with head_scale*log2(e) folded in.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "fmha_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace fmha {

namespace {

constexpr int kBlockQ = 128;   // query rows per tile (= TMEM lanes)
constexpr int kBlockKV = 128;  // keys per block
constexpr int kChunkElems = 64;                       // 16-bit elements per 128-byte swizzle row
constexpr int kChunkBytes = kBlockKV * 128;           // one 128-row x 128-byte box
constexpr int kThreads = 384;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum : int { kSiteLoad = 201, kSiteMmaQ = 202, kSiteMmaKV = 203, kSiteMmaP = 204, kSiteSoftmaxS = 205, kSiteEpilogueO = 206 };

template <int kHeadDim, int kQTiles>
struct Cfg {
  static constexpr int kChunks = kHeadDim / kChunkElems;          // 128-byte column blocks per row
  static constexpr int kTileBytes = kChunks * kChunkBytes;        // a 128-row Q, K or V tile
  static constexpr int kKvSlots = (kHeadDim == 256) ? 2 : 4;
  static constexpr int kQBytes = kQTiles * kTileBytes;
  static constexpr int kSmemBytes = kQBytes + kKvSlots * kTileBytes + 256 + 1024;
  static constexpr int kTmemS = 0;                                // S_t at columns [128 t, 128 t + 128)
  static constexpr int kTmemO = 128 * kQTiles;                    // O_t at kTmemO + t * kHeadDim
  static_assert(kTmemO + kQTiles * kHeadDim <= 512, "TMEM budget");
};

struct KernelArgs {
  int B, N, H, F, T;
  int causal;
  int is_bf16;
  float scale_log2;  // head_scale * log2(e)
  const uint16_t* bias;
  int64_t bias_strides[3];
  int bias_vec_ok;
  uint16_t* out;
  int64_t o_strides[3];
  int out_vec_ok;
  float* lse;
  int* status_word;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool bf16) {
  if (bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float unpack_lo(uint32_t w, bool bf16) {
  return bf16 ? __uint_as_float(w << 16) : __half2float(__ushort_as_half(static_cast<uint16_t>(w & 0xffffu)));
}
__device__ __forceinline__ float unpack_hi(uint32_t w, bool bf16) {
  return bf16 ? __uint_as_float(w & 0xffff0000u) : __half2float(__ushort_as_half(static_cast<uint16_t>(w >> 16)));
}

template <int kHeadDim, int kQTiles, int kPolyOf4>
__global__ void __launch_bounds__(kThreads, 1)
fmha_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const KernelArgs args) {
  using C = Cfg<kHeadDim, kQTiles>;
  constexpr int kSlots = C::kKvSlots;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + C::kQBytes;
  const uint32_t bar_base = kv_smem + kSlots * C::kTileBytes;
  // barriers: q_full, kv_full[kSlots], kv_empty[kSlots], s_full[2], p_ready[2], o_final[2]
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + kSlots + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 2 * kSlots + t); };
  auto p_ready = [&](int t) { return bar_base + 8u * (3 + 2 * kSlots + t); };
  auto o_final = [&](int t) { return bar_base + 8u * (5 + 2 * kSlots + t); };
  uint8_t* tail = smem_gen + C::kQBytes + kSlots * C::kTileBytes + 8 * (7 + 2 * kSlots);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ptx::AbortCtl ctl{abort_flag, args.status_word};

  // Heaviest query blocks (most visible keys under a causal mask) are scheduled first.
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int q0 = qb * (kBlockQ * kQTiles);
  const int kv_blocks_all = (args.T + kBlockKV - 1) / kBlockKV;
  int nblk[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < kQTiles; ++t) {
    const int row0 = q0 + t * kBlockQ;
    if (row0 < args.F) {
      int n = kv_blocks_all;
      if (args.causal) n = min(n, (row0 + kBlockQ - 1) / kBlockKV + 1);
      nblk[t] = n;
    }
  }
  const int nblk_max = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kSlots; ++s) {
      ptx::mbar_init(kv_full(s), 1);
      ptx::mbar_init(kv_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(s_full(t), 1);
      ptx::mbar_init(p_ready(t), 128);
      ptx::mbar_init(o_final(t), 1);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int valid_tiles = 0;
      for (int t = 0; t < kQTiles; ++t) valid_tiles += nblk[t] > 0 ? 1 : 0;
      ptx::mbar_expect_tx(q_full, valid_tiles * C::kTileBytes);
      for (int t = 0; t < kQTiles; ++t) {
        if (nblk[t] == 0) continue;
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          ptx::tma_load_4d(q_smem + t * C::kTileBytes + c * kChunkBytes, &tmap_q, q_full, c * kChunkElems,
                           q0 + t * kBlockQ, head, batch);
      }
      // load order: K_0, V_0, K_1, V_1, ...
      const int loads = 2 * nblk_max;
      for (int i = 0; i < loads; ++i) {
        const int slot = i % kSlots;
        const uint32_t use = i / kSlots;
        if (!ptx::mbar_wait(kv_empty(slot), (use & 1u) ^ 1u, ctl, kSiteLoad)) break;
        const int j = i >> 1;
        const CUtensorMap* map = (i & 1) ? &tmap_v : &tmap_k;
        ptx::mbar_expect_tx(kv_full(slot), C::kTileBytes);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c)
          ptx::tma_load_4d(kv_smem + slot * C::kTileBytes + c * kChunkBytes, map, kv_full(slot), c * kChunkElems,
                           j * kBlockKV, head, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk_max > 0) {
      const uint32_t fmt = args.is_bf16 ? 1u : 0u;
      // S = Q.K^T : M=128, N=128 keys, both operands K-major (head dim contiguous)
      const uint32_t idesc_s = ptx::umma_idesc(fmt, fmt, 0, 0, kBlockQ, kBlockKV);
      // O += P.V  : M=128, N=kHeadDim, A = P in TMEM, B = V with the head dim contiguous (MN-major)
      const uint32_t idesc_o = ptx::umma_idesc(fmt, fmt, 0, 1, kBlockQ, kHeadDim);
      auto issue_s = [&](int t, int slot) {
        const uint32_t qa = q_smem + t * C::kTileBytes;
        const uint32_t kb = kv_smem + slot * C::kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kChunkBytes + (ks & 3) * 32;
          ptx::umma_ss<false>(tmem_base + C::kTmemS + t * 128, ptx::umma_smem_desc(qa + off, 16, 1024),
                              ptx::umma_smem_desc(kb + off, 16, 1024), idesc_s, ks != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint32_t vb = kv_smem + slot * C::kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kBlockKV / 16; ++ks) {
          // 16 keys = 16 rows of 128 bytes; head-dim column blocks are kChunkBytes apart
          ptx::umma_ts_f16(tmem_base + C::kTmemO + t * kHeadDim, tmem_base + C::kTmemS + t * 128 + ks * 8,
                           ptx::umma_smem_desc(vb + ks * 2048, kChunkBytes, 1024), idesc_o,
                           (accumulate || ks != 0) ? 1u : 0u);
        }
      };
      bool alive = ptx::mbar_wait(q_full, 0, ctl, kSiteMmaQ);
      int load_idx = 0;  // index into the K_0, V_0, K_1, ... sequence
      if (alive) alive = ptx::mbar_wait(kv_full(0), 0, ctl, kSiteMmaKV);
      if (alive) {
        ptx::tc_fence_after_sync();
        for (int t = 0; t < kQTiles; ++t) {
          if (nblk[t] > 0) {
            issue_s(t, 0);
            ptx::umma_commit(s_full(t));
          }
        }
        ptx::umma_commit(kv_empty(0));
        load_idx = 1;
      }
      for (int j = 0; j < nblk_max && alive; ++j) {
        const int v_idx = load_idx;         // V_j
        const int k_idx = load_idx + 1;     // K_{j+1}
        const int v_slot = v_idx % kSlots;
        const int k_slot = k_idx % kSlots;
        const bool more = (j + 1) < nblk_max;
        if (!ptx::mbar_wait(kv_full(v_slot), (v_idx / kSlots) & 1u, ctl, kSiteMmaKV)) break;
        if (more && !ptx::mbar_wait(kv_full(k_slot), (k_idx / kSlots) & 1u, ctl, kSiteMmaKV)) break;
        for (int t = 0; t < kQTiles; ++t) {
          if (j >= nblk[t]) continue;
          if (!ptx::mbar_wait(p_ready(t), j & 1u, ctl, kSiteMmaP)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after_sync();
          issue_pv(t, v_slot, j > 0);
          if (j + 1 < nblk[t]) {
            issue_s(t, k_slot);
            ptx::umma_commit(s_full(t));
          } else {
            ptx::umma_commit(o_final(t));
          }
        }
        if (!alive) break;
        ptx::umma_commit(kv_empty(v_slot));
        if (more) ptx::umma_commit(kv_empty(k_slot));
        load_idx += 2;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = (warp - 4) >> 2;  // query tile of this warpgroup
    const int quarter = warp & 3;
    if (t < kQTiles && nblk[t] > 0) {
      const bool bf16 = args.is_bf16 != 0;
      const int row_in_tile = quarter * 32 + lane;
      const int f = q0 + t * kBlockQ + row_in_tile;
      const bool row_ok = f < args.F;
      const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t s_addr = tmem_base + lane_addr + C::kTmemS + t * 128;
      const uint32_t o_addr = tmem_base + lane_addr + C::kTmemO + t * kHeadDim;
      const uint16_t* bias_row = nullptr;
      if (args.bias != nullptr && row_ok)
        bias_row = args.bias + batch * args.bias_strides[0] + head * args.bias_strides[1] +
                   static_cast<int64_t>(f) * args.bias_strides[2];
      float m_run = -INFINITY;
      float l_run = 0.0f;
      bool alive = true;
      const int my_blocks = nblk[t];
      for (int j = 0; j < my_blocks; ++j) {
        if (!ptx::mbar_wait(s_full(t), j & 1u, ctl, kSiteSoftmaxS)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(s_addr + c * 32, r[c]);
        ptx::tmem_ld_wait();
        const int kv0 = j * kBlockKV;
        // Scores enter the exponential as x = r * mult - m.  Fast path: r is the raw Q.K^T and
        // mult = head_scale * log2(e) (> 0, so the row maximum can be taken on r).  With a bias
        // or a non-positive scale, r is first rewritten as the full log2-domain score and mult = 1.
        float mult = args.scale_log2;
        if (args.bias != nullptr || !(args.scale_log2 > 0.0f)) {
          mult = 1.0f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__uint_as_float(r[c][i]) * args.scale_log2);
          }
          if (bias_row != nullptr) {
            const uint16_t* bp = bias_row + kv0;
            const int count = min(kBlockKV, args.T - kv0);
            if (args.bias_vec_ok && count == kBlockKV) {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint4 w = __ldg(reinterpret_cast<const uint4*>(bp + c * 32) + g);
                  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int i = g * 8 + e * 2;
                    r[c][i] = __float_as_uint(fmaf(unpack_lo(ww[e], bf16), kLog2e, __uint_as_float(r[c][i])));
                    r[c][i + 1] = __float_as_uint(fmaf(unpack_hi(ww[e], bf16), kLog2e, __uint_as_float(r[c][i + 1])));
                  }
                }
              }
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const int col = c * 32 + i;
                  if (col < count) {
                    const uint32_t w = __ldg(bp + col);
                    r[c][i] = __float_as_uint(fmaf(unpack_lo(w, bf16), kLog2e, __uint_as_float(r[c][i])));
                  }
                }
              }
            }
          }
        }
        // masks: keys past T (tile padding) and, under causal, keys after the query
        const bool tail_block = kv0 + kBlockKV > args.T;
        const bool diag_block = args.causal && (kv0 + kBlockKV - 1 > q0 + t * kBlockQ);
        if (tail_block || diag_block) {
          int limit = args.T - kv0;                             // first masked column from the tail
          if (args.causal) limit = min(limit, f - kv0 + 1);     // columns > f - kv0 are masked
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= limit) r[c][i] = 0xff800000u;  // -inf
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = ptx::max3(mx0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
            mx1 = ptx::max3(mx1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
          }
        }
        const float mx = fmaxf(mx0, mx1) * mult;
        float alpha = 1.0f;
        if (mx - m_run > kRescaleThreshold) {  // also true on the first block (m_run = -inf)
          alpha = ptx::ex2_approx(m_run - mx);  // 0 on the first block
          m_run = mx;
        }
        // Rows that are entirely masked so far keep m_run = -inf; use 0 to avoid inf - inf.
        const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
        const uint64_t mult2 = ptx::f32x2(mult, mult);
        const uint64_t negm2 = ptx::f32x2(-m_use, -m_use);
        uint64_t sum_a = ptx::f32x2(0.0f, 0.0f), sum_b = ptx::f32x2(0.0f, 0.0f);
        // P (16-bit pairs) overwrites the first 64 columns of this tile's S: the 32 scores of
        // chunk c become 16 packed columns at [16 c, 16 c + 16), already read by this thread.
        // Of every four pairs, kPolyOf4 take their 2^x from the FMA pipe, the rest from the
        // special-function unit, so that neither pipe alone bounds the softmax.
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x2 = ptx::fma2(ptx::f32x2(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1])), mult2, negm2);
            float x0, x1, p0, p1;
            ptx::f32x2_split(x2, x0, x1);
            if (((i >> 1) & 3) < kPolyOf4) {
              ptx::ex2_poly2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f), p0, p1);
              sum_b = ptx::add2(sum_b, ptx::f32x2(p0, p1));
            } else {
              p0 = ptx::ex2_approx(x0);
              p1 = ptx::ex2_approx(x1);
              sum_a = ptx::add2(sum_a, ptx::f32x2(p0, p1));
            }
            pk[i >> 1] = pack2(p0, p1, bf16);
          }
          ptx::tmem_st_32x16(s_addr + c * 16, pk);
        }
        float s0, s1;
        ptx::f32x2_split(ptx::add2(sum_a, sum_b), s0, s1);
        l_run = l_run * alpha + (s0 + s1);
        // Rescale O when any row of the warp raised its maximum.  s_full(j) was committed after
        // P.V of block j-1, so O is quiescent here.
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < kHeadDim / 32; ++c) {
            uint32_t o[32];
            ptx::tmem_ld_32x32(o_addr + c * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            ptx::tmem_st_32x32(o_addr + c * 32, o);
          }
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(p_ready(t));
      }
      // ---- epilogue: O / l, one rounding, 16-byte stores
      if (alive && ptx::mbar_wait(o_final(t), 0, ctl, kSiteEpilogueO)) {
        ptx::tc_fence_after_sync();
        const float inv_l = 1.0f / l_run;
        uint16_t* orow = args.out + batch * args.o_strides[0] + head * args.o_strides[1] +
                         static_cast<int64_t>(f) * args.o_strides[2];
#pragma unroll 1
        for (int c = 0; c < kHeadDim / 32; ++c) {
          if (c * 32 >= args.H) break;  // padded head-dim columns
          uint32_t o[32];
          ptx::tmem_ld_32x32(o_addr + c * 32, o);
          ptx::tmem_ld_wait();
          if (row_ok) {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = pack2(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l, bf16);
            const int count = min(32, args.H - c * 32);
            if (args.out_vec_ok && count == 32) {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                reinterpret_cast<uint4*>(orow + c * 32)[g] = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                if (2 * i < count) orow[c * 32 + 2 * i] = static_cast<uint16_t>(w[i] & 0xffffu);
                if (2 * i + 1 < count) orow[c * 32 + 2 * i + 1] = static_cast<uint16_t>(w[i] >> 16);
              }
            }
          }
        }
        if (args.lse != nullptr && row_ok) {
          const int64_t idx = (static_cast<int64_t>(batch) * args.N + head) * args.F + f;
          args.lse[idx] = (m_run + log2f(l_run)) * kLn2;
        }
      }
    }
  }

  if (*abort_flag != 0) __nanosleep(2000000);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <int kHeadDim, int kQTiles, int kPolyOf4>
int launch_cfg(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  using C = Cfg<kHeadDim, kQTiles>;
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
    // Size-1 dimensions still need a legal stride; any 16-byte multiple will do.
    auto stride_bytes = [&](int64_t st, uint64_t fallback) -> uint64_t {
      return st > 0 ? static_cast<uint64_t>(st) * 2 : fallback;
    };
    const uint64_t row_pitch = stride_bytes(strides[2], static_cast<uint64_t>(p.H) * 2);
    s.strides_bytes[0] = row_pitch;
    s.strides_bytes[1] = stride_bytes(strides[1], row_pitch * rows);
    s.strides_bytes[2] = stride_bytes(strides[0], row_pitch * rows * p.N);
    s.box[0] = kChunkElems;
    s.box[1] = kBlockKV;
    s.box[2] = 1;
    s.box[3] = 1;
    return encode_tmap(out, base, s);
  };
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, p.q, p.q_strides, p.F)) != IXK_OK) return rc;
  if ((rc = make_map(&tk, p.k, p.k_strides, p.T)) != IXK_OK) return rc;
  if ((rc = make_map(&tv, p.v, p.v_strides, p.T)) != IXK_OK) return rc;

  KernelArgs a{};
  a.B = p.B;
  a.N = p.N;
  a.H = p.H;
  a.F = p.F;
  a.T = p.T;
  a.causal = p.causal ? 1 : 0;
  a.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
  a.scale_log2 = p.head_scale * kLog2e;
  a.bias = static_cast<const uint16_t*>(p.bias);
  a.out = static_cast<uint16_t*>(p.out);
  a.lse = p.lse;
  a.status_word = dev.status_word;
  bool bias_vec = p.bias != nullptr && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
  bool out_vec = (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
  for (int i = 0; i < 3; ++i) {
    a.bias_strides[i] = p.bias_strides[i];
    a.o_strides[i] = p.o_strides[i];
    bias_vec = bias_vec && (p.bias_strides[i] % 8 == 0);
    out_vec = out_vec && (p.o_strides[i] % 8 == 0);
  }
  a.bias_vec_ok = bias_vec ? 1 : 0;
  a.out_vec_ok = out_vec ? 1 : 0;

  auto* fn = &fmha_prefill_kernel<kHeadDim, kQTiles, kPolyOf4>;
  static thread_local int configured_device = -1;
  if (configured_device != dev.device) {
    IXK_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured_device = dev.device;
  }
  const int rows_per_cta = kBlockQ * kQTiles;
  dim3 grid((p.F + rows_per_cta - 1) / rows_per_cta, p.N, p.B);
  fn<<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, a);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

}  // namespace

int launch_prefill(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  if (p.N > 65535 || p.B > 65535) return fail(IXK_UNIMPLEMENTED, "num_heads and num_batches must be <= 65535");
  // Head-size buckets follow the reference's policy pick (fmha_forward.h:621-646): <=64, <=128, <=256.
  constexpr int kPoly = 2;  // pairs of every four whose 2^x runs on the FMA pipe
  if (p.H <= 64) return p.F > kBlockQ ? launch_cfg<64, 2, kPoly>(p, dev, stream) : launch_cfg<64, 1, kPoly>(p, dev, stream);
  if (p.H <= 128) {
    if (p.F <= kBlockQ) return launch_cfg<128, 1, kPoly>(p, dev, stream);
    // Tuning override for the main configuration: IXK_FMHA_POLY = 0..3.
    if (const char* env = std::getenv("IXK_FMHA_POLY")) {
      switch (std::atoi(env)) {
        case 0: return launch_cfg<128, 2, 0>(p, dev, stream);
        case 1: return launch_cfg<128, 2, 1>(p, dev, stream);
        case 3: return launch_cfg<128, 2, 3>(p, dev, stream);
        default: break;
      }
    }
    return launch_cfg<128, 2, kPoly>(p, dev, stream);
  }
  return launch_cfg<256, 1, kPoly>(p, dev, stream);
}

}  // namespace fmha
}  // namespace ixk
