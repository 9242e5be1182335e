// Flash-attention forward for sm_100a on tcgen05 / TMEM.
//
//   O = softmax(head_scale * Q.K^T + bias, masked) . V        one (batch, head, query block) per CTA
//
// Replaces FmhaForwardKernel (xla/service/gpu/xetla/sdp/fmha_forward.h:526-612).  Where the
// XeTLA kernel keeps Q in shared local memory, re-normalises P on every key block and reduces
// rows across sub-groups through shared memory, this one is built on the Blackwell units:
//
//   warps 0-3     softmax for query tile 0: one thread owns one row of S (a TMEM lane), so
//   warps 4-7     softmax for query tile 1  row max / row sum need no cross-thread traffic
//   warp 8        TMA producer: Q_0, K_0, Q_1, V_0, K_1, V_1 ... (K/V through a shared-memory ring)
//   warp 9        tcgen05.mma issuer (one thread, alternating between the tiles):
//                                      S_t = Q_t.K_j^T  (A, B from shared memory, S in TMEM)
//                                      O_t += P_t.V_j   (A = P from TMEM, B = V from shared memory)
//   warps 12-15   epilogue: O / row sum out of TMEM, one rounding, stores (both tiles); the softmax
//                 warps hand over 1 / row sum and go straight on to the next work item
// The two softmax warpgroups take 184 registers per thread (a whole row of S lives in registers),
// the control and epilogue warpgroups give their share up (setmaxnreg).
//
// CTAs are persistent: each walks a static list of (batch, head, query block) work items, heaviest
// first, and every barrier keeps counting across items, so the loads and the first S of the next
// item are issued while the current item's last softmax and its epilogue still run.
// A work item carries kQTiles tiles of 128 query rows; with two tiles the tensor core works on one
// tile's S / P.V while the other tile's softmax runs.  P is handed to the MMA issuer in four quarters
// so that P.V starts on the first 32 keys while the rest is still being exponentiated.  P overwrites
// S in place in TMEM as packed 16-bit pairs.  The running maximum is only raised when it moved by more than 2^8
// (exact: the same stale maximum scales P, the row sum and O), which keeps the O rescale off
// the common path.  exp is evaluated as exp2 with head_scale*log2(e) folded in.  bf16 P is cut
// out of the fp32 bit pattern by a byte permute (a rounding conversion shares the quarter-rate
// pipe with ex2); the mean truncation loss is compensated in the exponent and the row sum.
// O leaves through a swizzled staging box per tile and TMA stores: stores issued from registers
// (16 bytes per lane, a different line each) queue thousands of requests at every item boundary
// and hold up the barrier traffic of every other warp.  Q has a full/empty pair per tile, each
// K/V slot is handed back once per use behind the last tile's MMAs: a tcgen05.commit or a barrier
// round trip costs the single issuing thread 50-120 cycles during which the tensor core drains.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "fmha_sm100.h"
#include "ptx.cuh"

namespace ixk {
namespace fmha {

namespace {

constexpr int kBlockQ = 128;   // query rows per tile (= TMEM lanes)
constexpr int kBlockKV = 128;  // keys per block
constexpr int kChunkElems = 64;                       // 16-bit elements per 128-byte swizzle row
constexpr int kChunkBytes = kBlockKV * 128;           // one 128-row x 128-byte box
constexpr int kThreads = 512;  // warpgroups: softmax tile 0, softmax tile 1, {producer, MMA issuer, 2 idle}, epilogue
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kParts = 4;  // pieces in which a block of P is handed to the MMA issuer (1, 2 or 4)
constexpr int kEpilogueWarp = 12;  // first warp of the epilogue warpgroup
// per-thread register budgets after re-partitioning: 256 x 184 + 128 x 56 + 128 x 88 = 65536
constexpr int kSoftmaxRegs = 184;
constexpr int kControlRegs = 56;
constexpr int kEpilogueRegs = 88;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kTruncInflate = 1.0028179f;     // 1 + 2^-8 * (1 / (2 ln 2)): mean relative loss of bf16 truncation
constexpr float kTruncBiasLog2 = 0.0040597f;    // log2(kTruncInflate)
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum : int { kSiteLoad = 201, kSiteMmaQ = 202, kSiteMmaKV = 203, kSiteMmaP = 204, kSiteSoftmaxS = 205, kSiteEpilogueO = 206,
              kSiteLoadQ = 207, kSiteMmaO = 208, kSiteLoadBias = 209, kSiteSoftmaxBias = 210 };

constexpr int kBiasTileBytes = 2 * kChunkBytes;  // 128 query rows x 128 keys, 16-bit, as two swizzled boxes
constexpr int kBiasPrefetch = 8;  // 16-byte groups of a bias row (the first box) read before the scores arrive

template <int kHeadDim, int kQTiles, bool kBias>
struct Cfg {
  static constexpr int kChunks = kHeadDim / kChunkElems;          // 128-byte column blocks per row
  static constexpr int kTileBytes = kChunks * kChunkBytes;        // a 128-row Q, K or V tile
  // with a TMA-fed bias tile per query tile the K/V ring gives up one slot to make room
  static constexpr int kKvSlots = (kHeadDim == 256) ? 2 : (kBias ? 3 : 4);
  static constexpr int kQBytes = kQTiles * kTileBytes;
  static constexpr int kBiasBytes = kBias ? kQTiles * kBiasTileBytes : 0;
  // O leaves through shared memory and TMA stores, one 64-column box per query tile at a time
  // (no room is left for it beside the TMA-fed bias tiles: that variant stores from registers)
  static constexpr int kStageBytes = kBias ? 0 : kQTiles * kChunkBytes;
  static constexpr int kSmemBytes = kQBytes + kKvSlots * kTileBytes + kBiasBytes + kStageBytes + 320 + 2 * kBlockQ * 4 + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static constexpr int kTmemS = 0;                                // S_t at columns [128 t, 128 t + 128)
  static constexpr int kTmemO = 128 * kQTiles;                    // O_t at kTmemO + t * kHeadDim
  static_assert(kTmemO + kQTiles * kHeadDim <= 512, "TMEM budget");
};

struct KernelArgs {
  int B, N, H, F, T;
  int causal;
  int is_bf16;
  float scale_log2;  // head_scale * log2(e)
  float head_scale;
  const uint16_t* bias;
  int64_t bias_strides[3];
  int bias_vec_ok;
  uint16_t* out;
  int64_t o_strides[3];
  int out_vec_ok;
  int out_tma;  // O rows start on 16-byte boundaries: store through shared memory + TMA
  float* lse;
  int* status_word;
  int num_qblocks;  // query blocks of kBlockQ * kQTiles rows per (batch, head)
  int num_items;    // num_qblocks * N * B
  // 0 where K / V is one tensor broadcast over heads / batches (stride 0: multi-query attention),
  // 1 otherwise: multiplies the head / batch coordinate of the K and V loads
  int k_head_mul, k_batch_mul, v_head_mul, v_batch_mul;
  int use_schedule;  // the CTAs walk the host-made work list instead of the dealing formula
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

// One unit of work: a (batch, head, query block) triple and how many key blocks each of its
// query tiles visits.
struct Item {
  int q0, head, batch;
  int nblk0, nblk1;  // key blocks of query tile 0 / 1 (scalars: a runtime index would put an array in local memory)
  int nblk_max;
  int reversed;  // key blocks are walked from the diagonal down to block 0 (causal)
  __device__ __forceinline__ int nblk(int t) const { return t == 0 ? nblk0 : nblk1; }
  // The item takes nblk_max steps; tile t takes part in nblk(t) consecutive ones: the first
  // nblk(t) in forward order, the last nblk(t) in reversed order (every tile ends on block 0).
  __device__ __forceinline__ int first(int t) const { return reversed ? nblk_max - nblk(t) : 0; }
  __device__ __forceinline__ bool active(int t, int step) const {
    return step >= first(t) && step < first(t) + nblk(t);
  }
  __device__ __forceinline__ int key_block(int step) const { return reversed ? nblk_max - 1 - step : step; }
};

template <int kQTiles>
__device__ __forceinline__ Item get_item(const KernelArgs& args, int w) {
  // Causal: items are ordered heaviest first (the last query block sees the most keys), query
  // block by query block over all (batch, head) pairs, which the alternating deal below balances.
  // Non-causal: every item weighs the same, so the order is free and is chosen for L2: the query
  // blocks of one (batch, head) are neighbours, then the heads of one batch.  The CTAs of a round
  // then work on about a batch's worth of pairs at a time: K and V of a pair (and a bias slab
  // shared by the heads of a batch) come from HBM once and are found in L2 by the other query
  // blocks, instead of every pair's K and V being streamed again for every query block.
  const int pairs = args.N * args.B;
  Item it;
  int qb;
  if (args.causal) {
    const int rank = w / pairs;
    const int rest = w - rank * pairs;
    it.head = rest % args.N;
    it.batch = rest / args.N;
    qb = args.num_qblocks - 1 - rank;
  } else {
    const int pair = w / args.num_qblocks;
    qb = w - pair * args.num_qblocks;
    it.head = pair % args.N;
    it.batch = pair / args.N;
  }
  it.q0 = qb * (kBlockQ * kQTiles);
  const int kv_blocks_all = (args.T + kBlockKV - 1) / kBlockKV;
  it.nblk0 = it.nblk1 = 0;
#pragma unroll
  for (int t = 0; t < kQTiles; ++t) {
    const int row0 = it.q0 + t * kBlockQ;
    if (row0 < args.F) {
      int n = kv_blocks_all;
      if (args.causal) n = min(n, (row0 + kBlockQ - 1) / kBlockKV + 1);
      if (t == 0) it.nblk0 = n; else it.nblk1 = n;
    }
  }
  it.nblk_max = max(it.nblk0, it.nblk1);
  // Under a causal mask the second tile sees one key block more than the first.  Walking the
  // blocks backwards puts the step that only one tile takes part in at the START of the item,
  // where the other tile is still busy with the previous item's epilogue and its Q has not
  // arrived yet, instead of at the end, where it would leave half of the tensor core idle.
  // (With one tile per item nothing is gained, and the forward walk keeps the CTAs that share a
  // head on the same key blocks at the same time, which L2 rewards.)
  it.reversed = (args.causal && kQTiles == 2) ? 1 : 0;
  return it;
}

// A host-made work list: for every CTA the items it walks, in order.  Used for causal problems
// small enough for the table to travel as a kernel parameter (it lives in the parameter bank,
// nothing is allocated): the host deals the items so that the CTAs finish together AND so that the
// CTAs running at one time work on few (batch, head) pairs, whose K and V then stay in L2.
constexpr int kSchedMaxCtas = 148;
constexpr int kSchedMaxPerCta = 16;
struct Schedule {
  uint16_t count[kSchedMaxCtas];
  uint16_t item[kSchedMaxCtas * kSchedMaxPerCta];
};

// The i-th work item of a CTA.  With a work list: its i-th entry.  Otherwise items are dealt in
// rounds of gridDim.x, alternating direction (0..G-1, then G-1..0, ...), so that a CTA that drew a
// heavy item in one round draws a light one in the next: with items sorted by weight this keeps
// the per-CTA totals within a few percent.
__device__ __forceinline__ int item_of(const KernelArgs& args, const Schedule& sched, uint32_t round) {
  if (args.use_schedule)
    return round < sched.count[blockIdx.x] ? sched.item[blockIdx.x * kSchedMaxPerCta + round] : args.num_items;
  const int g = static_cast<int>(gridDim.x);
  const int c = static_cast<int>(blockIdx.x);
  return static_cast<int>(round) * g + ((round & 1u) ? (g - 1 - c) : c);
}

// tcgen05.mma with the shared-memory descriptors passed as (lo, hi) halves: the high half is a
// per-operand constant and the low half is a base plus a compile-time offset, which keeps the
// single issuing thread at a handful of instructions per MMA.
//
// The issuing warp runs its whole loop with all 32 lanes (uniform control flow) and elects one lane
// per instruction: the descriptor arithmetic then stays in the uniform datapath, and an MMA costs
// 10-20 issue cycles where the same code under `if (lane == 0)` takes about 50, which is most of
// the 64 cycles the MMA runs, so that the tensor core's queue never fills and every barrier round
// trip between two MMAs shows up as idle time.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
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
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                       uint32_t accumulate) {
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

template <int kHeadDim, int kQTiles, int kPolyOf4, bool kBias>
__global__ void __launch_bounds__(kThreads, 1)
fmha_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_bias,
                    const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ KernelArgs args,
                    const __grid_constant__ Schedule sched) {
  using C = Cfg<kHeadDim, kQTiles, kBias>;
  constexpr int kSlots = C::kKvSlots;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + C::kQBytes;
  const uint32_t bias_smem = kv_smem + kSlots * C::kTileBytes;  // kQTiles tiles when kBias
  const uint32_t stage_smem = bias_smem + C::kBiasBytes;        // kQTiles boxes of 128 rows x 128 bytes
  const uint32_t bar_base = stage_smem + C::kStageBytes;
  // barriers (8 bytes each)
  // Q has a full/empty pair per query tile: tile 0 issues its last S half a step before tile 1, and
  // the next item's first S then needs only 32 KB of Q instead of 64 KB to have arrived.
  auto q_full = [&](int t) { return bar_base + 8u * (t == 0 ? 0 : 22 + 2 * kSlots); };
  auto q_empty = [&](int t) { return bar_base + 8u * (t == 0 ? 1 : 23 + 2 * kSlots); };
  auto kv_full = [&](int s) { return bar_base + 8u * (2 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (2 + kSlots + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (2 + 2 * kSlots + t); };
  auto p_part = [&](int t, int quarter) { return bar_base + 8u * (4 + 2 * kSlots + t * 4 + quarter); };
  auto o_final = [&](int t) { return bar_base + 8u * (12 + 2 * kSlots + t); };
  auto o_free = [&](int t) { return bar_base + 8u * (14 + 2 * kSlots + t); };
  auto bias_full = [&](int t) { return bar_base + 8u * (16 + 2 * kSlots + t); };
  auto bias_empty = [&](int t) { return bar_base + 8u * (18 + 2 * kSlots + t); };
  auto stage_sync = [&](int t) { return bar_base + 8u * (20 + 2 * kSlots + t); };
  auto stats_full = [&](int t) { return bar_base + 8u * (24 + 2 * kSlots + t); };
  auto stats_empty = [&](int t) { return bar_base + 8u * (26 + 2 * kSlots + t); };
  uint8_t* tail = smem_gen + (bar_base - smem_base) + 8 * (28 + 2 * kSlots);
  static_assert(8 * (28 + 2 * kSlots) + 8 <= 320, "barrier area");
  // 1 / row sum of every query row, from the softmax warps to the epilogue warps
  float* inv_l_slot = reinterpret_cast<float*>(smem_gen + (bar_base - smem_base) + 320);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  ptx::AbortCtl ctl{abort_flag, args.status_word};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(q_full(t), 1);
      ptx::mbar_init(q_empty(t), 1);
    }
    for (int s = 0; s < kSlots; ++s) {
      ptx::mbar_init(kv_full(s), 1);
      ptx::mbar_init(kv_empty(s), 1);  // released once per use, behind the last tile's MMAs
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(s_full(t), 1);
      for (int quarter = 0; quarter < 4; ++quarter) ptx::mbar_init(p_part(t, quarter), 128);
      ptx::mbar_init(o_final(t), 1);
      ptx::mbar_init(o_free(t), 128);
      ptx::mbar_init(bias_full(t), 1);
      ptx::mbar_init(bias_empty(t), 128);
      ptx::mbar_init(stage_sync(t), 128);
      ptx::mbar_init(stats_full(t), 128);
      ptx::mbar_init(stats_empty(t), 128);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
    if (kBias) ptx::prefetch_tmap(&tmap_bias);
    if (C::kStageBytes > 0) ptx::prefetch_tmap(&tmap_o);
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    ptx::setmaxnreg_dec<kControlRegs>();
    if (lane == 0) {
      uint32_t load_idx = 0;  // position in the CTA-wide K_0, V_0, K_1, V_1, ... sequence
      [[maybe_unused]] uint32_t n_bias0 = 0, n_bias1 = 0;  // bias tiles loaded per query tile
      bool alive = true;
      uint32_t it = 0;
      for (int w = item_of(args, sched, 0); w < args.num_items && alive; w = item_of(args, sched, ++it)) {
        const Item item = get_item<kQTiles>(args, w);
        // Q of tile t, once the tile's last S of the previous item has been issued.  A tile with
        // no rows in this item still completes its phase, so that parities follow the item count.
        auto load_q = [&](int t) {
          if (!ptx::mbar_wait(q_empty(t), (it & 1u) ^ 1u, ctl, kSiteLoadQ)) {
            alive = false;
            return;
          }
          if (item.nblk(t) == 0) {
            ptx::mbar_arrive(q_full(t));
            return;
          }
          ptx::mbar_expect_tx(q_full(t), C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            ptx::tma_load_4d(q_smem + t * C::kTileBytes + c * kChunkBytes, &tmap_q, q_full(t), c * kChunkElems,
                             item.q0 + t * kBlockQ, item.head, item.batch);
        };
        // the tile that starts the item gets its Q first (tile 1 when the blocks run backwards)
        const int first_tile = (kQTiles == 2 && item.reversed) ? 1 : 0;
        load_q(first_tile);
        if (!alive) break;
        const int loads = 2 * item.nblk_max;
        for (int i = 0; i < loads; ++i, ++load_idx) {
          if (kQTiles == 2 && i == 1) {  // order: Q_0, K_0, Q_1, V_0, K_1, ...
            load_q(1 - first_tile);
            if (!alive) break;
          }
          const int slot = load_idx % kSlots;
          const uint32_t use = load_idx / kSlots;
          if (!ptx::mbar_wait(kv_empty(slot), (use & 1u) ^ 1u, ctl, kSiteLoad)) {
            alive = false;
            break;
          }
          const CUtensorMap* map = (i & 1) ? &tmap_v : &tmap_k;
          const int kv_head = item.head * ((i & 1) ? args.v_head_mul : args.k_head_mul);
          const int kv_batch = item.batch * ((i & 1) ? args.v_batch_mul : args.k_batch_mul);
          ptx::mbar_expect_tx(kv_full(slot), C::kTileBytes);
#pragma unroll
          for (int c = 0; c < C::kChunks; ++c)
            ptx::tma_load_4d(kv_smem + slot * C::kTileBytes + c * kChunkBytes, map, kv_full(slot), c * kChunkElems,
                             item.key_block(i >> 1) * kBlockKV, kv_head, kv_batch);
          if (kBias && (i & 1) == 0) {
            // right behind K_j: the bias tile of key block j for each query tile (one buffer per
            // tile, handed back by the softmax warpgroup as soon as it has read it)
            const int j = i >> 1;
            for (int t = 0; t < kQTiles && alive; ++t) {
              if (!item.active(t, j)) continue;
              if (!ptx::mbar_wait(bias_empty(t), ((t == 0 ? n_bias0 : n_bias1) & 1u) ^ 1u, ctl, kSiteLoadBias)) {
                alive = false;
                break;
              }
              if (t == 0) ++n_bias0; else ++n_bias1;
              ptx::mbar_expect_tx(bias_full(t), kBiasTileBytes);
#pragma unroll
              for (int c = 0; c < 2; ++c)
                ptx::tma_load_4d(bias_smem + t * kBiasTileBytes + c * kChunkBytes, &tmap_bias, bias_full(t),
                                 item.key_block(j) * kBlockKV + c * kChunkElems, item.q0 + t * kBlockQ,
                                 args.bias_strides[1] == 0 ? 0 : item.head, args.bias_strides[0] == 0 ? 0 : item.batch);
            }
            if (!alive) break;
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (all 32 lanes)
    ptx::setmaxnreg_dec<kControlRegs>();
    {
      const uint32_t fmt = args.is_bf16 ? 1u : 0u;
      // S = Q.K^T : M=128, N=128 keys, both operands K-major (head dim contiguous)
      const uint32_t idesc_s = ptx::umma_idesc(fmt, fmt, 0, 0, kBlockQ, kBlockKV);
      // O += P.V  : M=128, N=kHeadDim, A = P in TMEM, B = V with the head dim contiguous (MN-major)
      const uint32_t idesc_o = ptx::umma_idesc(fmt, fmt, 0, 1, kBlockQ, kHeadDim);
      // descriptor halves: K-major (Q, K): LBO 16 B (unused), SBO 1024 B; MN-major (V): LBO = one
      // 128-byte column block of the tile, SBO 1024 B
      const uint64_t kmajor = ptx::umma_smem_desc(0, 16, 1024);
      const uint64_t mnmajor = ptx::umma_smem_desc(0, kChunkBytes, 1024);
      const uint32_t k_lo = static_cast<uint32_t>(kmajor), k_hi = static_cast<uint32_t>(kmajor >> 32);
      const uint32_t v_lo = static_cast<uint32_t>(mnmajor), v_hi = static_cast<uint32_t>(mnmajor >> 32);
      auto issue_s = [&](int t, uint32_t slot) {
        const uint32_t qa = k_lo + ((q_smem + t * C::kTileBytes) >> 4);
        const uint32_t kb = k_lo + ((kv_smem + slot * C::kTileBytes) >> 4);
        const uint32_t d = tmem_base + C::kTmemS + t * 128;
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
          mma_ss(d, qa + off, k_hi, kb + off, k_hi, idesc_s, ks != 0 ? 1u : 0u);
        }
      };
      // quarter q covers keys [32 q, 32 q + 32) of the block = P columns [16 q, 16 q + 16)
      auto issue_pv = [&](int t, uint32_t slot, int quarter, bool accumulate) {
        const uint32_t vb = v_lo + ((kv_smem + slot * C::kTileBytes) >> 4);
        const uint32_t d = tmem_base + C::kTmemO + t * kHeadDim;
        const uint32_t a = tmem_base + C::kTmemS + t * 128;
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
          const int ks = quarter * 2 + k2;  // 16 keys = 16 rows of 128 bytes
          mma_ts(d, a + ks * 8, vb + ((ks * 2048) >> 4), v_hi, idesc_o, (accumulate || k2 != 0) ? 1u : 0u);
        }
      };
      // Q of a tile is released through tcgen05.commit when the tile's MMAs read it, by a plain
      // arrive when the tile had no work on it.
      auto release = [&](uint32_t bar, bool used) {
        if (used) {
          ptx::umma_commit_elect(bar);
        } else if (lane == 0) {
          ptx::mbar_arrive(bar);
        }
      };

      // Everything this thread does between two MMAs leaves the tensor core idle once its short
      // queue has drained, so the loop carries its state incrementally (ring slot and parity bits,
      // no divisions) and the per-tile code is instantiated with the tile as a constant.
      uint32_t slot = 0, slot_par = 0;  // ring slot of the next K/V tile to consume, parity of that use
      auto advance = [&]() {
        if (++slot == static_cast<uint32_t>(kSlots)) {
          slot = 0;
          slot_par ^= 1u;
        }
      };
      uint32_t p_par0 = 0, p_par1 = 0;    // parity of the next P block of each tile
      uint32_t of_par0 = 1, of_par1 = 1;  // parity on which o_free reports the previous item's O read out
      uint32_t q_par = 0;                 // parity of this item's q_full phases
      uint32_t it = 0;
      bool alive = true;
      auto wait = [&](uint32_t bar, uint32_t parity, int site) {
        if (!ptx::mbar_wait(bar, parity, ctl, site)) alive = false;
        return alive;
      };
      for (int w = item_of(args, sched, 0); w < args.num_items && alive; w = item_of(args, sched, ++it), q_par ^= 1u) {
        const Item item = get_item<kQTiles>(args, w);
        const int nblk_max = item.nblk_max;
        const int first0 = item.first(0), end0 = first0 + item.nblk0;
        const int first1 = item.first(1), end1 = first1 + item.nblk1;
        // One tile's share of step j: O_t += P_j.V_j, then S_t = Q_t.K_{j+1} for its next step.
        auto tile_turn = [&](auto tile_tag, int j, bool more, uint32_t v_slot, uint32_t k_slot, uint32_t k_par) {
          constexpr int t = decltype(tile_tag)::value;
          const int first = t == 0 ? first0 : first1;
          const int end = t == 0 ? end0 : end1;
          const bool active = j >= first && j < end;
          const bool next_s = j + 1 >= first && j + 1 < end;
          uint32_t& p_par = t == 0 ? p_par0 : p_par1;
          uint32_t& of_par = t == 0 ? of_par0 : of_par1;
          if (active) {
            // O_t of the previous item must have been read out before it is overwritten
            if (j == first && !wait(o_free(t), of_par, kSiteMmaO)) return;
            for (int part = 0; part < kParts; ++part) {
              if (!wait(p_part(t, part), p_par, kSiteMmaP)) return;
              ptx::tc_fence_after_sync();
#pragma unroll
              for (int q4 = 0; q4 < 4 / kParts; ++q4) {
                const int quarter = part * (4 / kParts) + q4;
                issue_pv(t, v_slot, quarter, j > first || quarter > 0);
              }
            }
            p_par ^= 1u;
          }
          if (next_s) {
            if (!active) {  // the tile joins at the next step: its Q is first needed here
              if (!wait(q_full(t), q_par, kSiteMmaQ)) return;
              ptx::tc_fence_after_sync();
            }
            if (kSlots == 2 && t == 0) {
              if (!wait(kv_full(k_slot), k_par, kSiteMmaKV)) return;
              ptx::tc_fence_after_sync();
            }
            issue_s(t, k_slot);
            ptx::umma_commit_elect(s_full(t));
          }
          // Both slots go back behind the last tile's MMAs (a commit covers everything this
          // thread has issued so far, the other tile's work included).
          if (t == kQTiles - 1) {
            ptx::umma_commit_elect(kv_empty(v_slot));
            if (more) ptx::umma_commit_elect(kv_empty(k_slot));
          }
          if (active && !next_s) {
            ptx::umma_commit_elect(o_final(t));
            of_par ^= 1u;
          }
          if (j == nblk_max - 2) release(q_empty(t), next_s);  // the item's last S has been issued
        };
        auto first_s = [&](auto tile_tag, uint32_t k_slot) {
          constexpr int t = decltype(tile_tag)::value;
          if ((t == 0 ? first0 : first1) == 0 && item.nblk(t) > 0) {  // a tile's Q is awaited where its first S is issued
            if (!wait(q_full(t), q_par, kSiteMmaQ)) return;
            ptx::tc_fence_after_sync();
            issue_s(t, k_slot);
            ptx::umma_commit_elect(s_full(t));
          }
          if (t == kQTiles - 1) ptx::umma_commit_elect(kv_empty(k_slot));
          if (nblk_max == 1) release(q_empty(t), item.nblk(t) > 0);
        };
        {
          if (!wait(kv_full(slot), slot_par, kSiteMmaKV)) break;
          ptx::tc_fence_after_sync();
          first_s(std::integral_constant<int, 0>{}, slot);
          if (kQTiles == 2 && alive) first_s(std::integral_constant<int, kQTiles - 1>{}, slot);
          advance();
        }
        for (int j = 0; j < nblk_max && alive; ++j) {
          const bool more = (j + 1) < nblk_max;
          // V_j and K_{j+1} are both needed in this step; asking for them here, where the issuer
          // would otherwise idle until P arrives, keeps the round trips off the MMA sequence.
          const uint32_t v_slot = slot;
          if (!wait(kv_full(v_slot), slot_par, kSiteMmaKV)) break;
          advance();
          const uint32_t k_slot = slot;  // K_{j+1}, present when `more`
          const uint32_t k_par = slot_par;
          if (more) {
            // (with a two-slot ring K_{j+1} was only requested when K_j's S had been issued: there
            // the wait stays behind P.V_j, where the load has had time to land)
            if (kSlots > 2 && !wait(kv_full(k_slot), k_par, kSiteMmaKV)) break;
            advance();
          }
          ptx::tc_fence_after_sync();
          tile_turn(std::integral_constant<int, 0>{}, j, more, v_slot, k_slot, k_par);
          if (kQTiles == 2 && alive) tile_turn(std::integral_constant<int, kQTiles - 1>{}, j, more, v_slot, k_slot, k_par);
        }
      }
    }
  } else if (warp >= kEpilogueWarp) {
    // ------------------------------------------------------------------ epilogue: O / l out of TMEM
    // Four warps (one per TMEM lane quarter) serve both query tiles.  The softmax warpgroups hand
    // over 1 / row sum and go on with the next item; O_t is read 32 columns at a time once the
    // tile's last P.V has landed, normalised, rounded once and stored.  With a staging box, rows
    // go to shared memory 128-byte-swizzled (thread = row, so each st.shared.v4 of a warp covers
    // every bank once per eight rows) and leave as one TMA store per 64 columns: from registers a
    // warp's 16-byte stores land in 32 different lines each, and that many requests hold up every
    // other warp's shared-memory and barrier traffic.
    ptx::setmaxnreg_dec<kEpilogueRegs>();
    const bool bf16 = args.is_bf16 != 0;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool elected = warp == kEpilogueWarp && lane == 0;  // issues every TMA store
    uint32_t n_fin0 = 0, n_fin1 = 0;    // items finished per tile
    uint32_t n_sync0 = 0, n_sync1 = 0;  // rendezvous of the four warps around a tile's staging box
    bool alive = true;
    uint32_t it = 0;
    for (int w = item_of(args, sched, 0); w < args.num_items && alive; w = item_of(args, sched, ++it)) {
      const Item item = get_item<kQTiles>(args, w);
      for (int tt = 0; tt < kQTiles && alive; ++tt) {
        const int t = item.reversed ? kQTiles - 1 - tt : tt;  // the tile that started first is served first
        if (item.nblk(t) == 0) continue;
        uint32_t& n_fin = t == 0 ? n_fin0 : n_fin1;
        uint32_t& n_sync = t == 0 ? n_sync0 : n_sync1;
        const uint32_t o_addr = tmem_base + lane_addr + C::kTmemO + t * kHeadDim;
        const int row0 = item.q0 + t * kBlockQ;
        const int f = row0 + row_in_tile;
        const bool row_ok = f < args.F;
        if (!ptx::mbar_wait(stats_full(t), n_fin & 1u, ctl, kSiteEpilogueO) ||
            !ptx::mbar_wait(o_final(t), n_fin & 1u, ctl, kSiteEpilogueO)) {
          alive = false;
          break;
        }
        ++n_fin;
        ptx::tc_fence_after_sync();
        const float inv_l = inv_l_slot[t * kBlockQ + row_in_tile];
        ptx::mbar_arrive(stats_empty(t));
        // 32 columns of this thread's row, normalised and packed to 16-bit pairs
        auto load_chunk = [&](int c, uint32_t (&wv)[16]) {
          uint32_t o[32];
          ptx::tmem_ld_32x32(o_addr + c * 32, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            wv[i] = pack2(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l, bf16);
        };
        constexpr int kOChunks = kHeadDim / 32;
        if (C::kStageBytes > 0 && args.out_tma) {
          const uint32_t stage = stage_smem + t * kChunkBytes;
          const uint32_t my_row = stage + row_in_tile * 128;
          auto rendezvous = [&]() {
            ptx::mbar_arrive(stage_sync(t));
            if (!ptx::mbar_wait(stage_sync(t), n_sync & 1u, ctl, kSiteEpilogueO)) alive = false;
            ++n_sync;
          };
#pragma unroll 1
          for (int pass = 0; pass < kHeadDim / 64 && alive; ++pass) {
            uint32_t lo[16], hi[16];
            load_chunk(2 * pass, lo);
            load_chunk(2 * pass + 1, hi);
            if (pass == kHeadDim / 64 - 1) {
              ptx::tc_fence_before_sync();
              ptx::mbar_arrive(o_free(t));  // O_t is in registers: the next item's P.V may overwrite it
            }
            // the box holds the previous 64 columns until their store has read them
            if (elected) ptx::bulk_wait_group_read<0>();
            rendezvous();
            if (!alive) break;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint32_t addr = my_row + static_cast<uint32_t>((g ^ (row_in_tile & 7)) << 4);
              const uint32_t* src = g < 4 ? &lo[4 * g] : &hi[4 * (g - 4)];
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(src[0]), "r"(src[1]), "r"(src[2]),
                           "r"(src[3])
                           : "memory");
            }
            ptx::fence_proxy_async_smem();
            rendezvous();
            if (!alive) break;
            if (elected && pass * 64 < args.H) {
              ptx::tma_store_4d(&tmap_o, stage, pass * 64, row0, item.head, item.batch);
              ptx::bulk_commit_group();
            }
          }
        } else {
          uint16_t* orow = args.out + item.batch * args.o_strides[0] + item.head * args.o_strides[1] +
                           static_cast<int64_t>(f) * args.o_strides[2];
#pragma unroll 1
          for (int c = 0; c < kOChunks; ++c) {
            uint32_t wv[16];
            load_chunk(c, wv);
            if (c == kOChunks - 1) {
              ptx::tc_fence_before_sync();
              ptx::mbar_arrive(o_free(t));
            }
            if (row_ok && c * 32 < args.H) {
              const int count = min(32, args.H - c * 32);
              if (args.out_vec_ok && count == 32) {
#pragma unroll
                for (int g = 0; g < 4; ++g)
                  reinterpret_cast<uint4*>(orow + c * 32)[g] =
                      make_uint4(wv[4 * g], wv[4 * g + 1], wv[4 * g + 2], wv[4 * g + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  if (2 * i < count) orow[c * 32 + 2 * i] = static_cast<uint16_t>(wv[i] & 0xffffu);
                  if (2 * i + 1 < count) orow[c * 32 + 2 * i + 1] = static_cast<uint16_t>(wv[i] >> 16);
                }
              }
            }
          }
        }
      }
    }
    // the staging boxes must outlive the TMA stores that read them
    if (C::kStageBytes > 0 && elected) ptx::bulk_wait_group<0>();
  } else if (warp > kMmaWarp) {
    ptx::setmaxnreg_dec<kControlRegs>();  // idle warps of the control warpgroup
  } else {
    // ------------------------------------------------------------------ softmax
    ptx::setmaxnreg_inc<kSoftmaxRegs>();
    const int t = warp >> 2;  // query tile of this warpgroup (warps 0-3: tile 0, warps 4-7: tile 1)
    const int quarter = warp & 3;
    if (t < kQTiles) {
      const bool bf16 = args.is_bf16 != 0;
      const int row_in_tile = quarter * 32 + lane;
      const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t s_addr = tmem_base + lane_addr + C::kTmemS + t * 128;
      const uint32_t o_addr = tmem_base + lane_addr + C::kTmemO + t * kHeadDim;
      uint32_t n_s = 0;  // S tiles consumed
      uint32_t n_o = 0;  // items finished
      [[maybe_unused]] uint32_t n_bias = 0;  // bias tiles consumed
      bool alive = true;
      uint32_t it = 0;
      for (int w = item_of(args, sched, 0); w < args.num_items && alive; w = item_of(args, sched, ++it)) {
        const Item item = get_item<kQTiles>(args, w);
        const int my_blocks = item.nblk(t);
        if (my_blocks == 0) continue;
        const int q0 = item.q0, head = item.head, batch = item.batch;
        const int f = q0 + t * kBlockQ + row_in_tile;
        const bool row_ok = f < args.F;
        const uint16_t* bias_row = nullptr;
        if (args.bias != nullptr && row_ok)
          bias_row = args.bias + batch * args.bias_strides[0] + head * args.bias_strides[1] +
                     static_cast<int64_t>(f) * args.bias_strides[2];
        float m_run = -INFINITY;
        float l_run = 0.0f;
        for (int j = 0; j < my_blocks; ++j) {
          // The bias tile of this block is in shared memory before the scores are ready: its first
          // box (keys 0-63) goes into registers while S is still on its way.
          [[maybe_unused]] uint4 bw[kBiasPrefetch];
          [[maybe_unused]] const uint8_t* bias_tile =
              smem_gen + (bias_smem - smem_base) + t * kBiasTileBytes + row_in_tile * 128;
          if constexpr (kBias) {
            if (!ptx::mbar_wait(bias_full(t), n_bias & 1u, ctl, kSiteSoftmaxBias)) {
              alive = false;
              break;
            }
            ++n_bias;
#pragma unroll
            for (int grp = 0; grp < kBiasPrefetch; ++grp)
              bw[grp] = *reinterpret_cast<const uint4*>(bias_tile + ((grp ^ (row_in_tile & 7)) << 4));
          }
          if (!ptx::mbar_wait(s_full(t), n_s & 1u, ctl, kSiteSoftmaxS)) {
            alive = false;
            break;
          }
          ++n_s;
          ptx::tc_fence_after_sync();
          uint32_t r[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(s_addr + c * 32, r[c]);
          ptx::tmem_ld_wait();
          const int kv0 = (item.reversed ? my_blocks - 1 - j : j) * kBlockKV;
          // Scores enter the exponential as x = r * mult - m.  Fast path: r is the raw Q.K^T and
          // mult = head_scale * log2(e) (> 0, so the row maximum can be taken on r).  With a
          // non-positive scale, r is first rewritten as the full log2-domain score and mult = 1.
          float mult = args.scale_log2;
          if (args.bias == nullptr && !(args.scale_log2 > 0.0f)) {
            mult = 1.0f;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
  #pragma unroll
              for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__uint_as_float(r[c][i]) * args.scale_log2);
            }
          }
          if (args.bias != nullptr) {
            // With a bias, r becomes the natural-log score head_scale * r + bias in one fused
            // multiply-add per element and mult = log2(e) (> 0 whatever the sign of the scale).
            mult = kLog2e;
            const float hs = args.head_scale;
            if (kBias) {
              // The bias tile was brought in by TMA as two 128-byte-swizzled boxes of 64 keys; this
              // thread reads its own row, 16 bytes at a time (8 consecutive rows touch 8 different
              // 16-byte columns, so the reads are bank-conflict free).
              const uint8_t* tile = bias_tile;
#pragma unroll
              for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const int grp = c * 4 + g;  // 16-byte group of 8 keys
                  const uint4 w = grp < kBiasPrefetch
                                      ? bw[grp < kBiasPrefetch ? grp : 0]
                                      : *reinterpret_cast<const uint4*>(tile + (grp >> 3) * kChunkBytes +
                                                                        (((grp & 7) ^ (row_in_tile & 7)) << 4));
                  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int i = g * 8 + e * 2;
                    r[c][i] = __float_as_uint(fmaf(__uint_as_float(r[c][i]), hs, unpack_lo(ww[e], bf16)));
                    r[c][i + 1] = __float_as_uint(fmaf(__uint_as_float(r[c][i + 1]), hs, unpack_hi(ww[e], bf16)));
                  }
                }
              }
              // The next tile is written by TMA, i.e. through the async proxy: this thread's reads
              // (generic proxy) have to be fenced against it, the barrier alone does not order them
              // (seen with an earlier hand-back: single rows picked up the next tile's values).
              ptx::fence_proxy_async_smem();
              ptx::mbar_arrive(bias_empty(t));
            } else if (bias_row != nullptr) {
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
                    const float bias_v = col < count ? unpack_lo(__ldg(bp + col), bf16) : 0.0f;
                    r[c][i] = __float_as_uint(fmaf(__uint_as_float(r[c][i]), hs, bias_v));
                  }
                }
              }
            } else {
  #pragma unroll
              for (int c = 0; c < 4; ++c) {
  #pragma unroll
                for (int i = 0; i < 32; ++i) r[c][i] = __float_as_uint(__uint_as_float(r[c][i]) * hs);
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
          // eight independent chains keep the row maximum off the latency-bound path
          float mxs[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 16) {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                mxs[e] = ptx::max3(mxs[e], __uint_as_float(r[c][i + 2 * e]), __uint_as_float(r[c][i + 2 * e + 1]));
            }
          }
          const float mx0 = fmaxf(ptx::max3(mxs[0], mxs[1], mxs[2]), mxs[3]);
          const float mx1 = fmaxf(ptx::max3(mxs[4], mxs[5], mxs[6]), mxs[7]);
          const float mx = fmaxf(mx0, mx1) * mult;
          float alpha = 1.0f;
          if (mx - m_run > kRescaleThreshold) {  // also true on the first block (m_run = -inf)
            alpha = ptx::ex2_approx(m_run - mx);  // 0 on the first block
            m_run = mx;
          }
          // Rows that are entirely masked so far keep m_run = -inf; use 0 to avoid inf - inf.
          // Rescale O when any row of the warp raised its maximum.  s_full was committed after
          // P.V of the previous block, so O is quiescent here; P.V of this block waits for p_lo.
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
          const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
          const uint64_t mult2 = ptx::f32x2(mult, mult);
          // bf16 P is made by truncating the fp32 bit pattern (one byte-permute per pair) instead of
          // a rounding conversion: conversions share the quarter-rate pipe with ex2, and at one per
          // pair they cost half as much again as the exponentials.  Truncation loses 0.28 % on
          // average (half an ulp over a log-uniform mantissa), so the exponent carries that much
          // extra (kTruncBias) and the row sum is deflated by the same factor in the epilogue.
          const bool trunc = bf16;
          const float bias_log2 = trunc ? kTruncBiasLog2 : 0.0f;
          const uint64_t negm2 = ptx::f32x2(bias_log2 - m_use, bias_log2 - m_use);
          uint64_t sum_a = ptx::f32x2(0.0f, 0.0f), sum_b = ptx::f32x2(0.0f, 0.0f);
          // P (16-bit pairs) overwrites the first 64 columns of this tile's S: the 32 scores of
          // chunk c become 16 packed columns at [16 c, 16 c + 16), already read by this thread.
          // Of every four pairs, kPolyOf4 take their 2^x from the FMA pipe, the rest from the
          // special-function unit, so that neither pipe alone bounds the softmax.
          auto exp_block = [&](auto trunc_tag) {
          constexpr bool kTrunc = decltype(trunc_tag)::value;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t x2 =
                  ptx::fma2(ptx::f32x2(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1])), mult2, negm2);
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
              pk[i >> 1] = kTrunc ? __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632) : pack2(p0, p1, false);
            }
            ptx::tmem_st_32x16(s_addr + c * 16, pk);
            if ((c + 1) % (4 / kParts) == 0) {
              // hand over this part of P
              ptx::tmem_st_wait();
              ptx::tc_fence_before_sync();
              ptx::mbar_arrive(p_part(t, c / (4 / kParts)));
            }
          }
          };
          if (trunc) {
            exp_block(std::true_type{});
          } else {
            exp_block(std::false_type{});
          }
          float s0, s1;
          ptx::f32x2_split(ptx::add2(sum_a, sum_b), s0, s1);
          l_run = l_run * alpha + (s0 + s1);
        }
        if (!alive) break;
        // ---- hand the row's normaliser to the epilogue warpgroup, which reads O out of TMEM once
        // the last P.V has landed; this warp goes straight on to the next item.
        if (!ptx::mbar_wait(stats_empty(t), (n_o & 1u) ^ 1u, ctl, kSiteEpilogueO)) {
          alive = false;
          break;
        }
        ++n_o;
        inv_l_slot[t * kBlockQ + row_in_tile] = (bf16 ? kTruncInflate : 1.0f) / l_run;  // the row sum carries the truncation bias
        ptx::mbar_arrive(stats_full(t));  // (release: the store above is visible to whoever sees the phase)
        if (args.lse != nullptr && row_ok) {
          const int64_t idx = (static_cast<int64_t>(batch) * args.N + head) * args.F + f;
          args.lse[idx] = (m_run + log2f(l_run) - (bf16 ? kTruncBiasLog2 : 0.0f)) * kLn2;
        }
      }
    }
  }

  if (*abort_flag != 0) __nanosleep(2000000);
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

// Work list for a causal launch.  Items are taken in an order made for L2 — the (batch, head)
// pairs in groups of 16, inside a group query block by query block from the heaviest down, so
// that a group's K and V are in use by many CTAs at once — and each goes to the CTA with the least
// work so far (cost = key blocks + 1.5 for the item's fixed part).  The two lightest query-block
// ranks of ALL pairs are held back to the end, where they fill the gaps the heavy items left:
// without them the finish times spread by up to a heavy item.  Returns false (formula dealing) for
// non-causal launches and for problems whose list does not fit the table.
template <int kQTiles>
bool build_schedule(const KernelArgs& a, int grid, Schedule* out) {
  if (!a.causal || grid > kSchedMaxCtas || a.num_items > 0xffff || a.num_items > grid * kSchedMaxPerCta) return false;
  const int pairs = a.N * a.B, nq = a.num_qblocks;
  if (nq < 3) return false;
  const int rows_per_item = kBlockQ * kQTiles;
  const int kv_blocks_all = (a.T + kBlockKV - 1) / kBlockKV;
  auto cost = [&](int qb) {   // in key-block steps, as get_item counts them (the later tile of the item sees the most keys)
    const int last_row0 = std::min(qb * rows_per_item + (kQTiles - 1) * kBlockQ, ((a.F - 1) / kBlockQ) * kBlockQ);
    const int n = std::min(kv_blocks_all, (last_row0 + kBlockQ - 1) / kBlockKV + 1);
    return 2 * n + 3;         // (doubled: 1.5 steps of fixed cost per item)
  };
  int load[kSchedMaxCtas];
  for (int c = 0; c < grid; ++c) {
    load[c] = 0;
    out->count[c] = 0;
  }
  bool ok = true;
  auto give = [&](int pair, int qb) {
    int best = 0;
    for (int c = 1; c < grid; ++c)
      if (load[c] < load[best]) best = c;
    if (out->count[best] >= kSchedMaxPerCta) {
      ok = false;
      return;
    }
    const int rank = nq - 1 - qb;   // the item numbering of get_item: rank-major, heaviest query block first
    out->item[best * kSchedMaxPerCta + out->count[best]++] = static_cast<uint16_t>(rank * pairs + pair);
    load[best] += cost(qb);
  };
  constexpr int kGroup = 16, kHeldBack = 2;
  for (int p0 = 0; p0 < pairs && ok; p0 += kGroup)
    for (int qb = nq - 1; qb >= kHeldBack && ok; --qb)
      for (int pr = p0; pr < std::min(pairs, p0 + kGroup) && ok; ++pr) give(pr, qb);
  for (int qb = kHeldBack - 1; qb >= 0 && ok; --qb)
    for (int pr = 0; pr < pairs && ok; ++pr) give(pr, qb);
  return ok;
}

template <int kHeadDim, int kQTiles, int kPolyOf4, bool kBias>
int launch_cfg(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  using C = Cfg<kHeadDim, kQTiles, kBias>;
  const CUtensorMapDataType dt = p.dtype == IXK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // A head / batch dimension with stride 0 (one K or V shared by all heads or batches) is encoded
  // with extent 1 and the kernel addresses it with coordinate 0; the host entry point has already
  // refused stride 0 wherever that is not a broadcast read (q, out, rows).
  auto make_map = [&](CUtensorMap* out, const void* base, const int64_t* strides, int rows) -> int {
    TmapSpec s{};
    s.dtype = dt;
    s.rank = 4;
    s.swizzle128 = true;
    s.dims[0] = p.H;
    s.dims[1] = rows;
    s.dims[2] = strides[1] == 0 ? 1 : p.N;
    s.dims[3] = strides[0] == 0 ? 1 : p.B;
    // Extent-1 dimensions still need a legal stride; any 16-byte multiple will do.
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
  CUtensorMap tq, tk, tv, tbias;
  int rc;
  if ((rc = make_map(&tq, p.q, p.q_strides, p.F)) != IXK_OK) return rc;
  if ((rc = make_map(&tk, p.k, p.k_strides, p.T)) != IXK_OK) return rc;
  if ((rc = make_map(&tv, p.v, p.v_strides, p.T)) != IXK_OK) return rc;
  CUtensorMap to = tq;  // placeholder unless O qualifies for TMA stores
  bool out_tma = C::kStageBytes > 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
  for (int i = 0; i < 3; ++i) out_tma = out_tma && p.o_strides[i] % 8 == 0;
  out_tma = out_tma && p.o_strides[2] >= p.H;
  if (out_tma && (rc = make_map(&to, p.out, p.o_strides, p.F)) != IXK_OK) return rc;
  tbias = tq;  // placeholder, never dereferenced unless kBias
  if (kBias) {
    // bias [B|1, N|1, F, T]: a broadcast dimension becomes extent 1 (coordinate always 0)
    TmapSpec s{};
    s.dtype = dt;
    s.rank = 4;
    s.swizzle128 = true;
    s.dims[0] = p.T;
    s.dims[1] = p.F;
    s.dims[2] = p.bias_strides[1] == 0 ? 1 : p.N;
    s.dims[3] = p.bias_strides[0] == 0 ? 1 : p.B;
    const uint64_t row_pitch = static_cast<uint64_t>(p.bias_strides[2]) * 2;
    s.strides_bytes[0] = row_pitch;
    s.strides_bytes[1] = p.bias_strides[1] == 0 ? row_pitch * p.F : static_cast<uint64_t>(p.bias_strides[1]) * 2;
    s.strides_bytes[2] = p.bias_strides[0] == 0 ? row_pitch * p.F * s.dims[2] : static_cast<uint64_t>(p.bias_strides[0]) * 2;
    s.box[0] = kChunkElems;
    s.box[1] = kBlockQ;
    s.box[2] = 1;
    s.box[3] = 1;
    if ((rc = encode_tmap(&tbias, p.bias, s)) != IXK_OK) return rc;
  }

  KernelArgs a{};
  a.B = p.B;
  a.N = p.N;
  a.H = p.H;
  a.F = p.F;
  a.T = p.T;
  a.causal = p.causal ? 1 : 0;
  a.is_bf16 = p.dtype == IXK_BF16 ? 1 : 0;
  a.scale_log2 = p.head_scale * kLog2e;
  a.head_scale = p.head_scale;
  a.bias = static_cast<const uint16_t*>(p.bias);
  a.out = static_cast<uint16_t*>(p.out);
  a.lse = p.lse;
  a.status_word = dev.status_word;
  a.k_head_mul = p.k_strides[1] == 0 ? 0 : 1;
  a.k_batch_mul = p.k_strides[0] == 0 ? 0 : 1;
  a.v_head_mul = p.v_strides[1] == 0 ? 0 : 1;
  a.v_batch_mul = p.v_strides[0] == 0 ? 0 : 1;
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
  a.out_tma = out_tma ? 1 : 0;

  auto* fn = &fmha_prefill_kernel<kHeadDim, kQTiles, kPolyOf4, kBias>;
  static thread_local int configured_device = -1;
  if (configured_device != dev.device) {
    IXK_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured_device = dev.device;
  }
  const int rows_per_item = kBlockQ * kQTiles;
  a.num_qblocks = (p.F + rows_per_item - 1) / rows_per_item;
  const int64_t items = static_cast<int64_t>(a.num_qblocks) * p.N * p.B;
  if (items > 0x7fffffff) return fail(IXK_UNIMPLEMENTED, "too many (batch, head, query block) work items");
  a.num_items = static_cast<int>(items);
  int grid = a.num_items < dev.sm_count ? a.num_items : dev.sm_count;
  // (5 KB: kept off the stack.  The list depends on the shape only, so a thread that launches the
  // same problem again, as a layer or a benchmark loop does, reuses the one it has.)
  static thread_local Schedule sched;
  static thread_local int sched_key[6] = {-1, -1, -1, -1, -1, -1};
  static thread_local bool sched_ok = false;
  const int key[6] = {a.B, a.N, a.F, a.T, a.causal, grid};
  if (!std::equal(key, key + 6, sched_key)) {
    sched_ok = build_schedule<kQTiles>(a, grid, &sched);
    std::copy(key, key + 6, sched_key);
  }
  a.use_schedule = sched_ok ? 1 : 0;
  fn<<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tbias, to, a, sched);
  IXK_CUDA_OK(cudaGetLastError());
  count_launch();
  return IXK_OK;
}

}  // namespace

// A bias whose rows start on 16-byte boundaries can be fetched by TMA; any other goes through
// per-thread global loads in the softmax warps.
bool bias_fits_tma(const Problem& p) {
  if (p.bias == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(p.bias) & 15u) != 0) return false;
  if (p.bias_strides[2] % 8 != 0 || p.bias_strides[2] < p.T) return false;
  return p.bias_strides[1] % 8 == 0 && p.bias_strides[0] % 8 == 0;
}

template <int kHeadDim, int kQTiles, int kPolyOf4>
int launch_bias(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  if (bias_fits_tma(p)) return launch_cfg<kHeadDim, kQTiles, kPolyOf4, true>(p, dev, stream);
  return launch_cfg<kHeadDim, kQTiles, kPolyOf4, false>(p, dev, stream);
}

int launch_prefill(const Problem& p, const DeviceInfo& dev, cudaStream_t stream) {
  // Head-size buckets follow the reference's policy pick (fmha_forward.h:621-646): <=64, <=128, <=256.
  constexpr int kPoly = 0;  // pairs of every four whose 2^x runs on the FMA pipe instead of the special-function unit
  if (p.H <= 64) return p.F > kBlockQ ? launch_bias<64, 2, kPoly>(p, dev, stream) : launch_bias<64, 1, kPoly>(p, dev, stream);
  if (p.H <= 128) {
    if (p.F <= kBlockQ) return launch_bias<128, 1, kPoly>(p, dev, stream);
    // Tuning override for the main configuration: IXK_FMHA_POLY = 0..2.
    if (const char* env = std::getenv("IXK_FMHA_POLY")) {
      switch (std::atoi(env)) {
        case 1: return launch_cfg<128, 2, 1, false>(p, dev, stream);
        case 2: return launch_cfg<128, 2, 2, false>(p, dev, stream);
        default: break;
      }
    }
    return launch_bias<128, 2, kPoly>(p, dev, stream);
  }
  return launch_bias<256, 1, kPoly>(p, dev, stream);
}

}  // namespace fmha
}  // namespace ixk

