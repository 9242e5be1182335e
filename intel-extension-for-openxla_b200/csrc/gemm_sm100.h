// Interface between the GEMM entry points (validation, normalisation) and the
// tcgen05 kernel launcher.
#pragma once

#include "host_common.h"

namespace ixk {
namespace gemm {

enum : int { kActNone = 0, kActRelu = 1, kActGelu = 2 };
// tcgen05.mma kinds (the values of ptx::kKind*, restated for host-only code)
enum : int { kKindF16 = 0, kKindF8 = 1, kKindTf32 = 2, kKindI8 = 3 };
constexpr int kMaxScatter = 8;  // destinations of a scattered output (= the most ranks a communicator has)

// A GEMM after normalisation: D is row-major [M,N]; A is [M,K], B is [K,N], each with
// either dimension contiguous.
struct Problem {
  int64_t M = 0, N = 0, K = 0, batch = 1;
  bool fp8 = false;          // any operand type other than the 16-bit floats (no split-K path)
  int kind = 0;              // tcgen05.mma kind: kKindF16 / kKindF8 / kKindTf32 / kKindI8
  int ab_dtype = IXK_BF16;   // 16-bit operand type when kind == kKindF16
  uint32_t a_fmt = 0, b_fmt = 0;  // tcgen05 operand format codes
  bool a_mn_major = false;  // A stored with M contiguous (column-major A)
  bool b_mn_major = false;  // B stored with N contiguous (row-major B)
  const void* a = nullptr;
  const void* b = nullptr;
  int64_t lda = 0, ldb = 0, a_batch_stride = 0, b_batch_stride = 0;
  bool a_broadcast = false;        // every batch reads the same A (three projections of one input)
  int64_t bias_batch_stride = 0;   // elements between the bias vectors of consecutive batches
  const void* c = nullptr;
  const void* bias = nullptr;
  void* d = nullptr;
  void* aux = nullptr;             // pre-activation values (the *_AUX epilogues); D's type and shape
  int64_t ld_aux = 0, aux_batch_stride = 0;
  int64_t ldc = 0, ldd = 0, c_batch_stride = 0, d_batch_stride = 0;
  int out_dtype = IXK_BF16;
  int bias_dtype = IXK_BF16;
  int act = kActNone;
  float acc_scale = 1.0f;
  float beta = 0.0f;
  int force_block_n = 0;  // tuning override; 0 = heuristic
  // Scattered output (row-parallel projection feeding an all-reduce): row block o of D, rows
  // [o * M / scatter_world, (o + 1) * M / scatter_world), is stored dense ([M / world, N], pitch N)
  // at scatter_dest[o], which may be another GPU's memory.  0 = D goes to `d` as usual.
  int scatter_world = 0;
  void* scatter_dest[kMaxScatter] = {};
};

// Kernel parameter block (passed by value).
struct KernelArgs {
  int M, N, K, batch;
  int tiles_m, tiles_n;
  int a_mn_major, b_mn_major;
  uint32_t idesc;
  const void* bias;
  const void* c;
  void* d;
  int64_t ldd, ldc, d_batch_stride, c_batch_stride;
  int out_dtype, bias_dtype, act;
  float acc_scale, beta;
  int d_vec_ok, c_vec_ok, bias_vec_ok;
  int d_tma;  // 16-bit D with 16-byte-aligned rows: stored through shared memory + TMA
  int a_broadcast;
  int64_t bias_batch_stride;
  void* aux;
  int64_t ld_aux, aux_batch_stride;
  int aux_vec_ok;
  int scatter_rows;  // rows per destination of a scattered output; 0 = one destination
  int* status_word;
};

int pick_block_n(int64_t M, int64_t N, int64_t batch, int sm_count);
int launch(const Problem& p, const DeviceInfo& dev, cudaStream_t stream);

// Split-K for skinny problems (gemm_splitk.cu): number of K chunks for a problem (1 = do not
// split; depends on the shape only, so the workspace query needs no device), the fp32 scratch it
// takes, and the two-kernel launch (partial GEMMs as a batch, then reduce + epilogue).
int split_k_factor(int64_t M, int64_t N, int64_t K, int64_t batch, bool fp8);
size_t split_k_workspace_bytes(int64_t M, int64_t N, int splits);
// (geglu: the N columns are [gate | up]; the reduce writes gelu(gate) * up, N / 2 columns, to p.d / p.ldd;
// splits may be 1 then: one GEMM into the scratch + the GeGLU pass)
int launch_split_k(const Problem& p, int splits, void* workspace, const DeviceInfo& dev, cudaStream_t stream,
                   bool geglu = false);

}  // namespace gemm
}  // namespace ixk
