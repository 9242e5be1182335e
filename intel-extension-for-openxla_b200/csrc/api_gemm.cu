// GEMM entry points: the host logic of RunGemm (xla/service/gpu/onednn_matmul_utils.cc:533-621)
// — attribute dictionary → matrix descriptors → column-major-output rewrite → typed dispatch —
// restated over the C ABI, in front of the tcgen05 kernel.
#include <cmath>
#include <cstdlib>
#include <utility>

#include "gemm_sm100.h"

namespace ixk {
namespace {

// MatrixDescriptor of the reference (xla/service/gpu/matrix_descriptor.h:31-47): storage is
// always read as row-major [num_rows, num_cols] with pitch leading_dim_stride; `transpose`
// says the logical matrix is the transpose of that storage.
struct MatrixDesc {
  const void* data;
  bool transpose;
  int64_t num_rows, num_cols, batch_stride, leading_dim_stride;
  int64_t reduced_dim() const { return transpose ? num_rows : num_cols; }
};

// onednn_matmul_utils.cc:547-590: a column-major layout becomes a transposed descriptor
// whose stored shape has rows and columns exchanged.
MatrixDesc make_desc(const ixk_matrix_layout& l, const void* data) {
  const bool t = l.order == IXK_COL_MAJOR;
  return MatrixDesc{data, t, t ? l.num_cols : l.num_rows, t ? l.num_rows : l.num_cols,
                    l.batch_stride, l.leading_dim_stride};
}

// onednn_matmul_utils.cc:520-530: D^T = B^T . A^T when the output is column-major.
void make_blas_compatible(MatrixDesc& lhs, MatrixDesc& rhs, MatrixDesc& out) {
  if (out.transpose) {
    std::swap(lhs, rhs);
    lhs.transpose = !lhs.transpose;
    rhs.transpose = !rhs.transpose;
    out.transpose = !out.transpose;
  }
}

bool is_fp8(int t) { return t == IXK_F8E4M3 || t == IXK_F8E5M2; }
int elem_bytes(int t) { return (t == IXK_F32 || t == IXK_S32) ? 4 : ((is_fp8(t) || t == IXK_S8) ? 1 : 2); }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_layout(const ixk_matrix_layout& l, const char* name) {
  if (l.order != IXK_ROW_MAJOR && l.order != IXK_COL_MAJOR)
    return fail(IXK_INVALID_ARGUMENT, std::string(name) + "_order must be 0 (row-major) or 1 (column-major)");
  if (l.num_rows < 0 || l.num_cols < 0)
    return fail(IXK_INVALID_ARGUMENT, std::string(name) + " has a negative dimension");
  const int64_t contiguous = l.order == IXK_ROW_MAJOR ? l.num_cols : l.num_rows;
  if (l.leading_dim_stride < contiguous)
    return fail(IXK_INVALID_ARGUMENT, std::string(name) + "_leading_dim_stride is smaller than the contiguous dimension");
  return IXK_OK;
}

int run(const ixk_gemm_desc* desc, const void* a, const void* b, const void* c, const void* bias,
        void* d, bool fp8_call, float inv_scale_a, float inv_scale_b, void* workspace, size_t workspace_bytes,
        void* stream, void* aux = nullptr, int64_t aux_ld = 0, bool aux_call = false,
        ixk_comm* scatter_comm = nullptr, size_t slots_offset = 0, bool geglu = false, int64_t geglu_ld = 0) {
  clear_error();
  if (desc == nullptr) return fail(IXK_INVALID_ARGUMENT, "desc is NULL");
  if (desc->reserved != 0) return fail(IXK_INVALID_ARGUMENT, "desc.reserved must be 0");
  int rc;
  if ((rc = check_layout(desc->lhs, "lhs")) != IXK_OK) return rc;
  if ((rc = check_layout(desc->rhs, "rhs")) != IXK_OK) return rc;
  if ((rc = check_layout(desc->output, "output")) != IXK_OK) return rc;
  if (desc->batch_size < 1) return fail(IXK_INVALID_ARGUMENT, "batch_size must be >= 1");

  // Epilogue → (vector bias?, activation).  onednn_matmul_utils.cc:90-136, :434-455.
  bool wants_bias = false;
  int act = gemm::kActNone;
  switch (desc->epilogue) {
    case IXK_EPILOGUE_DEFAULT: break;
    case IXK_EPILOGUE_RELU: act = gemm::kActRelu; break;
    case IXK_EPILOGUE_GELU: act = gemm::kActGelu; break;
    case IXK_EPILOGUE_BIAS: wants_bias = true; break;
    case IXK_EPILOGUE_BIAS_RELU: wants_bias = true; act = gemm::kActRelu; break;
    case IXK_EPILOGUE_BIAS_GELU: wants_bias = true; act = gemm::kActGelu; break;
    case IXK_EPILOGUE_GELU_AUX:
    case IXK_EPILOGUE_BIAS_GELU_AUX:
      // The reference stops here ("Unsupported Activation mode", onednn_matmul_utils.cc:321-322,
      // :452-453).  The auxiliary output needs a second result buffer, which only ixk_gemm_aux takes.
      if (!aux_call)
        return fail(IXK_UNIMPLEMENTED, "Unsupported Activation mode: the *_AUX epilogues write a second result; call ixk_gemm_aux");
      wants_bias = desc->epilogue == IXK_EPILOGUE_BIAS_GELU_AUX;
      act = gemm::kActGelu;
      break;
    default: return fail(IXK_INVALID_ARGUMENT, "Unknown Epilogue.");
  }
  if (aux_call && desc->epilogue != IXK_EPILOGUE_GELU_AUX && desc->epilogue != IXK_EPILOGUE_BIAS_GELU_AUX)
    return fail(IXK_INVALID_ARGUMENT, "ixk_gemm_aux takes the GELU_AUX and BIAS_GELU_AUX epilogues only");
  if (wants_bias != (bias != nullptr))
    return fail(IXK_INVALID_ARGUMENT, "bias must be given exactly for the BIAS* epilogues");
  if (!std::isfinite(desc->alpha) || !std::isfinite(desc->beta))
    return fail(IXK_INVALID_ARGUMENT, "alpha and beta must be finite");
  const bool has_c = desc->beta != 0.0f;
  if (has_c && c == nullptr) return fail(IXK_INVALID_ARGUMENT, "beta != 0 needs the C operand");

  // Type triples of RunGemm's TYPED_GEMM list (onednn_matmul_utils.cc:605-610) that the
  // tensor-core kernel covers, plus the fp8 operand kinds of the scaled GEMM.
  const int ta = desc->lhs.dtype, tb = desc->rhs.dtype, tc = desc->output.dtype;
  gemm::Problem p;
  if (fp8_call) {
    if (!is_fp8(ta) || !is_fp8(tb))
      return fail(IXK_INVALID_ARGUMENT, "ixk_gemm_fp8 needs F8E4M3/F8E5M2 operands");
    if (tc != IXK_BF16 && tc != IXK_F16 && tc != IXK_F32)
      return fail(IXK_UNIMPLEMENTED, "fp8 GEMM output must be BF16, F16 or F32");
    p.fp8 = true;
    p.kind = gemm::kKindF8;
    p.a_fmt = ta == IXK_F8E4M3 ? 0u : 1u;
    p.b_fmt = tb == IXK_F8E4M3 ? 0u : 1u;
    p.acc_scale = inv_scale_a * inv_scale_b * desc->alpha;
    p.bias_dtype = tc;
  } else {
    const bool f16_pair = (ta == IXK_BF16 && tb == IXK_BF16 && (tc == IXK_BF16 || tc == IXK_F32)) ||
                          (ta == IXK_F16 && tb == IXK_F16 && (tc == IXK_F16 || tc == IXK_F32));
    const bool f32_triple = ta == IXK_F32 && tb == IXK_F32 && tc == IXK_F32;
    const bool s8_triple = ta == IXK_S8 && tb == IXK_S8 && tc == IXK_S32;
    if (!f16_pair && !f32_triple && !s8_triple) {
      if (is_fp8(ta) || is_fp8(tb)) return fail(IXK_INVALID_ARGUMENT, "fp8 operands go through ixk_gemm_fp8");
      return fail(IXK_UNIMPLEMENTED,
                  "Unexpected GEMM lhs/rhs/output types: the tensor-core path takes (BF16,BF16,BF16|F32), "
                  "(F16,F16,F16|F32), (F32,F32,F32) and (S8,S8,S32)");   // onednn_matmul_utils.cc:605-620
    }
    if (f16_pair) {
      p.fp8 = false;
      p.kind = gemm::kKindF16;
      p.ab_dtype = ta;
      p.a_fmt = p.b_fmt = (ta == IXK_BF16) ? 1u : 0u;
      p.bias_dtype = ta;
    } else if (f32_triple) {
      // TF32 on the tensor cores: the hardware reads the upper 19 bits of each fp32 operand
      p.fp8 = true;   // (not a 16-bit problem: no split-K)
      p.kind = gemm::kKindTf32;
      p.a_fmt = p.b_fmt = 2u;
      p.bias_dtype = IXK_F32;
    } else {
      if (desc->epilogue != IXK_EPILOGUE_DEFAULT || desc->alpha != 1.0f || desc->beta != 0.0f)
        return fail(IXK_UNIMPLEMENTED, "(S8,S8,S32) takes the DEFAULT epilogue with alpha = 1 and beta = 0 only");
      p.fp8 = true;
      p.kind = gemm::kKindI8;
      p.a_fmt = p.b_fmt = 1u;  // signed 8-bit
      p.bias_dtype = IXK_S32;
    }
    p.acc_scale = desc->alpha;  // the product is scaled in fp32 before bias and residual are added
  }

  MatrixDesc lhs = make_desc(desc->lhs, a);
  MatrixDesc rhs = make_desc(desc->rhs, b);
  MatrixDesc out = make_desc(desc->output, d);
  const bool swapped = out.transpose;
  make_blas_compatible(lhs, rhs, out);

  // After the rewrite: D is row-major [M,N]; the logical lhs is [M,K], the logical rhs [K,N].
  p.M = out.num_rows;
  p.N = out.num_cols;
  p.K = lhs.reduced_dim();
  const int64_t lhs_m = lhs.transpose ? lhs.num_cols : lhs.num_rows;
  const int64_t rhs_k = rhs.transpose ? rhs.num_cols : rhs.num_rows;
  const int64_t rhs_n = rhs.transpose ? rhs.num_rows : rhs.num_cols;
  if (lhs_m != p.M || rhs_n != p.N || rhs_k != p.K)
    return fail(IXK_INVALID_ARGUMENT, "lhs [M,K], rhs [K,N] and output [M,N] shapes do not agree");
  p.batch = desc->batch_size;
  if (p.M == 0 || p.N == 0) return IXK_OK;  // nothing to write; pointers may be NULL
  if (a == nullptr || b == nullptr || (d == nullptr && scatter_comm == nullptr))
    return fail(IXK_INVALID_ARGUMENT, "a, b and d must be non-NULL");
  if (p.K == 0) return fail(IXK_UNIMPLEMENTED, "K == 0 is not supported");
  if (p.M > INT32_MAX || p.N > INT32_MAX || p.K > INT32_MAX)
    return fail(IXK_UNIMPLEMENTED, "dimensions above 2^31-1 are not supported");

  // lhs stored [rows, cols] row-major: not transposed → K contiguous (K-major);
  // transposed → stored [K, M] → M contiguous (MN-major).
  p.a = lhs.data;
  p.a_mn_major = lhs.transpose;
  p.lda = lhs.leading_dim_stride;
  p.a_batch_stride = lhs.batch_stride;
  // rhs stored row-major [K, N] when not transposed → N contiguous (MN-major);
  // transposed → stored [N, K] → K-major.
  p.b = rhs.data;
  p.b_mn_major = !rhs.transpose;
  p.ldb = rhs.leading_dim_stride;
  p.b_batch_stride = rhs.batch_stride;
  p.d = d;
  p.ldd = out.leading_dim_stride;
  p.d_batch_stride = out.batch_stride;
  p.c = has_c ? c : nullptr;
  p.ldc = p.ldd;
  p.c_batch_stride = p.d_batch_stride;
  p.bias = bias;
  p.out_dtype = tc;
  p.act = act;
  p.beta = desc->beta;
  (void)swapped;
  if (aux_call) {
    // aux has the output's type, order and shape (after a column-major output has been rewritten
    // it is row-major [M,N] like D), its own pitch, and D's batch spacing rule: dense batches.
    if (aux == nullptr) return fail(IXK_INVALID_ARGUMENT, "aux is NULL");
    if (aux_ld < p.N) return fail(IXK_INVALID_ARGUMENT, "aux_leading_dim_stride is smaller than the contiguous dimension");
    if ((reinterpret_cast<uintptr_t>(aux) % elem_bytes(tc)) != 0) return fail(IXK_INVALID_ARGUMENT, "aux is not aligned to its element size");
    p.aux = aux;
    p.ld_aux = aux_ld;
    p.aux_batch_stride = aux_ld * p.M;
  }

  const int es = elem_bytes(ta);
  if (!aligned16(p.a) || !aligned16(p.b))
    return fail(IXK_INVALID_ARGUMENT, "a and b must be 16-byte aligned (TMA)");
  if ((p.lda * es) % 16 != 0 || (p.ldb * es) % 16 != 0)
    return fail(IXK_UNIMPLEMENTED, "leading_dim_stride * element size must be a multiple of 16 bytes for lhs and rhs (TMA)");
  if (p.batch > 1 && ((p.a_batch_stride * es) % 16 != 0 || (p.b_batch_stride * es) % 16 != 0))
    return fail(IXK_UNIMPLEMENTED, "batch_stride * element size must be a multiple of 16 bytes for lhs and rhs (TMA)");
  if ((reinterpret_cast<uintptr_t>(p.d) % elem_bytes(tc)) != 0)
    return fail(IXK_INVALID_ARGUMENT, "d is not aligned to its element size");
  if (scatter_comm != nullptr) {
    // D leaves in row blocks, one per rank, for the exchange buffers of the ranks that own them
    if (swapped || p.batch != 1 || p.ldd != p.N || elem_bytes(tc) != 2)
      return fail(IXK_UNIMPLEMENTED, "a scattered output is row-major, dense, un-batched and 16-bit");
    if ((rc = comm::scatter_targets(scatter_comm, slots_offset, p.M, static_cast<size_t>(p.N) * 2, p.scatter_dest,
                                    &p.scatter_world)) != IXK_OK)
      return rc;
    p.d = p.scatter_dest[0];
    DeviceInfo dev;
    if ((rc = get_device_info(&dev)) != IXK_OK) return rc;
    return gemm::launch(p, dev, static_cast<cudaStream_t>(stream));
  }

  if (geglu) {
    // [gate | up] halves of one product, combined by the pass that follows the GEMM
    if (swapped || p.kind != gemm::kKindF16 || p.batch != 1 || p.M > 128 || desc->epilogue != IXK_EPILOGUE_DEFAULT ||
        desc->beta != 0.0f || desc->alpha != 1.0f || elem_bytes(tc) != 2 || p.ldd != p.N || p.N % 16 != 0)
      return fail(IXK_UNIMPLEMENTED, "GeGLU projection: 16-bit row-major problem with M <= 128, DEFAULT epilogue, alpha 1, "
                                     "beta 0, a dense [M, 2 N'] product with N' a multiple of 8");
    if (geglu_ld < p.N / 2) return fail(IXK_INVALID_ARGUMENT, "out_leading_dim_stride is smaller than N'");
    DeviceInfo dev;
    if ((rc = get_device_info(&dev)) != IXK_OK) return rc;
    const int splits = gemm::split_k_factor(p.M, p.N, p.K, p.batch, p.fp8);
    const size_t need = static_cast<size_t>(splits) * p.M * p.N * sizeof(float);
    if (workspace == nullptr || !aligned16(workspace) || workspace_bytes < need)
      return fail(IXK_WORKSPACE_TOO_SMALL, "GeGLU projection: need " + std::to_string(need) + " bytes of 16-byte aligned scratch");
    p.ldd = geglu_ld;   // of the [M, N'] result; the product itself goes to the scratch
    return gemm::launch_split_k(p, splits, workspace, dev, static_cast<cudaStream_t>(stream), true);
  }

  if (const char* env = std::getenv("IXK_GEMM_BLOCK_N")) p.force_block_n = std::atoi(env);

  DeviceInfo dev;
  if ((rc = get_device_info(&dev)) != IXK_OK) return rc;
  // Skinny problems are cut along K when the caller handed over enough scratch for the partials;
  // without it they run un-split (same result, fewer SMs busy).
  const int splits = (p.force_block_n > 0 || p.aux != nullptr) ? 1 : gemm::split_k_factor(p.M, p.N, p.K, p.batch, p.fp8);
  if (splits > 1 && workspace != nullptr && aligned16(workspace) &&
      workspace_bytes >= gemm::split_k_workspace_bytes(p.M, p.N, splits))
    return gemm::launch_split_k(p, splits, workspace, dev, static_cast<cudaStream_t>(stream));
  return gemm::launch(p, dev, static_cast<cudaStream_t>(stream));
}

// Three projections of one input: out_i = A . B_i (+ bias_i), i = 0..2, with the three [K,N]
// weight slabs stacked behind one another (XetlaQKVGemmKernel, gemm.h:111-171; kernels
// hgemm_impl.h:461-608: grid dimension 0 picks slab `b + k*n*id`, output out0/1/2 and bias
// `bias + n*id`).  Runs as ONE launch with the projection as the batch index when the three outputs
// are evenly spaced, A being read through a batch-less tensor map; otherwise as three launches.
int run_qkv(int dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
            const void* bias, void* out0, void* out1, void* out2, int64_t ldc, void* stream) {
  clear_error();
  if (dtype != IXK_BF16 && dtype != IXK_F16)
    return fail(IXK_UNIMPLEMENTED, "QKV GEMM takes BF16 or F16 (gemm.cc instantiates sycl::half and bf16 only)");
  if (m < 0 || n < 0 || k < 0) return fail(IXK_INVALID_ARGUMENT, "negative dimension");
  if (m == 0 || n == 0) return IXK_OK;
  if (k == 0) return fail(IXK_UNIMPLEMENTED, "K == 0 is not supported");
  if (a == nullptr || b == nullptr || out0 == nullptr || out1 == nullptr || out2 == nullptr)
    return fail(IXK_INVALID_ARGUMENT, "a, b and the three outputs must be non-NULL");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return fail(IXK_UNIMPLEMENTED, "dimensions above 2^31-1 are not supported");
  if (lda < k || ldb < n || ldc < n) return fail(IXK_INVALID_ARGUMENT, "leading dimension smaller than the row length");
  if (!aligned16(a) || !aligned16(b)) return fail(IXK_INVALID_ARGUMENT, "a and b must be 16-byte aligned (TMA)");
  if ((lda * 2) % 16 != 0 || (ldb * 2) % 16 != 0 || (k * n * 2) % 16 != 0)
    return fail(IXK_UNIMPLEMENTED, "lda, ldb and the slab size times 2 bytes must be multiples of 16 bytes (TMA)");
  for (void* o : {out0, out1, out2})
    if ((reinterpret_cast<uintptr_t>(o) & 1u) != 0) return fail(IXK_INVALID_ARGUMENT, "output is not aligned to its element size");

  gemm::Problem p;
  p.M = m;
  p.N = n;
  p.K = k;
  p.ab_dtype = dtype;
  p.a_fmt = p.b_fmt = (dtype == IXK_BF16) ? 1u : 0u;
  p.bias_dtype = dtype;
  p.out_dtype = dtype;
  p.a = a;
  p.a_mn_major = false;  // A row-major [M,K] (the reference falls back otherwise, gemm.h:158)
  p.lda = lda;
  p.b_mn_major = true;   // slabs row-major [K,N]
  p.ldb = ldb;
  p.ldc = p.ldd = ldc;
  DeviceInfo dev;
  int rc;
  if ((rc = get_device_info(&dev)) != IXK_OK) return rc;
  const intptr_t step01 = static_cast<const char*>(out1) - static_cast<const char*>(out0);
  const intptr_t step12 = static_cast<const char*>(out2) - static_cast<const char*>(out1);
  if (step01 == step12 && step01 > 0 && step01 % 2 == 0 && step01 / 2 >= (m - 1) * ldc + n) {
    p.batch = 3;
    p.a_broadcast = true;
    p.b = b;
    p.b_batch_stride = k * n;
    p.bias = bias;
    p.bias_batch_stride = n;
    p.d = out0;
    p.d_batch_stride = step01 / 2;
    return gemm::launch(p, dev, static_cast<cudaStream_t>(stream));
  }
  void* outs[3] = {out0, out1, out2};
  for (int i = 0; i < 3; ++i) {
    p.batch = 1;
    p.b = static_cast<const uint16_t*>(b) + static_cast<int64_t>(i) * k * n;
    p.bias = bias ? static_cast<const uint16_t*>(bias) + static_cast<int64_t>(i) * n : nullptr;
    p.d = outs[i];
    if ((rc = gemm::launch(p, dev, static_cast<cudaStream_t>(stream))) != IXK_OK) return rc;
  }
  return IXK_OK;
}

// Shape of the problem after the column-major-output rewrite, for the workspace query.
size_t workspace_query(const ixk_gemm_desc* desc) {
  if (desc == nullptr) return 0;
  const bool swap = desc->output.order == IXK_COL_MAJOR;
  const int64_t M = swap ? desc->output.num_cols : desc->output.num_rows;
  const int64_t N = swap ? desc->output.num_rows : desc->output.num_cols;
  const int64_t K = desc->lhs.num_cols;
  const bool fp8 = is_fp8(desc->lhs.dtype);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return gemm::split_k_workspace_bytes(M, N, gemm::split_k_factor(M, N, K, desc->batch_size, fp8));
}

}  // namespace
}  // namespace ixk

extern "C" {

int ixk_gemm(const ixk_gemm_desc* desc, const void* a, const void* b, const void* c,
             const void* bias, void* d, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm");
  return ixk::run(desc, a, b, c, bias, d, /*fp8_call=*/false, 1.0f, 1.0f, workspace, workspace_bytes, cuda_stream);
}

size_t ixk_gemm_workspace_bytes(const ixk_gemm_desc* desc) { return ixk::workspace_query(desc); }

int ixk_gemm_aux(const ixk_gemm_desc* desc, const void* a, const void* b, const void* c, const void* bias, void* d,
                 void* aux, int64_t aux_leading_dim_stride, void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm_aux");
  return ixk::run(desc, a, b, c, bias, d, /*fp8_call=*/false, 1.0f, 1.0f, nullptr, 0, cuda_stream, aux,
                  aux_leading_dim_stride, /*aux_call=*/true);
}

// Which buffer of the "__cublas$lt$matmul" custom call is which (sycl_custom_call.cc:167-205):
// operands are lhs, rhs, [C when beta != 0], [bias when the epilogue adds one]; the result that
// receives D is index 1 when the epilogue has an auxiliary output (which is then result 0), else
// index 0.  XLA aliases operand 2 with the result when beta != 0, so C and D are one buffer there.
int ixk_ffi_select_operands(int epilogue, float beta, int num_args, int num_results, ixk_ffi_operands* out) {
  ixk::clear_error();
  if (out == nullptr) return ixk::fail(IXK_INVALID_ARGUMENT, "out is NULL");
  if (epilogue < IXK_EPILOGUE_DEFAULT || epilogue > IXK_EPILOGUE_BIAS_GELU_AUX)
    return ixk::fail(IXK_INVALID_ARGUMENT, "Unknown Epilogue.");   // onednn_matmul_utils.cc:90-110
  const bool has_bias = epilogue == IXK_EPILOGUE_BIAS || epilogue == IXK_EPILOGUE_BIAS_RELU ||
                        epilogue == IXK_EPILOGUE_BIAS_GELU || epilogue == IXK_EPILOGUE_BIAS_GELU_AUX;
  const bool has_aux = epilogue == IXK_EPILOGUE_GELU_AUX || epilogue == IXK_EPILOGUE_BIAS_GELU_AUX;
  const bool has_c = beta != 0.0f;
  out->lhs_arg = 0;
  out->rhs_arg = 1;
  out->c_arg = has_c ? 2 : -1;
  out->bias_arg = has_bias ? (has_c ? 3 : 2) : -1;
  out->d_result = has_aux ? 1 : 0;
  out->aux_result = has_aux ? 0 : -1;
  const int need_args = 2 + (has_c ? 1 : 0) + (has_bias ? 1 : 0);
  if (num_args < need_args)
    return ixk::fail(IXK_INVALID_ARGUMENT, "the custom call has " + std::to_string(num_args) + " operands, this epilogue and beta need " +
                                               std::to_string(need_args));
  if (num_results < out->d_result + 1)
    return ixk::fail(IXK_INVALID_ARGUMENT, "the custom call has too few results for this epilogue");
  return IXK_OK;
}

int ixk_gemm_scatter(ixk_comm* comm, const ixk_gemm_desc* desc, const void* a, const void* b, const void* c,
                     const void* bias, size_t slots_offset, void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm_scatter");
  if (comm == nullptr) {
    ixk::clear_error();
    return ixk::fail(IXK_INVALID_ARGUMENT, "comm is NULL");
  }
  return ixk::run(desc, a, b, c, bias, nullptr, false, 1.0f, 1.0f, nullptr, 0, cuda_stream, nullptr, 0, false, comm, slots_offset);
}

int ixk_gemm_geglu(const ixk_gemm_desc* desc, const void* a, const void* b, void* out, int64_t out_leading_dim_stride,
                   void* workspace, size_t workspace_bytes, void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm_geglu");
  return ixk::run(desc, a, b, nullptr, nullptr, out, false, 1.0f, 1.0f, workspace, workspace_bytes, cuda_stream, nullptr, 0, false,
                  nullptr, 0, /*geglu=*/true, out_leading_dim_stride);
}

size_t ixk_gemm_geglu_workspace_bytes(const ixk_gemm_desc* desc) {
  if (desc == nullptr) return 0;
  const int64_t M = desc->output.num_rows, N = desc->output.num_cols, K = desc->lhs.num_cols;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return static_cast<size_t>(ixk::gemm::split_k_factor(M, N, K, desc->batch_size, false)) * M * N * sizeof(float);
}

int ixk_gemm_fp8(const ixk_gemm_desc* desc, const void* a, const void* b, const void* c,
                 const void* bias, void* d, float inv_scale_a, float inv_scale_b, void* workspace,
                 size_t workspace_bytes, void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm_fp8");
  return ixk::run(desc, a, b, c, bias, d, /*fp8_call=*/true, inv_scale_a, inv_scale_b, workspace, workspace_bytes,
                  cuda_stream);
}

int ixk_gemm_qkv(int dtype, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, const void* b,
                 int64_t ldb, const void* bias, void* out0, void* out1, void* out2, int64_t ldc,
                 void* cuda_stream) {
  IXK_API_RANGE("ixk_gemm_qkv");
  return ixk::run_qkv(dtype, m, n, k, a, lda, b, ldb, bias, out0, out1, out2, ldc, cuda_stream);
}

}  // extern "C"
