/* ixk.h — C ABI of libixk.so: the B200 (sm_100a) kernel library that stands in
 * for the kernel layer of intel-extension-for-openxla's PJRT plugin.
 *
 * The reference isolates its kernels behind two seams:
 *   - sycl_onednn.so, entered through RunGemmCustomCall
 *     (xla/service/gpu/sycl_onednn.h:31-37, xla/service/gpu/sycl_onednn.cc:38-54), and
 *   - the XeTLA attention entry points fmha_forward_kernel_{bf16,fp16}
 *     (xla/service/gpu/xetla/sdp/sdp_forward.h:22-36).
 * Every function below replaces one of those, with plain pointers and sizes
 * only.  All buffers are caller-owned device memory; nothing is retained past
 * the call; kernels are enqueued on the caller's stream and never synchronised.
 * No call allocates device memory except ixk_comm_create (a set-up call).
 * The first call of any entry point on a device looks up and clears the device's status word
 * (a host-side query and a 4-byte memset on the default stream): make it outside stream capture.
 * No entry point except the *_workspace_bytes queries is valid without a
 * B200-class GPU: there is no CPU fallback.
 */
#ifndef IXK_H_
#define IXK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
/* Replaces absl::Status at the boundary (xetla_gpu_fused_mha_runner.cc:60,
 * :145, :217 return Unimplemented / Internal; the reference CHECK-aborts on
 * layout violations at :114-116 — this library returns a code instead). */
typedef enum ixk_status {
  IXK_OK = 0,
  IXK_INVALID_ARGUMENT = 1,   /* malformed descriptor, null pointer, misalignment */
  IXK_UNIMPLEMENTED = 2,      /* valid request outside what the kernels cover      */
  IXK_WORKSPACE_TOO_SMALL = 3,
  IXK_CUDA_ERROR = 4,         /* a CUDA runtime/driver call failed                 */
  IXK_NO_DEVICE = 5,          /* no sm_100 device is current                       */
  IXK_DEVICE_TIMEOUT = 6      /* a bounded device-side wait gave up (see ixk_device_status) */
} ixk_status;

const char* ixk_status_string(int status);
/* Text of the last failure on the calling thread ("" if none). */
const char* ixk_last_error(void);
/* Library version, "major.minor.patch". */
const char* ixk_version(void);

/* ------------------------------------------------------------------- types */
/* Element types the reference dispatches on (onednn_matmul_utils.cc:605-610,
 * xetla_gpu_fused_mha_runner.cc:209-217), plus the two fp8 kinds of the scaled GEMM. */
typedef enum ixk_dtype {
  IXK_BF16 = 0,
  IXK_F16 = 1,
  IXK_F32 = 2,
  IXK_F8E4M3 = 3, /* e4m3fn: no inf, max 448   */
  IXK_F8E5M2 = 4, /* e5m2: IEEE-like, max 57344 */
  IXK_S8 = 5,     /* GEMM operands of the (S8,S8,S32) triple */
  IXK_S32 = 6     /* its output */
} ixk_dtype;

/* MatrixLayout::Order as read from the "*_order" attributes
 * (onednn_matmul_utils.cc:543-551). */
typedef enum ixk_order { IXK_ROW_MAJOR = 0, IXK_COL_MAJOR = 1 } ixk_order;

/* SYCLGemm::GemmBackendEpilogue, same names and order
 * (onednn_matmul_utils.h:35-44). */
typedef enum ixk_epilogue {
  IXK_EPILOGUE_DEFAULT = 0,
  IXK_EPILOGUE_RELU = 1,
  IXK_EPILOGUE_GELU = 2,
  IXK_EPILOGUE_BIAS = 3,
  IXK_EPILOGUE_BIAS_RELU = 4,
  IXK_EPILOGUE_BIAS_GELU = 5,
  IXK_EPILOGUE_GELU_AUX = 6,     /* second result: ixk_gemm_aux only (the reference rejects it,
                                    onednn_matmul_utils.cc:321-322, :452-453) */
  IXK_EPILOGUE_BIAS_GELU_AUX = 7 /* as above */
} ixk_epilogue;

/* One operand of the GEMM custom call: the six "{lhs,rhs,output}_*" attributes
 * RunGemm reads from the FFI dictionary (onednn_matmul_utils.cc:543-590).
 * num_rows/num_cols are the LOGICAL matrix shape; order says which of the two
 * is contiguous; leading_dim_stride is the pitch, in elements, of the other. */
typedef struct ixk_matrix_layout {
  int32_t order;              /* ixk_order */
  int32_t dtype;              /* ixk_dtype */
  int64_t num_rows;
  int64_t num_cols;
  int64_t batch_stride;       /* elements between consecutive batch members   */
  int64_t leading_dim_stride; /* elements between consecutive rows (row-major) or columns (col-major) */
} ixk_matrix_layout;

/* The attribute dictionary of "__cublas$gemm" / "__cublas$lt$matmul"
 * (sycl_custom_call.cc:154-205, onednn_matmul_utils.cc:533-621). */
typedef struct ixk_gemm_desc {
  ixk_matrix_layout lhs;    /* A: [M, K] */
  ixk_matrix_layout rhs;    /* B: [K, N] */
  ixk_matrix_layout output; /* D (and C, which XLA aliases with D when beta != 0): [M, N] */
  int64_t batch_size;
  float alpha;              /* any finite value (the reference CHECKs alpha == 1,
                               onednn_matmul_utils.cc:438) */
  float beta;               /* D = act(alpha*A.B + bias + beta*C); any finite value (the reference's
                               XeTLA path only takes 0 or 1, onednn_matmul_utils.cc:262-270) */
  int32_t epilogue;         /* ixk_epilogue */
  int32_t reserved;         /* must be 0 */
} ixk_gemm_desc;

/* ---------------------------------------------------------------- GEMM call */
/* Replaces RunGemmCustomCall (sycl_onednn.cc:38-54) → RunGemm
 * (onednn_matmul_utils.cc:533-621) → hgemm_* kernels
 * (xetla/gemm/hgemm_impl.h:101-459) / dnnl::matmul (onednn_matmul_utils.cc:394-491).
 *
 *   D = act(alpha*A.B + bias[n] + beta*C)    fp32 accumulate, one rounding to D's type
 *
 * (the residual is summed before the activation, as oneDNN's append_sum followed
 * by the eltwise post-op does, onednn_matmul_utils.cc:434-449.)
 * act = identity | relu | gelu_tanh by `epilogue`.  bias is a length-N vector
 * of A's type, N being the column count AFTER a column-major output has been
 * rewritten as D^T = B^T.A^T (onednn_matmul_utils.cc:520-530, bias dims :363-365).
 * c may be NULL iff beta == 0; c may alias d.  bias must be non-NULL exactly for
 * the BIAS* epilogues.  Type triples (lhs, rhs, output), the list of RunGemm
 * (onednn_matmul_utils.cc:605-610): (BF16,BF16,BF16) (F16,F16,F16) (BF16,BF16,F32) (F16,F16,F32);
 * (F32,F32,F32), computed on the tensor cores in TF32 — operands cut to 10 mantissa bits,
 * products summed in fp32 — which is the reference's XLA_FP32_MATH_MODE=TF32 setting
 * (xla/service/onednn_util.h:53-70), there is no full-fp32 mode here; (S8,S8,S32), exact integer
 * arithmetic, DEFAULT epilogue with alpha = 1 and beta = 0 only.  Others → IXK_UNIMPLEMENTED.
 * Requirements (else IXK_INVALID_ARGUMENT / IXK_UNIMPLEMENTED): pointers 16-byte
 * aligned, leading_dim_stride * sizeof(element) a multiple of 16 for A and B.  bias has A's
 * type for 16-bit operands and the output's type otherwise.
 * workspace is optional scratch (the reference hands its scratch allocator down
 * this path, sycl_onednn.h:37).  ixk_gemm_workspace_bytes returns what a problem
 * can use: non-zero only for skinny problems (M <= 128, one batch, a long K),
 * which then run split along K with fp32 partials in the workspace and a reduce
 * pass that applies the epilogue.  With workspace == NULL or fewer bytes the
 * single-pass kernel runs; results agree within fp32 summation order. */
int ixk_gemm(const ixk_gemm_desc* desc, const void* a, const void* b,
             const void* c, const void* bias, void* d, void* workspace,
             size_t workspace_bytes, void* cuda_stream);
size_t ixk_gemm_workspace_bytes(const ixk_gemm_desc* desc);

/* The two epilogues with an auxiliary output (GELU_AUX, BIAS_GELU_AUX of
 * onednn_matmul_utils.h:42-43, which the reference declares but answers with "Unsupported
 * Activation mode", onednn_matmul_utils.cc:321-322):
 *   aux = alpha*A.B + bias[n] + beta*C      (what the activation is applied to, D's type)
 *   D   = gelu_tanh(aux)
 * aux has the output's order and shape with its own pitch aux_leading_dim_stride (elements),
 * batches dense.  Everything else as ixk_gemm (no split-K workspace: the pass is single). */
int ixk_gemm_aux(const ixk_gemm_desc* desc, const void* a, const void* b, const void* c,
                 const void* bias, void* d, void* aux, int64_t aux_leading_dim_stride,
                 void* cuda_stream);

/* Which buffer of the "__cublas$lt$matmul" custom call is which: the operand unpacking of
 * SyclLtMatmul (sycl_custom_call.cc:167-205) as a plain function, for an XLA FFI handler to
 * call (csrc/xla_ffi_shim.cc) and for tests without XLA.  Indices into the call's operand list /
 * result list; -1 = absent. */
typedef struct ixk_ffi_operands {
  int32_t lhs_arg, rhs_arg;
  int32_t c_arg;      /* 2 when beta != 0 (XLA aliases it with the D result) */
  int32_t bias_arg;   /* 2, or 3 behind C, for the BIAS* epilogues */
  int32_t d_result;   /* 1 when the epilogue has an auxiliary output, else 0 */
  int32_t aux_result; /* 0 for the *_AUX epilogues */
} ixk_ffi_operands;
int ixk_ffi_select_operands(int epilogue, float beta, int num_args, int num_results,
                            ixk_ffi_operands* out);

/* fp8 scaled GEMM.  No counterpart kernel exists in the reference (its RunGemm
 * has no fp8 case, onednn_matmul_utils.cc:605-610); the contract is the one of
 * the fp8 example (example/fp8/run.py:120-121): operands quantised per tensor,
 *   D = cast( (sum_k Aq.Bq in fp32) * inv_scale_a * inv_scale_b ) [+ bias, act, beta*C as above]
 * lhs.dtype / rhs.dtype ∈ {F8E4M3, F8E5M2}; output.dtype ∈ {BF16, F16, F32}.
 * inv_scale_a / inv_scale_b are HOST floats (1/scale used at quantisation).
 * bias, if any, has D's type. */
int ixk_gemm_fp8(const ixk_gemm_desc* desc, const void* a, const void* b,
                 const void* c, const void* bias, void* d, float inv_scale_a,
                 float inv_scale_b, void* workspace, size_t workspace_bytes,
                 void* cuda_stream);

/* Gate and up projections of a GeGLU MLP in one product (the reference's Gemma example runs them
 * as two dots, a GELU and a multiply that XLA fuses, example/gemma/keras_nlp.patch:53-63 for the
 * block): b is [K, 2 N'] with the gate weights in the first N' columns and the up weights in the
 * last; desc describes the [M, 2 N'] product (row-major, dense, 16-bit, DEFAULT epilogue, alpha 1,
 * beta 0, batch 1, M <= 128: decode); out [M, N'] receives
 *   round(gelu_tanh(gate)) * round(up)   rounded once more,
 * the bits of a gate GEMM with the GELU epilogue, an up GEMM and an elementwise product.  The
 * product itself (split along K where that helps) lives in the workspace, which must hold
 * ixk_gemm_geglu_workspace_bytes(desc) bytes.  Other shapes: IXK_UNIMPLEMENTED (use the calls above). */
int ixk_gemm_geglu(const ixk_gemm_desc* desc, const void* a, const void* b, void* out,
                   int64_t out_leading_dim_stride, void* workspace, size_t workspace_bytes,
                   void* cuda_stream);
size_t ixk_gemm_geglu_workspace_bytes(const ixk_gemm_desc* desc);

/* Three projections of one input (the QKV-fusion pass).  Replaces
 * XetlaQKVGemmKernel::run (xetla/gemm/gemm.h:111-171) → HGEMM_QKV_KERNEL /
 * HGEMM_QKV_BIAS_KERNEL (xetla/gemm/hgemm_impl.h:461-608):
 *   out_i = A . B_i (+ bias_i),  i = 0, 1, 2      fp32 accumulate, one rounding
 * A row-major [m,k] with pitch lda; b holds the three row-major [k,n] weight
 * slabs one behind the other (slab i at b + i*k*n, pitch ldb, as hgemm_impl.h:518);
 * bias NULL or three length-n vectors (bias + i*n, :596-602); out0/1/2 row-major
 * [m,n] with pitch ldc, anywhere in memory (evenly spaced outputs run as one launch).
 * dtype ∈ {BF16, F16} for every operand.  Same alignment rules as ixk_gemm. */
int ixk_gemm_qkv(int dtype, int64_t m, int64_t n, int64_t k, const void* a,
                 int64_t lda, const void* b, int64_t ldb, const void* bias,
                 void* out0, void* out1, void* out2, int64_t ldc,
                 void* cuda_stream);

/* --------------------------------------------------------------- attention */
/* Arguments of fmha_forward_kernel_{bf16,fp16} (sdp_forward.h:22-36) plus the
 * strides the runner derives them from (xetla_gpu_fused_mha_runner.cc:96-123).
 * Strides are in ELEMENTS; the innermost (head_size) stride is 1, as the
 * runner CHECKs (:114-116).  Logical shapes: q,o [B,N,F,H]; k,v [B,N,T,H];
 * bias [B,N,F,T] with stride 0 on B and/or N meaning broadcast (the reference
 * wants it materialised per head, fmha_forward.h:229-242); lse [B,N,F] fp32. */
typedef struct ixk_fmha_desc {
  int32_t dtype;        /* IXK_BF16 or IXK_F16: q, k, v, bias, out */
  int32_t causal;       /* keep t <= f, diagonal anchored top-left (fmha_utils.h:45-96) */
  int32_t num_batches;  /* B */
  int32_t num_heads;    /* N */
  int32_t head_size;    /* H  (<= 256, multiple of 8) */
  int32_t num_queries;  /* F */
  int32_t num_keys;     /* T */
  float head_scale;     /* multiplies Q.K^T before the bias is added (fmha_forward.h:256-282) */
  float dropout_prob;   /* must be 0 (xetla_gpu_fused_mha_runner.cc:56-62) */
  int32_t reserved;     /* must be 0 */
  int64_t q_strides[3]; /* B, N, F */
  int64_t k_strides[3]; /* B, N, T */
  int64_t v_strides[3]; /* B, N, T */
  int64_t o_strides[3]; /* B, N, F */
  int64_t bias_strides[3]; /* B, N, F (innermost T stride is 1); ignored if bias == NULL */
} ixk_fmha_desc;

/* Replaces fmha_forward_kernel_bf16 / _fp16 (sdp_forward.cc:34-84):
 *   O[b,n,f,:] = softmax_t( head_scale * Q[b,n,f,:].K[b,n,t,:] + bias[b,n,f,t] ) . V[b,n,t,:]
 * with the softmax statistics in fp32.  One stated deviation in the prefill path for BF16: the
 * probabilities handed to the P.V product are cut to bf16 by truncation, with the mean loss
 * (0.28 %) put back through the exponent and taken out of the row sum again, where the reference
 * rounds P to the storage type (fmha_forward.h:364-382); results agree within the 2e-2 the
 * parity tests allow, F16 and the decode path round to nearest.  lse (may be NULL) receives
 * m + ln(l) per row — the reference's "activation" output when is_training
 * (fmha_forward.h:433-450).  workspace must hold ixk_fmha_fwd_workspace_bytes(desc)
 * bytes (non-zero only for the split-key decode path, F <= 16). */
int ixk_fmha_fwd(const ixk_fmha_desc* desc, const void* q, const void* k,
                 const void* v, const void* bias, void* out, float* lse,
                 void* workspace, size_t workspace_bytes, void* cuda_stream);
size_t ixk_fmha_fwd_workspace_bytes(const ixk_fmha_desc* desc);

/* Attention forward for callers that can neither pass scratch memory nor allocate any.
 * No counterpart in the reference (its runner always receives scratch from XLA's buffer
 * assignment, xetla_gpu_fused_mha_runner.h:36-41); added for hosts where that is not so: a
 * custom-call handler bound without a scratch allocator, or a process whose framework has already
 * reserved HBM for its own pool so that a library-side cudaMalloc would fail or stall the device.
 *
 * Same arguments and results as ixk_fmha_fwd, minus the workspace: the split-key decode path
 * keeps its partial results in an array of IXK_STATIC_SCRATCH_BYTES that is part of the library's
 * device image (each GPU that loads libixk.so holds that much memory until the process exits).
 * The call allocates nothing and frees nothing.
 *   - A problem whose ixk_fmha_fwd_workspace_bytes(desc) exceeds IXK_STATIC_SCRATCH_BYTES is
 *     refused with IXK_WORKSPACE_TOO_SMALL and nothing is launched; use ixk_fmha_fwd then.
 *   - The first call on each device looks up the array's device address.  The call itself
 *     allocates nothing, but with CUDA's lazy module loading it can be the moment at which the
 *     runtime loads the part of the library image that holds the array, i.e. when the device
 *     memory behind it is actually reserved.  Make that first call at start-up, outside any stream
 *     capture; from the second call on, the free device memory does not change.
 *   - All calls on a device share the one array, which still holds the previous call's partials:
 *     the kernels overwrite every element they later read, so nothing needs clearing, but two
 *     calls that may overlap on the GPU (different streams, no ordering between them) race on it.
 *     Order them, or give the concurrent ones their own workspace through ixk_fmha_fwd. */
#define IXK_STATIC_SCRATCH_BYTES (4u << 20)
int ixk_fmha_fwd_static_scratch(const ixk_fmha_desc* desc, const void* q, const void* k,
                                const void* v, const void* bias, void* out, float* lse,
                                void* cuda_stream);

/* Attention backward.  Replaces fmha_backward_kernel_bf16 / _fp16
 * (xla/service/gpu/xetla/sdp/sdp_backward.h:21-33, .cc:34-76), which the runner reaches from
 * RunFusedMHABackward (xla/service/gpu/xetla_gpu_fused_mha_runner.cc:227-473).  With
 *   P  = exp( head_scale * Q.K^T + bias - lse )        (masked as in the forward when causal)
 *   D  = rowsum(dO * O),   dP = dO.V^T,   dS = P * (dP - D)
 * it returns dV = P^T.dO, dK = head_scale * dS^T.Q, dQ = head_scale * dS.K
 * (fmha_backward.h:182-222, :489-700, :836-850); P and dS are rounded to dtype as matmul
 * operands, all sums are fp32, each gradient is rounded once.  No bias gradient (the reference
 * has none).  `fwd` describes q, k, v, bias and the forward output `out` (o_strides) exactly as in
 * the forward call; grad_out, dq, dk, dv are [B,N,F|T,H] views with their own strides (elements,
 * innermost 1).  The reference's dp_sum and grad_query_accum scratch arguments are the workspace:
 * ixk_fmha_bwd_workspace_bytes(desc) bytes, 16-byte aligned.  q, k, v, out, grad_out: 16-byte
 * aligned with strides that are multiples of 8; dq, dk, dv likewise.  head_size <= 128 runs as one
 * fused tensor-core kernel between a prepare and a convert pass; 128 < head_size <= 256 (the
 * reference's 64x128x256 policy, fmha_policy.h:107-116) runs as a chain of batched tensor-core
 * GEMMs over a group of heads at a time, with the score-sized intermediates (12 bytes per
 * query-key pair of the group, at most about 192 MB unless one head alone needs more) in the
 * workspace: same formulas and roundings, more HBM traffic. */
typedef struct ixk_fmha_bwd_desc {
  ixk_fmha_desc fwd;
  int64_t do_strides[3]; /* B, N, F */
  int64_t dq_strides[3]; /* B, N, F */
  int64_t dk_strides[3]; /* B, N, T */
  int64_t dv_strides[3]; /* B, N, T */
} ixk_fmha_bwd_desc;
int ixk_fmha_bwd(const ixk_fmha_bwd_desc* desc, const void* q, const void* k, const void* v,
                 const void* out, const void* bias, const void* grad_out, const float* lse,
                 void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes,
                 void* cuda_stream);
size_t ixk_fmha_bwd_workspace_bytes(const ixk_fmha_bwd_desc* desc);

/* ------------------------------------------------- between the custom calls */
/* The memory-bound steps a decoder layer runs between the calls above.  The
 * reference has no custom call for them: XLA compiles them as loop fusions
 * (the layers are example/gptj/jax_gptj.py and example/gemma/keras_nlp.patch:53-63).
 * They are here so that a layer driven through this library is one pass over
 * HBM per step instead of a chain of framework kernels.  dtype ∈ {BF16, F16};
 * pointers 16-byte aligned; cols, rotary_dim and all strides multiples of 8
 * elements (else IXK_INVALID_ARGUMENT). */
typedef enum ixk_norm_kind { IXK_NORM_LAYER = 0, IXK_NORM_RMS = 1 } ixk_norm_kind;
/* y[r,:] = (x[r,:] - mean) * rsqrt(var + eps)   (LAYER; biased variance)
 * y[r,:] =  x[r,:] * rsqrt(mean(x^2) + eps)     (RMS)
 * statistics in fp32, no learned gain or shift; ldx/ldy row pitches in elements;
 * cols <= 8192 (else IXK_UNIMPLEMENTED).  x and y may be the same buffer. */
int ixk_row_norm(int dtype, int kind, int64_t rows, int64_t cols, const void* x,
                 int64_t ldx, void* y, int64_t ldy, float eps, void* cuda_stream);
/* The same with a learned gain: y = normalised * (gain_offset + gain[col]), gain [cols] of the
 * input type; gain_offset = 1 gives the (1 + w) scale of Gemma's RMSNorm, 0 the usual w. */
int ixk_row_norm_gain(int dtype, int kind, int64_t rows, int64_t cols, const void* x, int64_t ldx,
                      const void* gain, float gain_offset, void* y, int64_t ldy, float eps,
                      void* cuda_stream);
/* Rotary position embedding in place, GPT-J convention: elements (2i, 2i+1),
 * 2i < rotary_dim, of every head rotate by the angle whose cosine / sine is
 * cos_table / sin_table[position, i] (fp32 tables [seq_len, rotary_dim/2]).
 * x addresses token t, head h at x + t*token_stride + h*head_stride; token t
 * sits at position t % seq_len.  Giving heads = 2 * heads_local and x = the
 * fused [tokens, 3, heads_local, head_dim] projection rotates q and k at once. */
int ixk_rotary_interleaved(int dtype, void* x, int64_t tokens, int64_t seq_len,
                           int64_t heads, int64_t rotary_dim, int64_t token_stride,
                           int64_t head_stride, const float* cos_table,
                           const float* sin_table, void* cuda_stream);
/* The half-split convention (Gemma, Llama): element i < rotary_dim/2 pairs with element
 * i + rotary_dim/2, same tables; rotary_dim a multiple of 16. */
int ixk_rotary_half(int dtype, void* x, int64_t tokens, int64_t seq_len,
                           int64_t heads, int64_t rotary_dim, int64_t token_stride,
                           int64_t head_stride, const float* cos_table,
                           const float* sin_table, void* cuda_stream);
/* This step's keys and values into a KV cache, both tensors in one launch (the slice_update of
 * the reference's Gemma example, example/gemma/keras_nlp.patch:15-17, which XLA compiles as a
 * dynamic-update-slice): cache[b, position, n, :] = new[b, n, :].  Strides in elements (the
 * cache's token stride lets [B,T,N,H] and [B,N,T,H] caches both work); the same strides for K and
 * V.  k_new / v_new may be slices of a fused QKV projection. */
int ixk_kv_append(int dtype, int64_t batch, int64_t heads, int64_t head_dim, const void* k_new,
                  const void* v_new, int64_t new_batch_stride, int64_t new_head_stride,
                  void* k_cache, void* v_cache, int64_t cache_batch_stride,
                  int64_t cache_token_stride, int64_t cache_head_stride, int64_t position,
                  void* cuda_stream);
/* out = x + partial                      (bias NULL)
 * out = x + round(partial + bias[col])   (bias given; the inner sum is rounded
 * to dtype before the residual add).  All [rows, cols] dense; out may alias x
 * or partial. */
int ixk_residual_add(int dtype, int64_t rows, int64_t cols, const void* x,
                     const void* partial, const void* bias, void* out,
                     void* cuda_stream);

/* ------------------------------------------------------ all-reduce over NVLink */
/* The exchange step of a tensor-parallel layer: the partial sums of a row-parallel projection,
 * one per GPU, summed into every GPU.  Replaces sycl_allreduce (xla/service/gpu/ccl_ops.h:40-46,
 * ccl_ops.cc:604-789) and its kernel allreduce_dpcpp (ccl_ops.cc:98-246): ranks read each other's
 * buffers directly (NVLink peer loads and stores), 16-bit floats are combined in fp32
 * (ccl_ops.cc:674-676).  The reference's participants are threads of one process that meet on the
 * host; here a rank is a process (or a thread) per GPU and the ranks meet on the device, through
 * flags in each other's memory, so a call costs no host synchronisation and a captured step
 * replays as a CUDA graph.
 *
 * Set-up (the only calls of this library that allocate device memory): every rank creates a
 * communicator, which allocates `buffer_bytes` of exchange buffer (plus 8 KB of flags) on the
 * current device and returns an IPC handle; the host passes all handles to every rank (in rank
 * order) and each rank connects.  Ranks that share a process skip IPC and connect with the peers'
 * ixk_comm_base() pointers (peer access between the devices must be enabled by the host).
 * After connecting, and again before destroying, the host must make the ranks meet (any host
 * barrier): a peer may not touch a buffer that is not there yet, or any more.
 *
 * Use: a rank's contribution is whatever lies at byte offset `in_offset` of ITS OWN exchange buffer
 * (ixk_comm_buffer(); the producing kernel writes there directly) — the same offset and count on
 * every rank.  `out` is this rank's result.  If `out` is the contribution itself (in place), or
 * lies elsewhere inside the exchange buffer (again the same offset on every rank) and the message
 * is at least 1 MiB, each rank reduces one slice and writes it to all ranks (2 x the message over
 * NVLink); otherwise each rank reads all contributions in full (one exchange, for latency-bound
 * messages) and `out` must not overlap the contribution.  Ranks are combined in rank order, so every
 * rank ends up with the same bits.  Calls on one communicator must be issued in the same order on
 * every rank and must not overlap on the GPU.  A rank whose peers do not arrive within the wait
 * limit (about a second unless changed) gives up: the kernel returns, ixk_device_status reports
 * IXK_DEVICE_TIMEOUT with site 301 (before reading) or 302 (before leaving), and the communicator
 * must be destroyed. */
typedef struct ixk_comm ixk_comm;
#define IXK_COMM_HANDLE_BYTES 64
#define IXK_COMM_MAX_RANKS 8
/* ReductionKind of the reference call (ccl_ops.cc:656-779). */
typedef enum ixk_reduce_kind {
  IXK_REDUCE_SUM = 0, IXK_REDUCE_PRODUCT = 1, IXK_REDUCE_MIN = 2, IXK_REDUCE_MAX = 3
} ixk_reduce_kind;
int ixk_comm_create(int rank, int world, size_t buffer_bytes, ixk_comm** comm,
                    void* handle_out /* IXK_COMM_HANDLE_BYTES, may be NULL */);
int ixk_comm_connect_ipc(ixk_comm* comm, const void* handles /* world x IXK_COMM_HANDLE_BYTES */);
int ixk_comm_connect_pointers(ixk_comm* comm, void* const* peer_bases /* world x ixk_comm_base() */);
void* ixk_comm_base(ixk_comm* comm);
void* ixk_comm_buffer(ixk_comm* comm);
size_t ixk_comm_buffer_bytes(ixk_comm* comm);
int ixk_comm_set_wait_limit(ixk_comm* comm, long long cycles);
/* A promise by the caller that lets the one-shot form (ixk_all_reduce to a buffer outside the
 * exchange buffer, ixk_all_reduce_residual) leave without its second meeting with the peers: no two
 * CONSECUTIVE calls on this communicator (of any kind, on any rank: the ranks issue the same
 * sequence) use overlapping contribution ranges.  Then a rank can only rewrite a range after it
 * has passed the first meeting of the call in between, i.e. after every peer has finished reading
 * the range.  A decode step with two exchanges at two offsets satisfies this by construction.
 * Off by default; the two-shot and scattered forms always keep both meetings. */
int ixk_comm_set_alternating(ixk_comm* comm, int on);
int ixk_comm_destroy(ixk_comm* comm);
/* dtype in {BF16, F16, F32}; kind: ixk_reduce_kind; count in elements. */
int ixk_all_reduce(ixk_comm* comm, int dtype, int kind, size_t in_offset, void* out,
                   size_t count, void* cuda_stream);
/* All-reduce fused with the residual add that follows a row-parallel projection:
 *   out = x + round(round(sum over ranks) [+ bias[col]])      [rows, cols] dense
 * the same bits as ixk_all_reduce followed by ixk_residual_add.  out may alias x, but not the
 * contribution. */
int ixk_all_reduce_residual(ixk_comm* comm, int dtype, size_t in_offset, const void* x,
                            const void* bias, void* out, int64_t rows, int64_t cols,
                            void* cuda_stream);
/* The two halves of the two-shot all-reduce as calls of their own (sycl_reduce_scatter /
 * sycl_allgather, ccl_ops.h:49-68; kernels ccl_ops.cc:518-559, :268-294).  count_per_rank elements
 * must be a whole number of 16-byte vectors.
 * Reduce-scatter: every rank's contribution is world * count_per_rank elements at in_offset of its
 * exchange buffer; rank r receives the combination of slice r in `out` (any local buffer).
 * All-gather: rank r's piece `in` (any local buffer) lands at out_offset + r * piece of EVERY
 * rank's exchange buffer.  Ordering rules as for ixk_all_reduce. */
int ixk_reduce_scatter(ixk_comm* comm, int dtype, int kind, size_t in_offset, void* out,
                       size_t count_per_rank, void* cuda_stream);
int ixk_all_gather(ixk_comm* comm, int dtype, const void* in, size_t out_offset,
                   size_t count_per_rank, void* cuda_stream);
/* A row-parallel projection fused with the first half of its all-reduce, then the second half
 * fused with the residual add (the reference runs the projection, sycl_allreduce and the add as
 * three steps: sycl_custom_call.cc:154-221, ccl_ops.cc:604-789).
 * ixk_gemm_scatter computes D = alpha * A.B [+ beta * C] [+ bias] as ixk_gemm does (desc.output
 * describes the whole [M, N] result: row-major, dense, 16-bit, batch 1; `c`, when beta != 0, is a
 * local [M, N] matrix of that layout), but stores row block o of D (rows [o * M / world,
 * (o + 1) * M / world)) straight into rank o's exchange buffer: slot `rank` of the `world` slots
 * of M / world x N elements that start at slots_offset.  The stores cross NVLink while the
 * tensor cores work on the following tiles.  Shapes: M a multiple of 128 * world, N of 8, and a
 * problem of at least 74 tiles of 256 x 256 (else IXK_UNIMPLEMENTED: use ixk_gemm +
 * ixk_all_reduce).  No waiting on peers inside this call.
 * ixk_all_reduce_scattered then, on every rank: waits for all ranks' projections, adds up the
 * slots of the rows this rank owns (in rank order, fp32), applies
 *   out = x + round(round(sum) [+ bias[col]])          (x == NULL: out = round(sum))
 * and writes those rows to the result at out_offset of EVERY rank's exchange buffer; when the
 * call has completed there, each rank holds the whole [rows, cols] result: the bits of ixk_gemm +
 * ixk_all_reduce + ixk_residual_add.  x ([rows, cols] dense) and bias are local; slots and result
 * must not overlap.  Ordering rules and time-outs as for ixk_all_reduce; the next
 * ixk_gemm_scatter on the same slots may be issued right after it on the same stream.
 * The scattered stores arrive in the peers' slots without any handshake: from the moment a peer
 * may reach its ixk_gemm_scatter, nothing else on this rank may still use the slot range (the pair
 * of calls itself is safe back to back, because ixk_all_reduce_scattered returns only when every
 * rank has read its slots; a range that other calls used before needs the ranks to meet first). */
int ixk_gemm_scatter(ixk_comm* comm, const ixk_gemm_desc* desc, const void* a, const void* b,
                     const void* c, const void* bias, size_t slots_offset, void* cuda_stream);
int ixk_all_reduce_scattered(ixk_comm* comm, int dtype, size_t slots_offset, const void* x,
                             const void* bias, size_t out_offset, int64_t rows, int64_t cols,
                             void* cuda_stream);
/* [begin, end) in elements of the slice rank `rank` reduces in the two-shot scheme: whole 16-byte
 * vectors split evenly, the last rank takes the remainder (ccl_ops.cc:103-114).  Host arithmetic. */
int ixk_all_reduce_slice(int dtype, size_t count, int rank, int world, size_t* begin, size_t* end);

/* ------------------------------------------------------------ diagnostics */
/* Every device-side wait in the tensor-core kernels is bounded; a wait that
 * gives up records a code in a per-device status word and the kernel drains and
 * returns.  Reads and clears that word (synchronises the device).  0 = clean. */
int ixk_device_status(int* status_word);
/* Exercises that mechanism on purpose: launches one small CTA whose first warp waits, with a
 * budget of `limit_cycles` (at most 1e8, i.e. well under 0.1 s), for a barrier phase that nothing
 * completes, and whose second warp depends on the first.  The kernel returns by itself; afterwards
 * ixk_device_status reports IXK_DEVICE_TIMEOUT with site code 901 and clears the word, and the
 * device is as usable as before.  cycles_out_device (device memory, may be NULL) receives the
 * cycles the CTA spent.  No counterpart in the reference, whose kernels have no device-side waits. */
int ixk_selftest_bounded_wait(long long limit_cycles, long long* cycles_out_device, void* cuda_stream);
/* With IXK_NVTX=1 in the environment every entry point that launches work is wrapped in an NVTX
 * range of its own name (for timelines of the calling program); off by default. */
/* Number of kernels this library has launched from this process (all threads). */
uint64_t ixk_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* IXK_H_ */
