// XLA FFI handlers that put libixk behind the custom-call targets the reference registers in
// xla/service/gpu/sycl_custom_call.cc:154-226 ("__cublas$gemm", "__cublas$lt$matmul"), on
// platform "CUDA".
//
// This translation unit needs XLA's FFI headers, which are not part of this repository: it
// compiles to nothing unless "xla/ffi/api/ffi.h" is on the include path (build.py compiles
// csrc/*.cu only; a maintainer adds this file to the plugin's own build).  The one piece of logic
// the handlers own — which operand is which — lives in libixk as ixk_ffi_select_operands and is
// tested there without XLA.
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define IXK_HAVE_XLA_FFI 1
#endif
#endif

#ifdef IXK_HAVE_XLA_FFI

#include <cstdint>
#include <string>

#include "ixk.h"
#include "xla/ffi/api/ffi.h"

namespace ixk_ffi {
namespace ffi = xla::ffi;

// PrimitiveType codes of xla_data.proto as they arrive in the "*_layout_dtype" attributes.
inline int ToIxkDtype(int32_t primitive_type) {
  switch (primitive_type) {
    case 16: return IXK_BF16;   // BF16
    case 10: return IXK_F16;    // F16
    case 11: return IXK_F32;    // F32
    case 2: return IXK_S8;      // S8
    case 4: return IXK_S32;     // S32
    case 20: return IXK_F8E4M3; // F8E4M3FN
    case 19: return IXK_F8E5M2; // F8E5M2
    default: return -1;
  }
}

// GemmBackendConfig_Epilogue (upstream backend_configs.proto) -> ixk_epilogue, the mapping of
// SYCLGemm::AsSYCLEpilogue (onednn_matmul_utils.cc:113-136).
inline int ToIxkEpilogue(int32_t e) {
  switch (e) {
    case 1: return IXK_EPILOGUE_DEFAULT;
    case 2: return IXK_EPILOGUE_RELU;
    case 4: return IXK_EPILOGUE_GELU;
    case 5: return IXK_EPILOGUE_GELU_AUX;
    case 6: return IXK_EPILOGUE_BIAS;
    case 7: return IXK_EPILOGUE_BIAS_RELU;
    case 8: return IXK_EPILOGUE_BIAS_GELU;
    case 9: return IXK_EPILOGUE_BIAS_GELU_AUX;
    default: return -1;
  }
}

inline ixk_matrix_layout Layout(const ffi::Dictionary& d, const char* prefix) {  // onednn_matmul_utils.cc:543-590
  auto key = [&](const char* s) { return std::string(prefix) + s; };
  ixk_matrix_layout l;
  l.order = *d.get<int32_t>(key("_order"));
  l.dtype = ToIxkDtype(*d.get<int32_t>(key("_layout_dtype")));
  l.num_rows = *d.get<int64_t>(key("_num_rows"));
  l.num_cols = *d.get<int64_t>(key("_num_cols"));
  l.batch_stride = *d.get<int64_t>(key("_batch_stride"));
  l.leading_dim_stride = *d.get<int64_t>(key("_leading_dim_stride"));
  return l;
}

inline ffi::Error ToError(int status) {
  if (status == IXK_OK) return ffi::Error::Success();
  // the two kinds the reference returns (xetla_gpu_fused_mha_runner.cc:60, :145)
  return ffi::Error(status == IXK_UNIMPLEMENTED ? ffi::ErrorCode::kUnimplemented : ffi::ErrorCode::kInternal,
                    ixk_last_error());
}

static ffi::Error LtMatmul(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::RemainingArgs args,
                           ffi::RemainingRets rets, ffi::Dictionary dict, bool plain_gemm) {
  ixk_gemm_desc desc{};
  desc.lhs = Layout(dict, "lhs");
  desc.rhs = Layout(dict, "rhs");
  desc.output = Layout(dict, "output");
  desc.batch_size = *dict.get<int64_t>("batch_size");
  desc.alpha = *dict.get<float>("alpha");
  desc.beta = *dict.get<float>("beta");
  desc.epilogue = plain_gemm ? IXK_EPILOGUE_DEFAULT : ToIxkEpilogue(*dict.get<int32_t>("epilogue"));
  ixk_ffi_operands sel;
  int st = ixk_ffi_select_operands(desc.epilogue, plain_gemm ? 0.0f : desc.beta, static_cast<int>(args.size()),
                                   static_cast<int>(rets.size()), &sel);
  if (st != IXK_OK) return ToError(st);
  auto arg = [&](int i) -> void* { return i < 0 ? nullptr : args.get<ffi::AnyBuffer>(i)->untyped_data(); };
  void* d = (*rets.get<ffi::AnyBuffer>(sel.d_result))->untyped_data();
  if (sel.aux_result >= 0) {
    void* aux = (*rets.get<ffi::AnyBuffer>(sel.aux_result))->untyped_data();
    st = ixk_gemm_aux(&desc, arg(sel.lhs_arg), arg(sel.rhs_arg), arg(sel.c_arg), arg(sel.bias_arg), d, aux,
                      desc.output.leading_dim_stride, stream);
    return ToError(st);
  }
  // Optional scratch: non-zero only for skinny (decode, M <= 128) problems, which then run split along K.
  size_t ws_bytes = ixk_gemm_workspace_bytes(&desc);
  void* ws = nullptr;
  if (ws_bytes != 0) {
    auto got = scratch.Allocate(ws_bytes);
    ws = got.has_value() ? *got : nullptr;
  }
  st = ixk_gemm(&desc, arg(sel.lhs_arg), arg(sel.rhs_arg), arg(sel.c_arg), arg(sel.bias_arg), d, ws, ws ? ws_bytes : 0,
                stream);
  return ToError(st);
}

static ffi::Error IxkGemm(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::RemainingArgs args,
                          ffi::RemainingRets rets, ffi::Dictionary dict) {
  return LtMatmul(stream, scratch, args, rets, dict, /*plain_gemm=*/true);   // sycl_custom_call.cc:154-165
}
static ffi::Error IxkLtMatmul(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::RemainingArgs args,
                              ffi::RemainingRets rets, ffi::Dictionary dict) {
  return LtMatmul(stream, scratch, args, rets, dict, /*plain_gemm=*/false);  // sycl_custom_call.cc:167-205
}

XLA_FFI_DEFINE_HANDLER(kIxkGemm, IxkGemm,
                       ffi::Ffi::Bind()
                           .Ctx<ffi::PlatformStream<cudaStream_t>>()
                           .Ctx<ffi::ScratchAllocator>()
                           .RemainingArgs()
                           .RemainingRets()
                           .Attrs());
XLA_FFI_DEFINE_HANDLER(kIxkLtMatmul, IxkLtMatmul,
                       ffi::Ffi::Bind()
                           .Ctx<ffi::PlatformStream<cudaStream_t>>()
                           .Ctx<ffi::ScratchAllocator>()
                           .RemainingArgs()
                           .RemainingRets()
                           .Attrs());
XLA_FFI_REGISTER_HANDLER(ffi::GetXlaFfiApi(), "__cublas$gemm", "CUDA", kIxkGemm);
XLA_FFI_REGISTER_HANDLER(ffi::GetXlaFfiApi(), "__cublas$lt$matmul", "CUDA", kIxkLtMatmul);

}  // namespace ixk_ffi

#endif  // IXK_HAVE_XLA_FFI
