"""Host-side mirror of the reference's kernel-layer interface, over libixk.so's C ABI.

The reference reaches its kernels through
  * RunGemmCustomCall(lhs, rhs, add, output, bias, stream, dict, epilogue, scratch)
    (xla/service/gpu/sycl_onednn.h:31-37), fed by the "__cublas$gemm" / "__cublas$lt$matmul"
    FFI handlers (xla/service/gpu/sycl_custom_call.cc:154-226), and
  * fmha_forward_kernel_{bf16,fp16}(queue, q, k, v, bias, dropout, dropout_prob, out, activation,
    B, N, H, F, T, head_scale, is_training) (xla/service/gpu/xetla/sdp/sdp_forward.h:22-36), called by
    RunXetlaGpuFMHA (xla/service/gpu/xetla_gpu_fused_mha_runner.cc:195-221).
The functions here keep those names, argument meanings and error behaviour; torch is used only
to hold device memory and streams.  There is no CPU path: every call needs the CUDA library and
raises IxkError otherwise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

__all__ = [
    "IxkError", "library_path", "load_library", "version", "launch_count", "device_status",
    "EPILOGUES", "run_gemm_custom_call", "gemm_attrs_for", "gemm", "gemm_fp8", "gemm_workspace_bytes",
    "fmha_forward_kernel", "fmha_forward_kernel_bf16", "fmha_forward_kernel_fp16", "fmha_workspace_bytes",
    "fmha_forward_kernel_static_scratch", "STATIC_SCRATCH_BYTES",
    "quantize_fp8",
]

# ----------------------------------------------------------------------------- ABI mirror

IXK_OK, IXK_INVALID_ARGUMENT, IXK_UNIMPLEMENTED, IXK_WORKSPACE_TOO_SMALL = 0, 1, 2, 3
IXK_CUDA_ERROR, IXK_NO_DEVICE, IXK_DEVICE_TIMEOUT = 4, 5, 6
IXK_BF16, IXK_F16, IXK_F32, IXK_F8E4M3, IXK_F8E5M2, IXK_S8, IXK_S32 = 0, 1, 2, 3, 4, 5, 6
ROW_MAJOR, COL_MAJOR = 0, 1
# SYCLGemm::GemmBackendEpilogue (xla/service/gpu/onednn_matmul_utils.h:35-44)
EPILOGUES = ("DEFAULT", "RELU", "GELU", "BIAS", "BIAS_RELU", "BIAS_GELU", "GELU_AUX", "BIAS_GELU_AUX")

_TORCH_TO_IXK = {
    torch.bfloat16: IXK_BF16, torch.float16: IXK_F16, torch.float32: IXK_F32,
    torch.float8_e4m3fn: IXK_F8E4M3, torch.float8_e5m2: IXK_F8E5M2, torch.int8: IXK_S8, torch.int32: IXK_S32,
}


class IxkError(RuntimeError):
    """A non-OK status from libixk.so; .status holds the ixk_status code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class _MatrixLayout(ctypes.Structure):
    _fields_ = [("order", ctypes.c_int32), ("dtype", ctypes.c_int32), ("num_rows", ctypes.c_int64),
                ("num_cols", ctypes.c_int64), ("batch_stride", ctypes.c_int64),
                ("leading_dim_stride", ctypes.c_int64)]


class _GemmDesc(ctypes.Structure):
    _fields_ = [("lhs", _MatrixLayout), ("rhs", _MatrixLayout), ("output", _MatrixLayout),
                ("batch_size", ctypes.c_int64), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
                ("epilogue", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class _FfiOperands(ctypes.Structure):
    _fields_ = [("lhs_arg", ctypes.c_int32), ("rhs_arg", ctypes.c_int32), ("c_arg", ctypes.c_int32),
                ("bias_arg", ctypes.c_int32), ("d_result", ctypes.c_int32), ("aux_result", ctypes.c_int32)]


class _FmhaDesc(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("causal", ctypes.c_int32), ("num_batches", ctypes.c_int32),
                ("num_heads", ctypes.c_int32), ("head_size", ctypes.c_int32), ("num_queries", ctypes.c_int32),
                ("num_keys", ctypes.c_int32), ("head_scale", ctypes.c_float), ("dropout_prob", ctypes.c_float),
                ("reserved", ctypes.c_int32), ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3),
                ("v_strides", ctypes.c_int64 * 3), ("o_strides", ctypes.c_int64 * 3),
                ("bias_strides", ctypes.c_int64 * 3)]


class _FmhaBwdDesc(ctypes.Structure):
    _fields_ = [("fwd", _FmhaDesc), ("do_strides", ctypes.c_int64 * 3), ("dq_strides", ctypes.c_int64 * 3),
                ("dk_strides", ctypes.c_int64 * 3), ("dv_strides", ctypes.c_int64 * 3)]


_LIB: Optional[ctypes.CDLL] = None

# Every symbol include/ixk.h declares: name -> (restype, argtypes)
_vp, _sz = ctypes.c_void_p, ctypes.c_size_t
ABI_SYMBOLS = {
    "ixk_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ixk_last_error": (ctypes.c_char_p, []),
    "ixk_version": (ctypes.c_char_p, []),
    "ixk_gemm": (ctypes.c_int, [ctypes.POINTER(_GemmDesc), _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ixk_gemm_workspace_bytes": (_sz, [ctypes.POINTER(_GemmDesc)]),
    "ixk_gemm_aux": (ctypes.c_int, [ctypes.POINTER(_GemmDesc), _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int64, _vp]),
    "ixk_ffi_select_operands": (ctypes.c_int, [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                               ctypes.POINTER(_FfiOperands)]),
    "ixk_gemm_geglu": (ctypes.c_int, [ctypes.POINTER(_GemmDesc), _vp, _vp, _vp, ctypes.c_int64, _vp, _sz, _vp]),
    "ixk_gemm_geglu_workspace_bytes": (_sz, [ctypes.POINTER(_GemmDesc)]),
    "ixk_gemm_fp8": (ctypes.c_int, [ctypes.POINTER(_GemmDesc), _vp, _vp, _vp, _vp, _vp, ctypes.c_float,
                                    ctypes.c_float, _vp, _sz, _vp]),
    "ixk_gemm_qkv": (ctypes.c_int, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp, ctypes.c_int64,
                                    _vp, ctypes.c_int64, _vp, _vp, _vp, _vp, ctypes.c_int64, _vp]),
    "ixk_fmha_fwd": (ctypes.c_int, [ctypes.POINTER(_FmhaDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ixk_fmha_bwd": (ctypes.c_int, [ctypes.POINTER(_FmhaBwdDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _sz, _vp]),
    "ixk_fmha_bwd_workspace_bytes": (_sz, [ctypes.POINTER(_FmhaBwdDesc)]),
    "ixk_row_norm": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, _vp, ctypes.c_int64,
                                    _vp, ctypes.c_int64, ctypes.c_float, _vp]),
    "ixk_rotary_interleaved": (ctypes.c_int, [ctypes.c_int, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp, _vp, _vp]),
    "ixk_row_norm_gain": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, _vp, ctypes.c_int64,
                                         _vp, ctypes.c_float, _vp, ctypes.c_int64, ctypes.c_float, _vp]),
    "ixk_rotary_half": (ctypes.c_int, [ctypes.c_int, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp, _vp, _vp]),
    "ixk_kv_append": (ctypes.c_int, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp, _vp, ctypes.c_int64,
                                     ctypes.c_int64, _vp, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp]),
    "ixk_residual_add": (ctypes.c_int, [ctypes.c_int, ctypes.c_int64, ctypes.c_int64, _vp, _vp, _vp, _vp, _vp]),
    "ixk_fmha_fwd_workspace_bytes": (_sz, [ctypes.POINTER(_FmhaDesc)]),
    "ixk_fmha_fwd_static_scratch": (ctypes.c_int, [ctypes.POINTER(_FmhaDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ixk_comm_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, ctypes.POINTER(_vp), _vp]),
    "ixk_comm_connect_ipc": (ctypes.c_int, [_vp, _vp]),
    "ixk_comm_connect_pointers": (ctypes.c_int, [_vp, ctypes.POINTER(_vp)]),
    "ixk_comm_base": (_vp, [_vp]),
    "ixk_comm_buffer": (_vp, [_vp]),
    "ixk_comm_buffer_bytes": (_sz, [_vp]),
    "ixk_comm_set_wait_limit": (ctypes.c_int, [_vp, ctypes.c_longlong]),
    "ixk_comm_set_alternating": (ctypes.c_int, [_vp, ctypes.c_int]),
    "ixk_comm_destroy": (ctypes.c_int, [_vp]),
    "ixk_all_reduce": (ctypes.c_int, [_vp, ctypes.c_int, ctypes.c_int, _sz, _vp, _sz, _vp]),
    "ixk_all_reduce_residual": (ctypes.c_int, [_vp, ctypes.c_int, _sz, _vp, _vp, _vp, ctypes.c_int64, ctypes.c_int64, _vp]),
    "ixk_reduce_scatter": (ctypes.c_int, [_vp, ctypes.c_int, ctypes.c_int, _sz, _vp, _sz, _vp]),
    "ixk_all_gather": (ctypes.c_int, [_vp, ctypes.c_int, _vp, _sz, _sz, _vp]),
    "ixk_gemm_scatter": (ctypes.c_int, [_vp, ctypes.POINTER(_GemmDesc), _vp, _vp, _vp, _vp, _sz, _vp]),
    "ixk_all_reduce_scattered": (ctypes.c_int, [_vp, ctypes.c_int, _sz, _vp, _vp, _sz, ctypes.c_int64, ctypes.c_int64, _vp]),
    "ixk_all_reduce_slice": (ctypes.c_int, [ctypes.c_int, _sz, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_sz),
                                            ctypes.POINTER(_sz)]),
    "ixk_selftest_bounded_wait": (ctypes.c_int, [ctypes.c_longlong, _vp, _vp]),
    "ixk_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "ixk_launch_count": (ctypes.c_uint64, []),
}


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libixk.so")


def load_library() -> ctypes.CDLL:
    """dlopen libixk.so and bind the ABI.  Raises IxkError if it has not been built — there is
    deliberately nothing to fall back to."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise IxkError(IXK_NO_DEVICE, f"{path} is missing: build it with "
                       f"`python {os.path.join(os.path.dirname(path), os.pardir, 'build.py')}` "
                       "(there is no CPU fallback)")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in ABI_SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib


def _check(status: int) -> None:
    if status != IXK_OK:
        lib = load_library()
        name = lib.ixk_status_string(status).decode()
        raise IxkError(status, f"{name}: {lib.ixk_last_error().decode()}")


def version() -> str:
    return load_library().ixk_version().decode()


def launch_count() -> int:
    return int(load_library().ixk_launch_count())


def device_status() -> int:
    """Synchronises the device; returns the status word (0 = clean) and raises IxkError on a
    recorded device-side timeout."""
    word = ctypes.c_int(0)
    _check(load_library().ixk_device_status(ctypes.byref(word)))
    return word.value


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream_ptr(stream) -> ctypes.c_void_p:
    if stream is None:
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream)


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise IxkError(IXK_NO_DEVICE, "operands must be CUDA tensors: libixk has no CPU path")


# ----------------------------------------------------------------------------- GEMM

def gemm_desc_from_attrs(attrs: dict, epilogue: str) -> "_GemmDesc":
    """The C descriptor for the attribute dictionary of a GEMM custom call."""
    if epilogue not in EPILOGUES:
        raise IxkError(IXK_INVALID_ARGUMENT, "Unknown Epilogue.")  # onednn_matmul_utils.cc:52-54
    d = _GemmDesc()
    for name, field in (("lhs", d.lhs), ("rhs", d.rhs), ("output", d.output)):
        field.order = int(attrs[f"{name}_order"])
        field.dtype = int(attrs[f"{name}_layout_dtype"])
        field.num_rows = int(attrs[f"{name}_num_rows"])
        field.num_cols = int(attrs[f"{name}_num_cols"])
        field.batch_stride = int(attrs[f"{name}_batch_stride"])
        field.leading_dim_stride = int(attrs[f"{name}_leading_dim_stride"])
    d.batch_size = int(attrs["batch_size"])
    d.alpha = float(attrs.get("alpha", 1.0))
    d.beta = float(attrs.get("beta", 0.0))
    d.epilogue = EPILOGUES.index(epilogue)
    d.reserved = 0
    return d


def run_gemm_custom_call(lhs: torch.Tensor, rhs: torch.Tensor, add: Optional[torch.Tensor],
                         output: torch.Tensor, bias: Optional[torch.Tensor], stream, attrs: dict,
                         epilogue: str, *, inv_scale_a: Optional[float] = None,
                         inv_scale_b: Optional[float] = None, workspace: Optional[torch.Tensor] = None,
                         aux: Optional[torch.Tensor] = None) -> None:
    """RunGemmCustomCall (xla/service/gpu/sycl_onednn.cc:38-54): buffers + the FFI attribute
    dictionary RunGemm reads (xla/service/gpu/onednn_matmul_utils.cc:543-595).  `attrs` keys:
    {lhs,rhs,output}_{order,num_rows,num_cols,batch_stride,leading_dim_stride,layout_dtype},
    batch_size, alpha, beta.  `add` is the C operand read when beta != 0 (it may be `output`).
    With inv_scale_a/b given the operands are fp8 and the scaled-GEMM entry point is used.
    `workspace` is the scratch the reference's handler passes down (sycl_onednn.h:37): skinny
    problems (M <= 128) use it to split K over more SMs; see gemm_workspace_bytes().  `aux` is the
    second result of the GELU_AUX / BIAS_GELU_AUX epilogues (the pre-activation values, the
    output's type, shape and order)."""
    if epilogue not in EPILOGUES:
        raise IxkError(IXK_INVALID_ARGUMENT, "Unknown Epilogue.")  # onednn_matmul_utils.cc:52-54
    _require_cuda(lhs, rhs, add, output, bias, aux)
    lib = load_library()
    d = gemm_desc_from_attrs(attrs, epilogue)
    sp = _stream_ptr(stream)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    if aux is not None:
        order = int(attrs["output_order"])
        aux_ld = aux.stride(-2) if order == ROW_MAJOR else aux.stride(-1)
        st = lib.ixk_gemm_aux(ctypes.byref(d), _ptr(lhs), _ptr(rhs), _ptr(add), _ptr(bias), _ptr(output), _ptr(aux),
                              int(aux_ld), sp)
    elif inv_scale_a is not None or inv_scale_b is not None:
        st = lib.ixk_gemm_fp8(ctypes.byref(d), _ptr(lhs), _ptr(rhs), _ptr(add), _ptr(bias), _ptr(output),
                              float(inv_scale_a), float(inv_scale_b), _ptr(workspace), ws_bytes, sp)
    else:
        st = lib.ixk_gemm(ctypes.byref(d), _ptr(lhs), _ptr(rhs), _ptr(add), _ptr(bias), _ptr(output),
                          _ptr(workspace), ws_bytes, sp)
    _check(st)


def gemm_workspace_bytes(lhs: torch.Tensor, rhs: torch.Tensor, out_shape=None) -> int:
    """Scratch bytes ixk_gemm can make use of for lhs @ rhs (0 unless the problem is skinny)."""
    d = _GemmDesc()
    m, k = lhs.shape[-2], lhs.shape[-1]
    n = rhs.shape[-1]
    d.lhs.num_rows, d.lhs.num_cols, d.lhs.dtype = m, k, _TORCH_TO_IXK[lhs.dtype]
    d.rhs.num_rows, d.rhs.num_cols = k, n
    d.output.num_rows, d.output.num_cols = m, n
    d.batch_size = lhs.shape[0] if lhs.dim() == 3 else 1
    return int(load_library().ixk_gemm_workspace_bytes(ctypes.byref(d)))


def _matrix_attrs(prefix: str, t: torch.Tensor) -> dict:
    """Layout attributes of a 2-D or 3-D (batched) tensor view: whichever of the last two
    dimensions has stride 1 decides the order."""
    if t.dim() not in (2, 3):
        raise IxkError(IXK_INVALID_ARGUMENT, f"{prefix}: expected a 2-D or 3-D tensor")
    rows, cols = t.shape[-2], t.shape[-1]
    sr, sc = t.stride(-2), t.stride(-1)
    if sc == 1 and (sr >= cols or rows == 1):
        order, ld = ROW_MAJOR, (sr if rows > 1 else max(sr, cols))
    elif sr == 1 and (sc >= rows or cols == 1):
        order, ld = COL_MAJOR, (sc if cols > 1 else max(sc, rows))
    else:
        raise IxkError(IXK_INVALID_ARGUMENT, f"{prefix}: neither of the last two dimensions is contiguous")
    bs = t.stride(0) if t.dim() == 3 else rows * cols
    return {f"{prefix}_order": order, f"{prefix}_num_rows": rows, f"{prefix}_num_cols": cols,
            f"{prefix}_batch_stride": bs, f"{prefix}_leading_dim_stride": ld,
            f"{prefix}_layout_dtype": _TORCH_TO_IXK[t.dtype]}


def gemm_attrs_for(lhs: torch.Tensor, rhs: torch.Tensor, output: torch.Tensor, beta: float = 0.0,
                   alpha: float = 1.0) -> dict:
    """The attribute dictionary XLA's GEMM rewriter would attach for these three tensor views."""
    attrs = {}
    attrs.update(_matrix_attrs("lhs", lhs))
    attrs.update(_matrix_attrs("rhs", rhs))
    attrs.update(_matrix_attrs("output", output))
    attrs["batch_size"] = output.shape[0] if output.dim() == 3 else 1
    attrs["alpha"] = float(alpha)
    attrs["beta"] = float(beta)
    attrs["algorithm"] = 0
    return attrs


def gemm(lhs: torch.Tensor, rhs: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
         c: Optional[torch.Tensor] = None, beta: float = 0.0, epilogue: str = "DEFAULT",
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         stream=None, workspace: Optional[torch.Tensor] = None, alpha: float = 1.0,
         aux: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(alpha * lhs @ rhs + bias + beta*c) through "__cublas$lt$matmul"'s path.  Any mix of
    row-/column-major 2-D (or batched 3-D) views is passed through as-is, never copied.  With a
    *_AUX epilogue `aux` receives the values the activation is applied to."""
    if out is None:
        shape = (*lhs.shape[:-1], rhs.shape[-1])
        out = torch.empty(shape, device=lhs.device, dtype=out_dtype or lhs.dtype)
    attrs = gemm_attrs_for(lhs, rhs, out, beta, alpha)
    run_gemm_custom_call(lhs, rhs, c, out, bias, stream, attrs, epilogue, workspace=workspace, aux=aux)
    return out


def gemm_geglu(x: torch.Tensor, w_gate_up: torch.Tensor, *, out: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """gelu_tanh(x @ w[:, :N']) * (x @ w[:, N':]) for x [M <= 128, K] and w [K, 2 N'] in one GEMM and one
    combining pass (decode-time GeGLU).  `workspace`: uint8 scratch of gemm_geglu_workspace_bytes()
    bytes (allocated here when absent)."""
    m, n2 = x.shape[-2], w_gate_up.shape[-1]
    if out is None:
        out = torch.empty((m, n2 // 2), device=x.device, dtype=x.dtype)
    d = gemm_desc_from_attrs(gemm_attrs_for(x, w_gate_up, torch.empty((m, n2), device="meta", dtype=x.dtype)), "DEFAULT")
    lib = load_library()
    need = int(lib.ixk_gemm_geglu_workspace_bytes(ctypes.byref(d)))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    _check(lib.ixk_gemm_geglu(ctypes.byref(d), _ptr(x), _ptr(w_gate_up), _ptr(out), out.stride(-2), _ptr(workspace),
                              workspace.numel() * workspace.element_size(), _stream_ptr(stream)))
    return out


def quantize_fp8(x: torch.Tensor, dtype: torch.dtype):
    """Per-tensor scaled, saturating quantisation used by the fp8 configuration:
    scale = max_finite / amax(x); returns (fp8 tensor, scale).  Works on any device (it is
    input preparation, not part of the timed path)."""
    fmax = torch.finfo(dtype).max
    amax = x.abs().max().item()
    scale = fmax / amax if amax > 0 else 1.0
    q = (x.float() * scale).clamp_(-fmax, fmax).to(dtype)
    return q, scale


def gemm_fp8(lhs_q: torch.Tensor, rhs_q: torch.Tensor, inv_scale_a: float, inv_scale_b: float, *,
             bias: Optional[torch.Tensor] = None, epilogue: str = "DEFAULT",
             out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
             stream=None) -> torch.Tensor:
    """out = cast((lhs_q @ rhs_q in fp32) * inv_scale_a * inv_scale_b [+ bias, act])."""
    if out is None:
        out = torch.empty((*lhs_q.shape[:-1], rhs_q.shape[-1]), device=lhs_q.device, dtype=out_dtype)
    attrs = gemm_attrs_for(lhs_q, rhs_q, out, 0.0)
    run_gemm_custom_call(lhs_q, rhs_q, None, out, bias, stream, attrs, epilogue,
                         inv_scale_a=inv_scale_a, inv_scale_b=inv_scale_b)
    return out


def gemm_qkv(x: torch.Tensor, w_qkv: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
             outs=None, stream=None):
    """Three projections of one input, as XetlaQKVGemmKernel (xetla/gemm/gemm.h:111-171) runs them:
    x [m,k] row-major, w_qkv [3,k,n] (three row-major slabs one behind the other), bias [3,n] or
    None -> (q, k, v), each [m,n].  `outs` may give the three output tensors (any placement; a
    contiguous [3,m,n] buffer runs as one launch)."""
    if x.dim() != 2 or w_qkv.dim() != 3 or w_qkv.shape[0] != 3 or w_qkv.shape[1] != x.shape[1]:
        raise IxkError(IXK_INVALID_ARGUMENT, "x must be [m,k] and w_qkv [3,k,n]")
    if x.stride(1) != 1 or not w_qkv.is_contiguous():
        raise IxkError(IXK_INVALID_ARGUMENT, "x must be row-major and w_qkv contiguous")
    m, k = x.shape
    n = w_qkv.shape[2]
    if outs is None:
        buf = torch.empty(3, m, n, dtype=x.dtype, device=x.device)
        outs = (buf[0], buf[1], buf[2])
    for o in outs:
        if o.shape != (m, n) or o.stride(1) != 1 or o.stride(0) != outs[0].stride(0) or o.dtype != x.dtype:
            raise IxkError(IXK_INVALID_ARGUMENT, "outputs must be row-major [m,n] of the input type with one pitch")
    if bias is not None and (bias.shape != (3, n) or not bias.is_contiguous() or bias.dtype != x.dtype):
        raise IxkError(IXK_INVALID_ARGUMENT, "bias must be a contiguous [3,n] tensor of the input type")
    lib = load_library()
    _check(lib.ixk_gemm_qkv(_TORCH_TO_IXK[x.dtype], m, n, k, x.data_ptr(), x.stride(0), w_qkv.data_ptr(), n,
                            bias.data_ptr() if bias is not None else None, outs[0].data_ptr(), outs[1].data_ptr(),
                            outs[2].data_ptr(), outs[0].stride(0), _stream_ptr(stream)))
    return tuple(outs)


# ----------------------------------------------------------------------------- between the calls

NORM_LAYER, NORM_RMS = 0, 1


def row_norm(x: torch.Tensor, *, kind: int = NORM_LAYER, eps: float = 1e-5, out: Optional[torch.Tensor] = None,
             stream=None, gain: Optional[torch.Tensor] = None, gain_offset: float = 0.0) -> torch.Tensor:
    """LayerNorm (zero shift) or RMSNorm over the last dimension of a dense tensor; with `gain` [cols]
    the normalised row is multiplied by (gain_offset + gain) before the one rounding."""
    if not x.is_contiguous():
        raise IxkError(IXK_INVALID_ARGUMENT, "row_norm wants a contiguous tensor")
    out = torch.empty_like(x) if out is None else out
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise IxkError(IXK_INVALID_ARGUMENT, "out must match x")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if gain is not None:
        if gain.shape != (cols,) or gain.dtype != x.dtype or not gain.is_contiguous():
            raise IxkError(IXK_INVALID_ARGUMENT, "gain must be a dense [cols] vector of the input type")
        _check(load_library().ixk_row_norm_gain(_TORCH_TO_IXK[x.dtype], kind, rows, cols, x.data_ptr(), cols, gain.data_ptr(),
                                                float(gain_offset), out.data_ptr(), cols, eps, _stream_ptr(stream)))
        return out
    _check(load_library().ixk_row_norm(_TORCH_TO_IXK[x.dtype], kind, rows, cols, x.data_ptr(), cols, out.data_ptr(),
                                       cols, eps, _stream_ptr(stream)))
    return out


def rotary_interleaved_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, rotary_dim: int,
                        stream=None, half_split: bool = False) -> torch.Tensor:
    """In place on x [tokens, heads, head_dim] (any token pitch, unit element stride): pairs (2i, 2i+1)
    of the first rotary_dim elements of every head (half_split: pairs (i, i + rotary_dim/2)), token
    t at position t % seq_len; cos/sin fp32 [seq_len, rotary_dim/2]."""
    if x.dim() != 3 or x.stride(2) != 1:
        raise IxkError(IXK_INVALID_ARGUMENT, "x must be [tokens, heads, head_dim] with unit element stride")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous() \
            or cos.shape != (seq_len, rotary_dim // 2) or sin.shape != cos.shape:
        raise IxkError(IXK_INVALID_ARGUMENT, "cos/sin must be contiguous fp32 [seq_len, rotary_dim/2]")
    if rotary_dim > x.shape[2]:
        raise IxkError(IXK_INVALID_ARGUMENT, "rotary_dim exceeds head_dim")
    fn = load_library().ixk_rotary_half if half_split else load_library().ixk_rotary_interleaved
    _check(fn(_TORCH_TO_IXK[x.dtype], x.data_ptr(), x.shape[0], seq_len, x.shape[1], rotary_dim, x.stride(0), x.stride(1),
              cos.data_ptr(), sin.data_ptr(), _stream_ptr(stream)))
    return x


def rotary_half_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, rotary_dim: int, stream=None):
    """The half-split convention of the Gemma family: see rotary_interleaved_."""
    return rotary_interleaved_(x, cos, sin, seq_len, rotary_dim, stream, half_split=True)


def kv_append_(k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, position: int,
               stream=None) -> None:
    """k_cache / v_cache [B, T, heads, head_dim] (any strides with unit element stride, the same for
    both): cache[:, position] = new, new [B, heads, head_dim] views (e.g. slices of a fused QKV
    projection), both tensors in one launch."""
    B, T, N, H = k_cache.shape
    if v_cache.shape != k_cache.shape or v_cache.stride() != k_cache.stride() or k_new.shape != (B, N, H) or \
            v_new.shape != (B, N, H) or k_new.stride() != v_new.stride() or k_cache.stride(3) != 1 or k_new.stride(2) != 1:
        raise IxkError(IXK_INVALID_ARGUMENT, "caches [B,T,N,H] and new rows [B,N,H] of matching shapes and strides are expected")
    if not 0 <= position < T:
        raise IxkError(IXK_INVALID_ARGUMENT, "position outside the cache")
    _check(load_library().ixk_kv_append(_TORCH_TO_IXK[k_cache.dtype], B, N, H, k_new.data_ptr(), v_new.data_ptr(),
                                        k_new.stride(0), k_new.stride(1), k_cache.data_ptr(), v_cache.data_ptr(),
                                        k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), position, _stream_ptr(stream)))


def residual_add(x: torch.Tensor, partial: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """x + partial, or x + round(partial + bias) with bias along the last dimension."""
    if not x.is_contiguous() or not partial.is_contiguous() or partial.numel() != x.numel() or partial.dtype != x.dtype:
        raise IxkError(IXK_INVALID_ARGUMENT, "x and partial must be dense tensors of one size and type")
    cols = x.shape[-1]
    if bias is not None and (bias.shape != (cols,) or bias.dtype != x.dtype or not bias.is_contiguous()):
        raise IxkError(IXK_INVALID_ARGUMENT, "bias must be a dense [cols] vector of the input type")
    out = torch.empty_like(x) if out is None else out
    if out.numel() != x.numel() or out.dtype != x.dtype or not out.is_contiguous():
        raise IxkError(IXK_INVALID_ARGUMENT, "out must match x")
    rows = x.numel() // cols if cols else 0
    _check(load_library().ixk_residual_add(_TORCH_TO_IXK[x.dtype], rows, cols, x.data_ptr(), partial.data_ptr(),
                                           bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                           _stream_ptr(stream)))
    return out


# ----------------------------------------------------------------------------- attention

def _fmha_desc(query, key, value, bias, out, head_scale, causal, dropout_prob) -> _FmhaDesc:
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4 or out.dim() != 4:
        raise IxkError(IXK_INVALID_ARGUMENT, "q, k, v, out must be 4-D [B,N,S,H] views")
    B, N, F, H = query.shape
    T = key.shape[2]
    # The descriptor carries one B, N and H for all four tensors: a K of [B,1,T,H] has to be
    # handed over as an expanded (stride-0) view, not as a smaller tensor that would be read
    # as if it had N heads.
    if tuple(key.shape) != (B, N, T, H) or value.shape != key.shape or out.shape != query.shape:
        raise IxkError(IXK_INVALID_ARGUMENT, "k and v must be [B,N,T,H] and out [B,N,F,H] with q's B, N and H "
                       "(share K/V between heads with .expand(), which gives stride 0)")
    if not (key.dtype == value.dtype == out.dtype == query.dtype) or (bias is not None and bias.dtype != query.dtype):
        raise IxkError(IXK_INVALID_ARGUMENT, "q, k, v, bias and out must have one element type")
    d = _FmhaDesc()
    d.dtype = _TORCH_TO_IXK[query.dtype]
    d.causal = 1 if causal else 0
    d.num_batches, d.num_heads, d.head_size, d.num_queries, d.num_keys = B, N, H, F, T
    d.head_scale = float(head_scale)
    d.dropout_prob = float(dropout_prob)
    d.reserved = 0
    for name, t in (("q", query), ("k", key), ("v", value), ("o", out)):
        if t.stride(3) != 1 and t.shape[3] > 1:
            # xetla_gpu_fused_mha_runner.cc:114-116 CHECKs the same
            raise IxkError(IXK_INVALID_ARGUMENT, f"{name}: head_size must be the contiguous dimension")
        getattr(d, f"{name}_strides")[:] = [t.stride(0), t.stride(1), t.stride(2)]
    if bias is not None:
        if bias.dim() != 4 or bias.shape[3] != T or bias.shape[2] != F:
            raise IxkError(IXK_INVALID_ARGUMENT, "bias must be [B|1, N|1, F, T]")
        if bias.stride(3) != 1:
            raise IxkError(IXK_INVALID_ARGUMENT, "bias: the key dimension must be contiguous")
        d.bias_strides[:] = [bias.stride(0) if bias.shape[0] > 1 else 0,
                             bias.stride(1) if bias.shape[1] > 1 else 0, bias.stride(2)]
    return d


def fmha_workspace_bytes(query, key, value, bias, out, head_scale, causal=False) -> int:
    d = _fmha_desc(query, key, value, bias, out, head_scale, causal, 0.0)
    return int(load_library().ixk_fmha_fwd_workspace_bytes(ctypes.byref(d)))


def fmha_forward_kernel(stream, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                        bias: Optional[torch.Tensor], dropout, dropout_prob: float, out: torch.Tensor,
                        activation: Optional[torch.Tensor], head_scale: float, is_training: bool = False,
                        *, causal: bool = False, workspace: Optional[torch.Tensor] = None) -> None:
    """fmha_forward_kernel_{bf16,fp16} (xla/service/gpu/xetla/sdp/sdp_forward.cc:34-84), the dtype
    taken from `query`.  q/out are [B,N,F,H] views, k/v [B,N,T,H] views (any strides with H
    contiguous, so [B,S,N,H] storage is passed as a permuted view); `activation` receives the
    log-sum-exp rows when is_training (xla/service/gpu/xetla/sdp/fmha_forward.h:433-450).
    `dropout` must be None: the runner rejects dropout (xetla_gpu_fused_mha_runner.cc:56-62).
    `causal` is a real flag here; the reference compiles it out (sdp_forward.cc:41) and expects
    callers to fold the mask into `bias`."""
    _require_cuda(query, key, value, bias, out, activation)
    if dropout is not None:
        raise IxkError(IXK_UNIMPLEMENTED, "Unimplemented dropout")
    if is_training and activation is None:
        raise IxkError(IXK_INVALID_ARGUMENT, "is_training needs the activation (log-sum-exp) buffer")
    lib = load_library()
    d = _fmha_desc(query, key, value, bias, out, head_scale, causal, 0.0 if dropout_prob in (None, 1.0) else dropout_prob)
    need = int(lib.ixk_fmha_fwd_workspace_bytes(ctypes.byref(d)))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=query.device)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    st = lib.ixk_fmha_fwd(ctypes.byref(d), _ptr(query), _ptr(key), _ptr(value), _ptr(bias), _ptr(out),
                          _ptr(activation if is_training else None), _ptr(workspace), ws_bytes, _stream_ptr(stream))
    _check(st)


def _fmha_bwd_desc(query, key, value, out, bias, grad_out, grad_query, grad_key, grad_value, head_scale,
                   causal) -> _FmhaBwdDesc:
    d = _FmhaBwdDesc()
    d.fwd = _fmha_desc(query, key, value, bias, out, head_scale, causal, 0.0)
    for name, t, like in (("do", grad_out, query), ("dq", grad_query, query), ("dk", grad_key, key),
                          ("dv", grad_value, value)):
        if t.shape != like.shape or t.dtype != like.dtype:
            raise IxkError(IXK_INVALID_ARGUMENT, f"{name}: shape and type must match the tensor it is the gradient of")
        if t.stride(3) != 1 and t.shape[3] > 1:
            raise IxkError(IXK_INVALID_ARGUMENT, f"{name}: head_size must be the contiguous dimension")
        getattr(d, f"{name}_strides")[:] = [t.stride(0), t.stride(1), t.stride(2)]
    return d


def fmha_backward_workspace_bytes(query, key, value, out, bias, grad_out, grad_query, grad_key, grad_value,
                                  head_scale, causal=False) -> int:
    d = _fmha_bwd_desc(query, key, value, out, bias, grad_out, grad_query, grad_key, grad_value, head_scale, causal)
    return int(load_library().ixk_fmha_bwd_workspace_bytes(ctypes.byref(d)))


def fmha_backward_kernel(stream, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: torch.Tensor,
                         bias: Optional[torch.Tensor], grad_out: torch.Tensor, activation: torch.Tensor,
                         grad_query: torch.Tensor, grad_key: torch.Tensor, grad_value: torch.Tensor,
                         head_scale: float, *, causal: bool = False,
                         workspace: Optional[torch.Tensor] = None) -> None:
    """fmha_backward_kernel_{bf16,fp16} (xla/service/gpu/xetla/sdp/sdp_backward.cc:34-76), the dtype
    taken from `query`.  query/out/grad_out/grad_query are [B,N,F,H] views, key/value and their
    gradients [B,N,T,H] views (any strides with H contiguous); `activation` is the forward's
    log-sum-exp [B,N,F] fp32.  The reference's dp_sum and grad_query_accum scratch buffers are one
    `workspace` here (allocated if not given)."""
    _require_cuda(query, key, value, out, bias, grad_out, activation, grad_query, grad_key, grad_value)
    if activation is None or activation.dtype != torch.float32 or not activation.is_contiguous() \
            or activation.shape != query.shape[:3]:
        raise IxkError(IXK_INVALID_ARGUMENT, "activation must be the forward's dense fp32 [B,N,F] log-sum-exp")
    lib = load_library()
    d = _fmha_bwd_desc(query, key, value, out, bias, grad_out, grad_query, grad_key, grad_value, head_scale, causal)
    need = int(lib.ixk_fmha_bwd_workspace_bytes(ctypes.byref(d)))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=query.device)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    st = lib.ixk_fmha_bwd(ctypes.byref(d), _ptr(query), _ptr(key), _ptr(value), _ptr(out), _ptr(bias), _ptr(grad_out),
                          _ptr(activation), _ptr(grad_query), _ptr(grad_key), _ptr(grad_value), _ptr(workspace),
                          ws_bytes, _stream_ptr(stream))
    _check(st)


STATIC_SCRATCH_BYTES = 4 << 20  # IXK_STATIC_SCRATCH_BYTES in include/ixk.h


def fmha_forward_kernel_static_scratch(stream, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                       bias: Optional[torch.Tensor], out: torch.Tensor,
                                       activation: Optional[torch.Tensor], head_scale: float, *,
                                       causal: bool = False) -> None:
    """fmha_forward_kernel for a caller that cannot provide (or allocate) scratch memory: the
    decode path's partial results go to a fixed array inside the library instead
    (ixk_fmha_fwd_static_scratch).  Nothing is allocated here either — not even through torch.
    Problems needing more than STATIC_SCRATCH_BYTES raise IxkError(WORKSPACE_TOO_SMALL).  Calls on
    one device share that array: do not let two of them overlap on the GPU."""
    _require_cuda(query, key, value, bias, out, activation)
    d = _fmha_desc(query, key, value, bias, out, head_scale, causal, 0.0)
    st = load_library().ixk_fmha_fwd_static_scratch(ctypes.byref(d), _ptr(query), _ptr(key), _ptr(value), _ptr(bias),
                                                    _ptr(out), _ptr(activation), _stream_ptr(stream))
    _check(st)


def fmha_forward_kernel_bf16(stream, query, key, value, bias, dropout, dropout_prob, out, activation,
                             num_batches, num_heads, head_size, num_queries, num_keys, head_scale,
                             is_training, *, causal=False):
    """Positional twin of the reference declaration (xla/service/gpu/xetla/sdp/sdp_forward.h:30-36);
    the sizes must agree with the tensor views."""
    if query.dtype != torch.bfloat16:
        raise IxkError(IXK_INVALID_ARGUMENT, "Invalid MHA datatype")  # xetla_gpu_fused_mha_runner.cc:145
    if tuple(query.shape) != (num_batches, num_heads, num_queries, head_size) or key.shape[2] != num_keys:
        raise IxkError(IXK_INVALID_ARGUMENT, "sizes do not match the tensor views")
    fmha_forward_kernel(stream, query, key, value, bias, dropout, dropout_prob, out, activation, head_scale,
                        is_training, causal=causal)


def fmha_forward_kernel_fp16(stream, query, key, value, bias, dropout, dropout_prob, out, activation,
                             num_batches, num_heads, head_size, num_queries, num_keys, head_scale,
                             is_training, *, causal=False):
    """fp16 twin (xla/service/gpu/xetla/sdp/sdp_forward.h:22-28)."""
    if query.dtype != torch.float16:
        raise IxkError(IXK_INVALID_ARGUMENT, "Invalid MHA datatype")
    if tuple(query.shape) != (num_batches, num_heads, num_queries, head_size) or key.shape[2] != num_keys:
        raise IxkError(IXK_INVALID_ARGUMENT, "sizes do not match the tensor views")
    fmha_forward_kernel(stream, query, key, value, bias, dropout, dropout_prob, out, activation, head_scale,
                        is_training, causal=causal)
