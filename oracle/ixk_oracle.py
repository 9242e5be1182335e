"""CPU oracle for the three kernel paths (TEST INFRASTRUCTURE — never the product path).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this
module; the library itself has no CPU fallback.

PARITY UNPINNED: the reference's kernels for these paths (SYCL/ESIMD on XeTLA v0.3.7.2,
intel/xetla@ae46a690, and oneDNN v3.7, oneapi-src/oneDNN@5e922403) cannot be compiled or
imported in this environment, and the reference ships no golden vectors for them — its GEMM
accuracy test is commented out (test/jax_ut.patch:582-616) and its attention test compares
against an un-jitted jnp expression at atol 3e-2 / 1e-2 (test/jax_ut.patch:978-998).
What this module restates is therefore the arithmetic the reference's call sites specify,
in numpy float32, and it is cross-checked in tests/ against independent implementations
(torch CPU scaled_dot_product_attention / gelu(approximate="tanh") and ml_dtypes' fp8 casts).

Sections:
  * element types: bf16 / fp16 rounding, fp8 e4m3fn / e5m2 saturating quantisation
  * gemm_custom_call: RunGemm's layout handling + the epilogue chain
  * fmha_forward: the flash-attention forward of fmha_forward.h, un-tiled
  * fp8_scaled_gemm: the contract of the fp8 example
"""
from __future__ import annotations

import math

import numpy as np

# --------------------------------------------------------------------------- element types

BF16, F16, F32, F8E4M3, F8E5M2 = 0, 1, 2, 3, 4  # ixk_dtype values (include/ixk.h)
ROW_MAJOR, COL_MAJOR = 0, 1

EPILOGUES = ("DEFAULT", "RELU", "GELU", "BIAS", "BIAS_RELU", "BIAS_GELU", "GELU_AUX", "BIAS_GELU_AUX")
# SYCLGemm::GemmBackendEpilogue order, xla/service/gpu/onednn_matmul_utils.h:35-44.


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even; NaN stays NaN."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    nan = np.isnan(x)
    out = rounded.astype(np.uint16)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16, returned as float32."""
    return bf16_to_f32(bf16_bits(x))


def round_f16(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_to(x: np.ndarray, dtype: int) -> np.ndarray:
    """Round a float32 array to `dtype` and return it as float32."""
    if dtype == BF16:
        return round_bf16(x)
    if dtype == F16:
        return round_f16(x)
    if dtype == F32:
        return np.asarray(x, dtype=np.float32)
    raise ValueError(f"round_to: unsupported dtype {dtype}")


def _fp8_tables(exp_bits: int, man_bits: int, bias: int, fn: bool):
    """All non-negative finite values of an 8-bit float, indexed by their 7-bit code."""
    vals = np.full(128, np.nan, dtype=np.float64)
    for code in range(128):
        e = code >> man_bits
        m = code & ((1 << man_bits) - 1)
        if fn:
            if code == 0x7F:  # e4m3fn: the single NaN code; everything else is finite
                continue
        elif e == (1 << exp_bits) - 1:  # IEEE-like: top exponent is inf / NaN
            continue
        if e == 0:
            vals[code] = m * 2.0 ** (1 - bias - man_bits)
        else:
            vals[code] = (1 + m / (1 << man_bits)) * 2.0 ** (e - bias)
    return vals


_E4M3 = _fp8_tables(4, 3, 7, fn=True)    # max finite 448 (code 0x7E)
_E5M2 = _fp8_tables(5, 2, 15, fn=False)  # max finite 57344 (code 0x7B)
FP8_MAX = {F8E4M3: 448.0, F8E5M2: 57344.0}


def fp8_decode(codes: np.ndarray, dtype: int) -> np.ndarray:
    """uint8 fp8 codes -> float32."""
    table = _E4M3 if dtype == F8E4M3 else _E5M2
    codes = np.asarray(codes, dtype=np.uint8)
    mag = table[codes & 0x7F]
    return np.where(codes & 0x80, -mag, mag).astype(np.float32)


def fp8_encode_sat(x: np.ndarray, dtype: int) -> np.ndarray:
    """float32 -> fp8 codes (uint8): clamp to +-max finite, then round to nearest, ties to the
    even code.  (Saturating on purpose: a plain ml_dtypes cast turns e4m3fn overflow into NaN.)"""
    table = _E4M3 if dtype == F8E4M3 else _E5M2
    n_finite = int(np.sum(~np.isnan(table)))
    finite = table[:n_finite]  # ascending
    x = np.asarray(x, dtype=np.float32)
    mag = np.minimum(np.abs(x).astype(np.float64), finite[-1])
    hi = np.searchsorted(finite, mag, side="left")
    hi = np.clip(hi, 0, n_finite - 1)
    lo = np.clip(hi - 1, 0, n_finite - 1)
    d_hi = finite[hi] - mag
    d_lo = mag - finite[lo]
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    code = np.where(np.signbit(x), code | np.uint8(0x80), code)
    return np.where(np.isnan(x), np.uint8(0x7F if dtype == F8E4M3 else 0x7E), code).astype(np.uint8)


def quantize_fp8(x: np.ndarray, dtype: int):
    """Per-tensor scaled quantisation of the fp8 config: scale = max_finite / amax;
    returns (codes uint8, scale float).  Dequantised value = decode(codes) / scale."""
    amax = float(np.max(np.abs(x)))
    scale = FP8_MAX[dtype] / amax if amax > 0 else 1.0
    return fp8_encode_sat(np.asarray(x, np.float32) * np.float32(scale), dtype), scale


# --------------------------------------------------------------------------- GEMM custom call

def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """oneDNN eltwise_gelu_tanh (xla/service/gpu/onednn_matmul_utils.cc:447) ==
    XeTLA gelu_fwd_op_t (xla/service/gpu/xetla/gemm/hgemm_impl.h:331,439), in float32."""
    x = np.asarray(x, dtype=np.float32)
    u = np.float32(math.sqrt(2.0 / math.pi)) * (x + np.float32(0.044715) * x * x * x)
    return np.float32(0.5) * x * (np.float32(1.0) + np.tanh(u))


def _logical(mat: np.ndarray, layout: dict) -> np.ndarray:
    """View a flat/2-D/3-D storage array as the logical [batch, rows, cols] float32 matrix
    described by a layout dict with the reference's attribute names
    (xla/service/gpu/onednn_matmul_utils.cc:543-590)."""
    rows, cols = layout["num_rows"], layout["num_cols"]
    ld, bs, batch = layout["leading_dim_stride"], layout.get("batch_stride", 0), layout.get("batch_size", 1)
    flat = np.asarray(mat, dtype=np.float32).reshape(-1)
    out = np.empty((batch, rows, cols), dtype=np.float32)
    for b in range(batch):
        base = b * bs
        if layout["order"] == ROW_MAJOR:
            idx = base + np.arange(rows)[:, None] * ld + np.arange(cols)[None, :]
        else:
            idx = base + np.arange(rows)[:, None] + np.arange(cols)[None, :] * ld
        out[b] = flat[idx]
    return out


def gemm_epilogue(acc: np.ndarray, bias, c, beta: float, epilogue: str, out_dtype: int, alpha: float = 1.0,
                  with_aux: bool = False):
    """The post-accumulation chain on float32 accumulators, one rounding at the end:
    alpha (the addmm form alpha*acc + beta*res, xla/service/gpu/xetla/gemm/epilogue_impl.h:83),
    bias add (:237-241), residual beta*C (:161, onednn append_sum at onednn_matmul_utils.cc:439),
    activation applied after the sum (:441-449), cast to the output type.
    The *_AUX epilogues (declared at onednn_matmul_utils.h:42-43, rejected by the reference's
    kernels, :321-322) are GELU with the pre-activation values as a second result: with_aux=True
    returns (D, aux), both rounded to the output type."""
    if epilogue not in EPILOGUES:
        raise ValueError("Unknown Epilogue.")
    if epilogue.endswith("_AUX") and not with_aux:
        raise NotImplementedError("Unsupported Activation mode")  # onednn_matmul_utils.cc:321-322
    v = np.asarray(acc, dtype=np.float32) * np.float32(alpha)
    if "BIAS" in epilogue:
        v = v + np.asarray(bias, dtype=np.float32)[None, :]
    if beta != 0.0:
        v = v + np.float32(beta) * np.asarray(c, dtype=np.float32)
    pre = v
    if epilogue.endswith("RELU"):
        v = np.maximum(v, np.float32(0))
    elif "GELU" in epilogue:
        v = gelu_tanh(v)
    if with_aux:
        return round_to(v, out_dtype), round_to(pre, out_dtype)
    return round_to(v, out_dtype)


def tf32_operand(x: np.ndarray, mode: str = "truncate") -> np.ndarray:
    """An fp32 GEMM operand as the TF32 math mode sees it (the reference's XLA_FP32_MATH_MODE=TF32,
    xla/service/onednn_util.h:53-70: 8 exponent bits, 10 mantissa bits): the low 13 mantissa bits are
    dropped ("truncate", what a tensor core does with fp32 bits) or rounded to nearest, ties away
    from zero ("round", what a conversion instruction does)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    if mode == "round":
        bits = bits + np.uint32(0x1000)
    return (bits & np.uint32(0xFFFFE000)).view(np.float32)


def gemm_s8(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """(S8,S8,S32) of RunGemm's type list (xla/service/gpu/onednn_matmul_utils.cc:610): exact integer
    products summed in 32 bits (int64 here, then wrapped, so that overflow behaves as two's complement)."""
    acc = np.asarray(a, dtype=np.int64) @ np.asarray(b, dtype=np.int64)
    return acc.astype(np.int32)


def gemm_custom_call(attrs: dict, lhs, rhs, c, bias, epilogue: str, out_dtype: int) -> np.ndarray:
    """RunGemm (xla/service/gpu/onednn_matmul_utils.cc:533-621) on float32 copies of the
    (already type-rounded) operands.  `attrs` carries the reference's dictionary keys:
    {lhs,rhs,output}_{order,num_rows,num_cols,batch_stride,leading_dim_stride}, batch_size,
    alpha, beta.  Returns the logical [batch, M, N] result, rounded to out_dtype, as float32.

    A column-major output is produced as D^T = B^T.A^T (:520-530); the bias then runs along
    the columns of that rewritten problem (:363-365), i.e. along the ORIGINAL rows."""
    alpha = float(attrs.get("alpha", 1.0))   # the reference CHECKs alpha == 1 (onednn_matmul_utils.cc:438)
    batch = attrs.get("batch_size", 1)

    def lay(p):
        return dict(order=attrs[f"{p}_order"], num_rows=attrs[f"{p}_num_rows"], num_cols=attrs[f"{p}_num_cols"],
                    batch_stride=attrs.get(f"{p}_batch_stride", 0),
                    leading_dim_stride=attrs[f"{p}_leading_dim_stride"], batch_size=batch)

    a = _logical(lhs, lay("lhs"))
    b = _logical(rhs, lay("rhs"))
    beta = float(attrs.get("beta", 0.0))
    cc = _logical(c, lay("output")) if beta != 0.0 else None
    transposed_out = attrs["output_order"] == COL_MAJOR
    out = np.empty((batch, attrs["output_num_rows"], attrs["output_num_cols"]), dtype=np.float32)
    for i in range(batch):
        acc = a[i] @ b[i]  # float32 accumulate
        if transposed_out:
            res = gemm_epilogue(acc.T, bias, None if cc is None else cc[i].T, beta, epilogue, out_dtype, alpha).T
        else:
            res = gemm_epilogue(acc, bias, None if cc is None else cc[i], beta, epilogue, out_dtype, alpha)
        out[i] = res
    return out


# --------------------------------------------------------------------------- fused attention

def gemm_qkv(a: np.ndarray, b3: np.ndarray, bias3=None, *, dtype: int = BF16):
    """Three projections of one input, out_i = A . B_i (+ bias_i): what HGEMM_QKV_KERNEL /
    HGEMM_QKV_BIAS_KERNEL compute (xla/service/gpu/xetla/gemm/hgemm_impl.h:461-608: grid
    dimension 0 picks the weight slab b + k*n*id, the output out0/1/2 and the bias slab bias + n*id),
    fp32 accumulation and one rounding to the 16-bit type.  a [m,k], b3 [3,k,n], bias3 [3,n] or
    None, all already holding values representable in `dtype`; returns three float32 [m,n] arrays."""
    a = np.asarray(a, dtype=np.float32)
    b3 = np.asarray(b3, dtype=np.float32)
    outs = []
    for i in range(3):
        acc = a.astype(np.float64) @ b3[i].astype(np.float64)
        if bias3 is not None:
            acc = acc + np.asarray(bias3, dtype=np.float32)[i][None, :].astype(np.float64)
        outs.append(round_to(acc.astype(np.float32), dtype))
    return tuple(outs)


def fmha_forward(q, k, v, bias=None, *, head_scale: float, causal: bool = False, dtype: int = BF16,
                 round_p: bool = True):
    """fmha_forward_t (xla/service/gpu/xetla/sdp/fmha_forward.h:256-568), un-tiled.

    q [B,N,F,H], k/v [B,N,T,H] float32 arrays holding values already rounded to `dtype`;
    bias broadcastable to [B,N,F,T].  Per row: s = head_scale * q.k (fp32, :256-282), + bias,
    -inf where causal and t > f (top-left anchored, fmha_utils.h:45-96), softmax in fp32
    (:331-371), normalised P rounded to `dtype` before P.V (:364-382), O accumulated in fp32 and
    rounded once (:390-396).  Returns (O float32 [B,N,F,H], LSE float32 [B,N,F] = m + ln l, :433-450).
    """
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    B, N, F, H = q.shape
    T = k.shape[2]
    out = np.empty((B, N, F, H), np.float32)
    lse = np.empty((B, N, F), np.float32)
    if bias is not None:
        bias = np.broadcast_to(np.asarray(bias, np.float32), (B, N, F, T))
    mask = None
    if causal:
        mask = np.arange(T)[None, :] > np.arange(F)[:, None]
    for b in range(B):
        for n in range(N):
            s = (q[b, n] @ k[b, n].T) * np.float32(head_scale)
            if bias is not None:
                s = s + bias[b, n]
            if mask is not None:
                s = np.where(mask, -np.inf, s).astype(np.float32)
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True, dtype=np.float32)
            pn = p / l
            if round_p:
                pn = round_to(pn, dtype)
            out[b, n] = round_to(pn @ v[b, n], dtype)
            lse[b, n] = (m + np.log(l))[:, 0]
    return out, lse


def fmha_backward(q, k, v, out, grad_out, lse, bias=None, *, head_scale: float, causal: bool = False,
                  dtype: int = BF16, round_p: bool = True):
    """fmha_backward_t (xla/service/gpu/xetla/sdp/fmha_backward.h), un-tiled.

    q, out, grad_out [B,N,F,H]; k, v [B,N,T,H]; lse [B,N,F] as the forward returns it; bias
    broadcastable to [B,N,F,T].  D = rowsum(dO * O) in fp32 (:182-222); P is recomputed from the
    saved row statistic, P = exp(head_scale * Q.K^T + bias - lse) (:489-545), with the causal
    mask of the forward; dP = dO.V^T, dS = P * (dP - D) (:556-584); P and dS are rounded to
    `dtype` where the kernel stores them as matmul operands; dV = P^T.dO, dK = head_scale *
    dS^T.Q (:671), dQ = head_scale * dS.K accumulated in fp32 and rounded once (:842).
    Returns (dQ, dK, dV) float32 holding values rounded to `dtype`."""
    q, k, v = (np.asarray(a, np.float32) for a in (q, k, v))
    out, grad_out = np.asarray(out, np.float32), np.asarray(grad_out, np.float32)
    lse = np.asarray(lse, np.float32)
    B, N, F, H = q.shape
    T = k.shape[2]
    dq = np.empty_like(q)
    dk = np.empty_like(k)
    dv = np.empty_like(v)
    if bias is not None:
        bias = np.broadcast_to(np.asarray(bias, np.float32), (B, N, F, T))
    mask = (np.arange(T)[None, :] > np.arange(F)[:, None]) if causal else None
    scale = np.float32(head_scale)
    for b in range(B):
        for n in range(N):
            delta = (grad_out[b, n] * out[b, n]).sum(axis=1, keepdims=True, dtype=np.float32)
            s = (q[b, n] @ k[b, n].T) * scale
            if bias is not None:
                s = s + bias[b, n]
            p = np.exp(s - lse[b, n][:, None]).astype(np.float32)
            if mask is not None:
                p = np.where(mask, np.float32(0), p)
            dp = grad_out[b, n] @ v[b, n].T
            ds = p * (dp - delta)
            if round_p:
                p, ds = round_to(p, dtype), round_to(ds, dtype)
            dv[b, n] = round_to(p.T @ grad_out[b, n], dtype)
            dk[b, n] = round_to((ds.T @ q[b, n]) * scale, dtype)
            dq[b, n] = round_to((ds @ k[b, n]) * scale, dtype)
    return dq, dk, dv


# --------------------------------------------------------------------------- fp8 scaled GEMM

def fp8_scaled_gemm(a_codes, a_dtype: int, a_scale: float, b_codes, b_dtype: int, b_scale: float,
                    out_dtype: int = BF16) -> np.ndarray:
    """float32 matmul of the dequantised operands (the reference result the fp8 config names):
    (decode(Aq)/sa) @ (decode(Bq)/sb), rounded to out_dtype.  a_codes [M,K], b_codes [K,N]."""
    a = fp8_decode(a_codes, a_dtype) / np.float32(a_scale)
    b = fp8_decode(b_codes, b_dtype) / np.float32(b_scale)
    return round_to(a @ b, out_dtype)


def fp8_scaled_gemm_kernel_order(a_codes, a_dtype, a_scale, b_codes, b_dtype, b_scale, out_dtype=BF16):
    """Same quantity in the order the kernel evaluates it: accumulate the raw fp8 products in
    fp32, multiply by 1/(sa*sb) once, round.  Used to separate accumulation-order noise from bugs."""
    acc = fp8_decode(a_codes, a_dtype) @ fp8_decode(b_codes, b_dtype)
    return round_to(acc * np.float32((1.0 / a_scale) * (1.0 / b_scale)), out_dtype)


# --------------------------------------------------------------------------- tolerance

def check_close(actual, expected, *, rtol: float, atol: float, what: str = "") -> float:
    """|actual - expected| <= atol + rtol*|expected| elementwise; raises AssertionError with the
    worst offender.  Returns the max absolute error."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    if actual.shape != expected.shape:
        raise AssertionError(f"{what}: shape {actual.shape} != {expected.shape}")
    err = np.abs(actual - expected)
    bound = atol + rtol * np.abs(expected)
    bad = ~(err <= bound)  # catches NaN too
    if bad.any():
        idx = np.unravel_index(np.argmax(np.where(bad, err, -1)), err.shape)
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{err.size} elements out of tolerance (rtol={rtol}, atol={atol}); "
            f"worst at {idx}: got {actual[idx]!r}, want {expected[idx]!r}")
    return float(err.max()) if err.size else 0.0
