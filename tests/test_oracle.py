"""CPU: the oracle against the committed golden vectors (made by torch's CPU kernels) and
against independent implementations of the element formats."""
import os

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def test_bf16_rounding_matches_torch(orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10 ** rng.uniform(-30, 30, 20000).astype(np.float32),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, np.inf, -np.inf], np.float32)])
    want = torch.from_numpy(x).bfloat16().view(torch.uint16).numpy()
    assert np.array_equal(orc.bf16_bits(x), want)
    assert np.array_equal(orc.round_bf16(x), torch.from_numpy(x).bfloat16().float().numpy())
    assert np.isnan(orc.round_bf16(np.array([np.nan], np.float32))[0])


def test_fp8_decode_all_codes(orc):
    import ml_dtypes
    codes = np.arange(256, dtype=np.uint8)
    for dt, ml in ((orc.F8E4M3, ml_dtypes.float8_e4m3fn), (orc.F8E5M2, ml_dtypes.float8_e5m2)):
        want = codes.view(ml).astype(np.float32)
        got = orc.fp8_decode(codes, dt)
        finite = np.isfinite(want)
        assert np.array_equal(got[finite], want[finite])


def test_fp8_saturating_cast_matches_golden_sweep(orc):
    g = load("fp8.npz")
    for name, dt in (("e4m3", orc.F8E4M3), ("e5m2", orc.F8E5M2)):
        got = orc.fp8_encode_sat(g["sweep"], dt)
        want = g[f"sweep_{name}"]
        # +0 / -0 carry the sign bit in both
        assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]


def test_fp8_cast_matches_ml_dtypes_in_range(orc):
    import ml_dtypes
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(50000) * 100).astype(np.float32)
    x = np.clip(x, -448, 448)
    assert np.array_equal(orc.fp8_encode_sat(x, orc.F8E4M3), x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8))
    y = (rng.standard_normal(50000) * 10000).astype(np.float32)
    y = np.clip(y, -57344, 57344)
    assert np.array_equal(orc.fp8_encode_sat(y, orc.F8E5M2), y.astype(ml_dtypes.float8_e5m2).view(np.uint8))


def test_quantize_fp8_uses_full_range(orc):
    x = np.array([[0.5, -2.0], [1.0, 0.25]], np.float32)
    codes, scale = orc.quantize_fp8(x, orc.F8E4M3)
    assert scale == pytest.approx(224.0)
    assert np.array_equal(orc.fp8_decode(codes, orc.F8E4M3), np.array([[112, -448], [224, 56]], np.float32))


def test_gelu_matches_torch(orc):
    x = torch.linspace(-12, 12, 10001)
    want = torch.nn.functional.gelu(x, approximate="tanh").numpy()
    np.testing.assert_allclose(orc.gelu_tanh(x.numpy()), want, rtol=1e-5, atol=1e-6)


def test_gemm_golden(orc):
    g = load("gemm_bf16.npz")
    x, w, b, c = (orc.bf16_to_f32(g[k]) for k in ("x", "w", "b", "c"))
    acc = x @ w
    for key, epi, beta, cc in (("out_bias_gelu", "BIAS_GELU", 0.0, None), ("out_bias_beta", "BIAS", 0.5, c),
                               ("out_relu", "RELU", 0.0, None)):
        got = orc.gemm_epilogue(acc, b, cc, beta, epi, orc.BF16)
        want = orc.bf16_to_f32(g[key])
        # identical up to one bf16 ulp where the two fp32 evaluations straddle a rounding boundary
        orc.check_close(got, want, rtol=2 ** -7, atol=1e-6, what=key)
        assert np.mean(got == want) > 0.99


def _attrs(M, K, N, lo, ro, oo, beta=0.0, lda=None, ldb=None, ldo=None):
    return {
        "lhs_order": lo, "lhs_num_rows": M, "lhs_num_cols": K, "lhs_batch_stride": M * K,
        "lhs_leading_dim_stride": lda or (K if lo == 0 else M),
        "rhs_order": ro, "rhs_num_rows": K, "rhs_num_cols": N, "rhs_batch_stride": K * N,
        "rhs_leading_dim_stride": ldb or (N if ro == 0 else K),
        "output_order": oo, "output_num_rows": M, "output_num_cols": N, "output_batch_stride": M * N,
        "output_leading_dim_stride": ldo or (N if oo == 0 else M),
        "batch_size": 1, "alpha": 1.0, "beta": beta,
    }


@pytest.mark.parametrize("lo", [0, 1])
@pytest.mark.parametrize("ro", [0, 1])
def test_gemm_custom_call_layouts(orc, lo, ro):
    rng = np.random.default_rng(2)
    M, K, N = 5, 7, 3
    a = orc.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    b = orc.round_bf16(rng.standard_normal((K, N)).astype(np.float32))
    a_store = a if lo == 0 else np.ascontiguousarray(a.T)
    b_store = b if ro == 0 else np.ascontiguousarray(b.T)
    got = orc.gemm_custom_call(_attrs(M, K, N, lo, ro, 0), a_store, b_store, None, None, "DEFAULT", orc.F32)
    np.testing.assert_allclose(got[0], a @ b, rtol=1e-6, atol=1e-6)


def test_gemm_custom_call_col_major_output_bias_runs_along_rows(orc):
    """With a column-major output the call is rewritten as D^T = B^T.A^T and the bias vector
    follows the columns of the rewritten problem (onednn_matmul_utils.cc:520-530, :363-365)."""
    rng = np.random.default_rng(3)
    M, K, N = 4, 6, 5
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    bias = rng.standard_normal(M).astype(np.float32)
    got = orc.gemm_custom_call(_attrs(M, K, N, 0, 0, 1), a, b, None, bias, "BIAS", orc.F32)
    np.testing.assert_allclose(got[0], a @ b + bias[:, None], rtol=1e-6, atol=1e-6)


def test_gemm_custom_call_alpha_aux_and_unknown_epilogue(orc):
    a = np.zeros((2, 2), np.float32)
    with pytest.raises(NotImplementedError):      # one result only: the reference's answer for *_AUX
        orc.gemm_custom_call(_attrs(2, 2, 2, 0, 0, 0), a, a, None, None, "GELU_AUX", orc.F32)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 6)).astype(np.float32)
    w = rng.standard_normal((6, 3)).astype(np.float32)
    scaled = _attrs(4, 6, 3, 0, 0, 0)
    scaled["alpha"] = -0.5
    got = orc.gemm_custom_call(scaled, x, w, None, None, "DEFAULT", orc.F32)
    np.testing.assert_allclose(got[0], -0.5 * (x @ w), rtol=1e-6, atol=1e-6)
    b = rng.standard_normal(3).astype(np.float32)
    d, aux = orc.gemm_epilogue(x @ w, b, None, 0.0, "BIAS_GELU_AUX", orc.F32, alpha=2.0, with_aux=True)
    np.testing.assert_allclose(aux, 2.0 * (x @ w) + b, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(d, orc.gelu_tanh(aux), rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError):
        orc.gemm_custom_call(_attrs(2, 2, 2, 0, 0, 0), a, a, None, None, "SILU", orc.F32)


def test_fmha_golden_bf16(orc):
    g = load("fmha_bf16.npz")
    q, k, v, bias = (orc.bf16_to_f32(g[n]) for n in ("q", "k", "v", "bias"))
    scale = float(g["scale"])
    o, _ = orc.fmha_forward(q, k, v, None, head_scale=scale, causal=True, round_p=False)
    orc.check_close(o, orc.round_bf16(g["o_causal"]), rtol=2 ** -7, atol=1e-5, what="causal")
    o, lse = orc.fmha_forward(q, k, v, bias, head_scale=scale, causal=False, round_p=False)
    orc.check_close(o, orc.round_bf16(g["o_bias"]), rtol=2 ** -7, atol=1e-5, what="bias")
    np.testing.assert_allclose(lse, g["lse_bias"], rtol=1e-5, atol=1e-5)
    # the reference's rounding of P to bf16 moves the result by less than the test tolerance
    o_rp, _ = orc.fmha_forward(q, k, v, bias, head_scale=scale, causal=False, round_p=True)
    orc.check_close(o_rp, g["o_bias"], rtol=2e-2, atol=2e-2, what="bias, P rounded")


def test_fmha_golden_f16_ragged(orc):
    g = load("fmha_f16_ragged.npz")
    q, k, v = (g[n].view(np.float16).astype(np.float32) for n in ("q", "k", "v"))
    o, _ = orc.fmha_forward(q, k, v, None, head_scale=float(g["scale"]), dtype=orc.F16, round_p=False)
    orc.check_close(o, orc.round_f16(g["o"]), rtol=2 ** -10, atol=1e-5, what="f16 ragged")


def test_fmha_causal_is_top_left_anchored(orc):
    """F != T: keys t > f are masked (fmha_utils.h:63), so query 0 sees exactly key 0."""
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 1, 3, 8)).astype(np.float32)
    k = rng.standard_normal((1, 1, 9, 8)).astype(np.float32)
    v = rng.standard_normal((1, 1, 9, 8)).astype(np.float32)
    o, lse = orc.fmha_forward(q, k, v, None, head_scale=1.0, causal=True, dtype=orc.F32, round_p=False)
    np.testing.assert_allclose(o[0, 0, 0], v[0, 0, 0], rtol=1e-6)
    assert lse[0, 0, 0] == pytest.approx(float(q[0, 0, 0] @ k[0, 0, 0]), rel=1e-5)


def test_fp8_gemm_golden(orc):
    g = load("fp8.npz")
    for name, dt in (("e4m3", orc.F8E4M3), ("e5m2", orc.F8E5M2)):
        aq, sa = orc.quantize_fp8(g["a"], dt)
        bq, sb = orc.quantize_fp8(g["b"], dt)
        assert np.array_equal(aq, g[f"aq_{name}"]) and np.array_equal(bq, g[f"bq_{name}"])
        assert sa == pytest.approx(float(g[f"sa_{name}"])) and sb == pytest.approx(float(g[f"sb_{name}"]))
        got = orc.fp8_scaled_gemm(aq, dt, sa, bq, dt, sb, orc.F32)
        np.testing.assert_allclose(got, g[f"ref_{name}"], rtol=1e-5, atol=1e-5)
        alt = orc.fp8_scaled_gemm_kernel_order(aq, dt, sa, bq, dt, sb, orc.F32)
        np.testing.assert_allclose(alt, got, rtol=1e-5, atol=1e-5)


def test_check_close_reports(orc):
    with pytest.raises(AssertionError, match="out of tolerance"):
        orc.check_close(np.array([1.0, 2.0]), np.array([1.0, 2.5]), rtol=0.0, atol=0.1, what="x")
    with pytest.raises(AssertionError):
        orc.check_close(np.array([np.nan]), np.array([0.0]), rtol=1.0, atol=1.0)
    assert orc.check_close(np.array([1.0]), np.array([1.05]), rtol=0.0, atol=0.1) == pytest.approx(0.05)


def test_qkv_gemm_matches_three_separate_products(orc):
    """The fused form must equal the three separate matmuls it replaces
    (example/qkv_fusion/test_qkv_fusion.py:24-35 compares exactly those)."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(5, 96, generator=g).bfloat16()
    w = (torch.randn(3, 96, 40, generator=g) / 10).bfloat16()
    b = torch.randn(3, 40, generator=g).bfloat16()
    got = orc.gemm_qkv(x.float().numpy(), w.float().numpy(), b.float().numpy(), dtype=orc.BF16)
    for i in range(3):
        want = (x.float() @ w[i].float() + b[i].float()).bfloat16().float().numpy()
        assert np.max(np.abs(got[i] - want)) <= 2e-2 * max(1.0, float(np.max(np.abs(want))))


def test_fmha_backward_matches_autograd(orc):
    """The backward oracle (P recomputed from the saved log-sum-exp, dS = P * (dP - D)) against
    torch autograd of plain fp32 attention, with the operand roundings switched off."""
    import math
    import torch
    g = torch.Generator().manual_seed(5)
    B, N, F, T, H = 2, 2, 70, 90, 32
    for causal, with_bias in ((False, False), (True, False), (False, True)):
        q = torch.randn(B, N, F, H, generator=g, requires_grad=True)
        k = torch.randn(B, N, T, H, generator=g, requires_grad=True)
        v = torch.randn(B, N, T, H, generator=g, requires_grad=True)
        bias = torch.randn(B, 1, F, T, generator=g) if with_bias else None
        do = torch.randn(B, N, F, H, generator=g)
        scale = 1.0 / math.sqrt(H)
        s = (q @ k.transpose(-1, -2)) * scale
        if bias is not None:
            s = s + bias
        if causal:
            s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(F)[:, None], float("-inf"))
        out = torch.softmax(s, dim=-1) @ v
        out.backward(do)
        lse = torch.logsumexp(s, dim=-1)
        dq, dk, dv = orc.fmha_backward(q.detach().numpy(), k.detach().numpy(), v.detach().numpy(), out.detach().numpy(),
                                       do.numpy(), lse.detach().numpy(), None if bias is None else bias.numpy(),
                                       head_scale=scale, causal=causal, dtype=orc.F32, round_p=False)
        for got, want in ((dq, q.grad), (dk, k.grad), (dv, v.grad)):
            np.testing.assert_allclose(got, want.numpy(), rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("fname", ["fmha_bwd_bf16.npz", "fmha_bwd_h256_bf16.npz"])
def test_fmha_backward_golden(orc, fname):
    """Backward oracle (bf16 operand rounding on) against autograd gradients of fp32 attention,
    at head size 64 and at 256."""
    g = np.load(os.path.join(GOLDEN, fname))
    q, k, v, do = (orc.bf16_to_f32(g[n]) for n in ("q", "k", "v", "do"))
    bias = orc.bf16_to_f32(g["bias"])
    for name in ("causal", "bias"):
        dq, dk, dv = orc.fmha_backward(q, k, v, g[f"o_{name}"], do, g[f"lse_{name}"],
                                       bias if name == "bias" else None, head_scale=float(g["scale"]),
                                       causal=name == "causal")
        for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            orc.check_close(got, g[f"{key}_{name}"], rtol=2e-2, atol=2e-2, what=f"golden {key} {name}")


def test_tf32_and_int8_models(orc):
    x = np.array([1.0 + 2.0 ** -11, 1.0 + 2.0 ** -10, -3.0 - 2.0 ** -12, 1e-30], np.float32)
    t = orc.tf32_operand(x, "truncate")
    r = orc.tf32_operand(x, "round")
    assert t[0] == 1.0 and t[1] == np.float32(1.0 + 2.0 ** -10) and t[2] == -3.0
    assert r[0] == np.float32(1.0 + 2.0 ** -10) and r[2] == -3.0        # half an ulp rounds away; a quarter does not
    assert np.all((t.view(np.uint32) & 0x1FFF) == 0) and np.all((r.view(np.uint32) & 0x1FFF) == 0)
    a = np.full((1, 4), -128, np.int8)
    assert orc.gemm_s8(a, a.T)[0, 0] == 4 * 128 * 128
    big = np.full((1, 140000), 127, np.int8)        # 140000 * 127^2 > 2^31: wraps like the hardware's 32-bit sum
    assert orc.gemm_s8(big, big.T)[0, 0] == np.int64(140000 * 127 * 127).astype(np.int32)
