"""GPU parity: fp8 (e4m3 / e5m2) scaled GEMM against the fp32 matmul of the dequantised
operands.  Tolerance: the bf16 output tolerance (rtol 2e-2, atol 2e-2 x output RMS) — the
kernel's only error sources are fp32 accumulation order and the final rounding."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def f32(t):
    return t.float().cpu().numpy()


ODT = {torch.float8_e4m3fn: 3, torch.float8_e5m2: 4}


def test_golden_vectors(pkg, orc, cuda):
    g = np.load(os.path.join(GOLDEN, "fp8.npz"))
    for name, dt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        aq = torch.from_numpy(g[f"aq_{name}"].copy()).view(dt).to(cuda)
        bq = torch.from_numpy(g[f"bq_{name}"].copy()).view(dt).to(cuda)
        out = pkg.gemm_fp8(aq, bq, 1.0 / float(g[f"sa_{name}"]), 1.0 / float(g[f"sb_{name}"]), out_dtype=torch.float32)
        np.testing.assert_allclose(f32(out), g[f"ref_{name}"], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("shape", [(128, 128, 256), (256, 512, 384), (130, 144, 208), (16, 4096, 1024)])
@pytest.mark.parametrize("b_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_scaled_gemm(pkg, orc, cuda, shape, b_dtype, lb):
    M, K, N = shape
    g = torch.Generator().manual_seed(M + 3 * K + 5 * N)
    a32 = torch.randn(M, K, generator=g)
    b32 = torch.randn(K, N, generator=g)
    aq, sa = pkg.quantize_fp8(a32, torch.float8_e4m3fn)
    bq, sb = pkg.quantize_fp8(b32, b_dtype)
    bd = bq.to(cuda) if lb == "row" else bq.to(cuda).t().contiguous().t()
    out = pkg.gemm_fp8(aq.to(cuda), bd, 1.0 / sa, 1.0 / sb)
    want = orc.fp8_scaled_gemm(aq.view(torch.uint8).numpy(), orc.F8E4M3, sa, bq.view(torch.uint8).numpy(), ODT[b_dtype], sb)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2 * rms, what=f"fp8 {shape} {b_dtype} B {lb}")


@pytest.mark.parametrize("b_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_scaled_gemm_on_cta_pairs(pkg, orc, cuda, b_dtype, lb):
    """A shape that runs on the CTA-pair kernel (odd row-block count, ragged N and K)."""
    M, K, N = 1280 + 128, 400, 4608 + 48
    g = torch.Generator().manual_seed(103)
    aq, sa = pkg.quantize_fp8(torch.randn(M, K, generator=g), torch.float8_e4m3fn)
    bq, sb = pkg.quantize_fp8(torch.randn(K, N, generator=g), b_dtype)
    bd = bq.to(cuda) if lb == "row" else bq.to(cuda).t().contiguous().t()
    out = pkg.gemm_fp8(aq.to(cuda), bd, 1.0 / sa, 1.0 / sb)
    want = orc.fp8_scaled_gemm(aq.view(torch.uint8).numpy(), orc.F8E4M3, sa, bq.view(torch.uint8).numpy(), ODT[b_dtype], sb)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2 * rms, what=f"fp8 pair B {lb}")


def test_e5m2_lhs_and_bias_epilogue(pkg, orc, cuda):
    M, K, N = 192, 256, 128
    g = torch.Generator().manual_seed(5)
    aq, sa = pkg.quantize_fp8(torch.randn(M, K, generator=g), torch.float8_e5m2)
    bq, sb = pkg.quantize_fp8(torch.randn(K, N, generator=g), torch.float8_e4m3fn)
    bias = torch.randn(N, generator=g).bfloat16()
    out = pkg.gemm_fp8(aq.to(cuda), bq.to(cuda), 1.0 / sa, 1.0 / sb, bias=bias.to(cuda), epilogue="BIAS_RELU")
    acc = (orc.fp8_decode(aq.view(torch.uint8).numpy(), orc.F8E5M2) / np.float32(sa)) @ \
          (orc.fp8_decode(bq.view(torch.uint8).numpy(), orc.F8E4M3) / np.float32(sb))
    want = orc.gemm_epilogue(acc, f32(bias), None, 0.0, "BIAS_RELU", orc.BF16)
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2 * float(np.sqrt(np.mean(want ** 2))) + 1e-3, what="e5m2 lhs")


def test_exact_integers_at_full_size(pkg, cuda):
    """Configuration 3 at full size (16384x8192 . 8192x8192): small integers are exact in fp8 and
    their dot products exact in fp32, so the kernel must reproduce them bit for bit; checked on a
    strip of rows, plus additivity over B (a size-independent property) on the whole output."""
    M, K, N = 16384, 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(41)
    a = torch.randint(-2, 3, (M, K), generator=g, device=cuda).float().to(torch.float8_e4m3fn)
    b1 = torch.randint(-1, 2, (K, N), generator=g, device=cuda).float()
    b2 = torch.randint(-1, 2, (K, N), generator=g, device=cuda).float()
    o1 = pkg.gemm_fp8(a, b1.to(torch.float8_e4m3fn), 1.0, 1.0, out_dtype=torch.float32)
    o2 = pkg.gemm_fp8(a, b2.to(torch.float8_e5m2), 1.0, 1.0, out_dtype=torch.float32)
    o12 = pkg.gemm_fp8(a, (b1 + b2).to(torch.float8_e4m3fn), 1.0, 1.0, out_dtype=torch.float32)
    assert torch.equal(o12, o1 + o2)
    rows = torch.tensor([0, 127, 128, 8191, 16383], device=cuda)
    assert torch.equal(o1[rows], a[rows].float() @ b1)


@pytest.mark.parametrize("b_dtype", [torch.float8_e4m3fn, torch.float8_e5m2], ids=["e4m3", "e5m2"])
def test_full_size_on_the_configuration_inputs(pkg, orc, cuda, b_dtype):
    """Configuration 3 on its own inputs: A[16384,8192], B[8192,8192] ~ N(0,1) in fp32, quantised per
    tensor with scale = max_finite / amax (A e4m3, B e4m3 or e5m2), bf16 out.  The oracle recomputes
    two 128-row strips (first and last) over all 8192 columns from the dequantised operands."""
    M, K, N = 16384, 8192, 8192
    g = torch.Generator().manual_seed(73)
    aq, sa = pkg.quantize_fp8(torch.randn(M, K, generator=g), torch.float8_e4m3fn)
    bq, sb = pkg.quantize_fp8(torch.randn(K, N, generator=g), b_dtype)
    out = pkg.gemm_fp8(aq.to(cuda), bq.to(cuda), 1.0 / sa, 1.0 / sb)
    a_codes, b_codes = aq.view(torch.uint8).numpy(), bq.view(torch.uint8).numpy()
    for r0 in (0, M - 128):
        want = orc.fp8_scaled_gemm(a_codes[r0:r0 + 128], orc.F8E4M3, sa, b_codes, ODT[b_dtype], sb)
        rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        orc.check_close(f32(out[r0:r0 + 128]), want, rtol=2e-2, atol=2e-2 * rms, what=f"C3 rows {r0}..{r0 + 127}")


def test_bf16_operands_rejected_by_fp8_entry(pkg, cuda):
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm_fp8(x, x, 1.0, 1.0)
    assert e.value.status == pkg.IXK_INVALID_ARGUMENT
