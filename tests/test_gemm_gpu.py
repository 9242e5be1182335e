"""GPU parity: the tcgen05 GEMM + fused epilogue, through the C ABI, against the CPU oracle.

Tolerance (stated by the task for this path): bf16 results within rtol 2e-2 / atol 2e-2 of the
fp32-accumulated reference; fp16 outputs are held to 2e-3, fp32 outputs to 1e-3 (the only
differences are accumulation order and the final rounding)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = {torch.bfloat16: (2e-2, 2e-2), torch.float16: (2e-3, 2e-3), torch.float32: (1e-3, 1e-3)}


def f32(t):
    return t.float().cpu().numpy()


def as_layout(t, order):
    """Same logical matrix, row- or column-major storage."""
    return t if order == "row" else t.t().contiguous().t()


def test_golden_vectors(pkg, orc, cuda):
    g = np.load(os.path.join(GOLDEN, "gemm_bf16.npz"))
    x, w, b, c = (torch.from_numpy(g[k].copy()).view(torch.bfloat16).to(cuda) for k in ("x", "w", "b", "c"))
    for key, epi, beta in (("out_bias_gelu", "BIAS_GELU", 0.0), ("out_bias_beta", "BIAS", 0.5), ("out_relu", "RELU", 0.0)):
        out = pkg.gemm(x, w, bias=b if "BIAS" in epi else None, c=c if beta else None, beta=beta, epilogue=epi)
        orc.check_close(f32(out), orc.bf16_to_f32(g[key]), rtol=2e-2, atol=2e-2, what=key)


@pytest.mark.parametrize("shape", [(128, 64, 256), (256, 512, 384), (200, 136, 328), (1, 64, 8), (300, 72, 40),
                                   (64, 4096, 512), (129, 264, 520)])
@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_layouts_and_ragged_shapes(pkg, orc, cuda, shape, la, lb):
    M, K, N = shape
    if (la == "col" and M % 8) or (lb == "row" and N % 8) or K % 8:
        pytest.skip("pitch not a multiple of 16 bytes: rejected, see test_unaligned_pitch_is_rejected")
    g = torch.Generator().manual_seed(M * 131 + K * 17 + N)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(K, N, generator=g) * 0.1).bfloat16()
    b = torch.randn(N, generator=g).bfloat16()
    c = torch.randn(M, N, generator=g).bfloat16()
    out = pkg.gemm(as_layout(x.to(cuda), la), as_layout(w.to(cuda), lb), bias=b.to(cuda), c=c.to(cuda), beta=0.5,
                   epilogue="BIAS_GELU")
    want = orc.gemm_epilogue(f32(x) @ f32(w), f32(b), f32(c), 0.5, "BIAS_GELU", orc.BF16)
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2, what=f"{shape} A {la} B {lb}")


@pytest.mark.parametrize("epilogue", ["DEFAULT", "RELU", "GELU", "BIAS", "BIAS_RELU", "BIAS_GELU"])
@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                             (torch.bfloat16, torch.float32), (torch.float16, torch.float32)])
def test_epilogues_and_type_triples(pkg, orc, cuda, epilogue, dtype, out_dtype):
    """The six epilogues of the reference enum that have a kernel, over RunGemm's 16-bit type
    triples (onednn_matmul_utils.cc:605-608)."""
    M, K, N = 192, 160, 136
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(K, N, generator=g) * 0.1).to(dtype)
    b = torch.randn(N, generator=g).to(dtype)
    out = pkg.gemm(x.to(cuda), w.to(cuda), bias=b.to(cuda) if "BIAS" in epilogue else None, epilogue=epilogue,
                   out_dtype=out_dtype)
    assert out.dtype == out_dtype
    odt = {torch.bfloat16: orc.BF16, torch.float16: orc.F16, torch.float32: orc.F32}[out_dtype]
    want = orc.gemm_epilogue(f32(x) @ f32(w), f32(b), None, 0.0, epilogue, odt)
    rtol, atol = TOL[out_dtype]
    orc.check_close(f32(out), want, rtol=rtol, atol=atol, what=epilogue)


@pytest.mark.parametrize("beta", [1.0, -0.75])
def test_beta_residual_in_place(pkg, orc, cuda, beta):
    """XLA aliases C with the output when beta != 0 (sycl_custom_call.cc:188-195); any beta is honoured."""
    M, K, N = 130, 96, 264
    g = torch.Generator().manual_seed(11)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(K, N, generator=g) * 0.1).bfloat16()
    c = torch.randn(M, N, generator=g).bfloat16()
    d = c.to(cuda).clone()
    pkg.gemm(x.to(cuda), w.to(cuda), c=d, beta=beta, out=d)
    want = orc.gemm_epilogue(f32(x) @ f32(w), None, f32(c), beta, "DEFAULT", orc.BF16)
    orc.check_close(f32(d), want, rtol=2e-2, atol=2e-2, what=f"beta={beta}")


def test_batched_and_padded_pitch(pkg, orc, cuda):
    g = torch.Generator().manual_seed(13)
    x_store = torch.randn(3, 100, 80, generator=g).half()
    x = x_store[:, :, :72]                      # pitch 80, 72 used
    w = torch.randn(3, 72, 96, generator=g).half()
    out = pkg.gemm(x.to(cuda)[:, :, :72] if False else x_store.to(cuda)[:, :, :72], w.to(cuda), out_dtype=torch.float32)
    want = np.einsum("bmk,bkn->bmn", f32(x), f32(w))
    orc.check_close(f32(out), want, rtol=1e-3, atol=1e-3, what="batched")


def test_column_major_output_and_bias_direction(pkg, orc, cuda):
    """Column-major D is computed as D^T = B^T.A^T; the bias then runs along the original rows,
    exactly as the oracle's gemm_custom_call restates (onednn_matmul_utils.cc:520-530, :363-365)."""
    M, K, N = 104, 72, 96
    g = torch.Generator().manual_seed(17)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = torch.randn(K, N, generator=g).bfloat16()
    bias = torch.randn(M, generator=g).bfloat16()
    out = torch.empty(N, M, dtype=torch.bfloat16, device=cuda).t()   # logical [M, N], column-major
    attrs = pkg.gemm_attrs_for(x, w, out)
    pkg.run_gemm_custom_call(x.to(cuda), w.to(cuda), None, out, bias.to(cuda), None, attrs, "BIAS")
    want = orc.gemm_custom_call(attrs, f32(x), f32(w), None, f32(bias), "BIAS", orc.BF16)[0]
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2, what="col-major out")


def test_gemm_ut_shapes_col_major_b(pkg, orc, cuda):
    """Shapes of the reference's gemm_ut (test/jax_ut.patch:540-580): (1,256,128,8) and
    (1,1024,64,128) with B column-major, GELU epilogue, bf16 and fp16."""
    for (batch, M, K, N) in ((1, 256, 128, 8), (1, 1024, 64, 128)):
        for dtype, odt in ((torch.bfloat16, orc.BF16), (torch.float16, orc.F16)):
            g = torch.Generator().manual_seed(M + N)
            x = torch.randn(M, K, generator=g).to(dtype)
            w = torch.randn(K, N, generator=g).to(dtype)
            out = pkg.gemm(x.to(cuda), as_layout(w.to(cuda), "col"), epilogue="GELU")
            want = orc.gemm_epilogue(f32(x) @ f32(w), None, None, 0.0, "GELU", odt)
            rtol, atol = TOL[dtype]
            orc.check_close(f32(out), want, rtol=max(rtol, 4e-3), atol=max(atol, 2e-2), what=f"gemm_ut {M}x{K}x{N}")


def test_qkv_fusion_shape(pkg, orc, cuda):
    """example/qkv_fusion/test_qkv_fusion.py:37-51: fp16, m=4, k=n=4096, one activation against
    three weights — run as one [K,3N] GEMM; the reference holds it to atol=rtol=1e-3 on outputs of
    O(1) magnitude (weights scaled to keep them there)."""
    m, k, n = 4, 4096, 4096
    g = torch.Generator().manual_seed(23)
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(k, 3 * n, generator=g) / 64).half()
    out = pkg.gemm(x.to(cuda), w.to(cuda), out_dtype=torch.float32)
    want = f32(x) @ f32(w)
    orc.check_close(f32(out), want, rtol=1e-3, atol=1e-3, what="qkv")


@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                             (torch.bfloat16, torch.float32)])
def test_cta_pair_tiles(pkg, orc, cuda, monkeypatch, la, lb, dtype, out_dtype):
    """Shapes large enough for the CTA-pair kernel (256 x 256 tiles on two SMs): an odd number of
    row blocks (the last pair has an empty half), ragged N and K, every operand layout, bias +
    GELU + residual; the single-CTA kernel must give the same numbers on the same inputs."""
    M, K, N = 1152 + 40, 328, 4608 + 72
    g = torch.Generator().manual_seed(97)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(K, N, generator=g) * 0.1).to(dtype)
    b = torch.randn(N, generator=g).to(dtype)
    c = torch.randn(M, N, generator=g).to(out_dtype)
    run = lambda: pkg.gemm(as_layout(x.to(cuda), la), as_layout(w.to(cuda), lb), bias=b.to(cuda), c=c.to(cuda), beta=0.5,
                           epilogue="BIAS_GELU", out_dtype=out_dtype)
    out = run()
    odt = {torch.bfloat16: orc.BF16, torch.float16: orc.F16, torch.float32: orc.F32}[out_dtype]
    want = orc.gemm_epilogue(f32(x) @ f32(w), f32(b), f32(c), 0.5, "BIAS_GELU", odt)
    rtol, atol = TOL[out_dtype]
    orc.check_close(f32(out), want, rtol=max(rtol, 4e-3), atol=max(atol, 4e-3), what=f"pair A {la} B {lb}")
    monkeypatch.setenv("IXK_GEMM_PAIR", "0")
    single = run()
    assert torch.equal(out, single)   # same products in the same order: bit-identical


def test_cta_pair_batched(pkg, orc, cuda):
    B, M, K, N = 2, 768, 192, 3328
    g = torch.Generator().manual_seed(101)
    x = torch.randn(B, M, K, generator=g).bfloat16()
    w = (torch.randn(B, K, N, generator=g) * 0.1).bfloat16()
    out = pkg.gemm(x.to(cuda), w.to(cuda))
    for i in range(B):
        want = orc.gemm_epilogue(f32(x[i]) @ f32(w[i]), None, None, 0.0, "DEFAULT", orc.BF16)
        orc.check_close(f32(out[i]), want, rtol=2e-2, atol=2e-2, what=f"pair batch {i}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
@pytest.mark.parametrize("placement", ["stacked", "scattered"])
@pytest.mark.parametrize("shape", [(4, 4096, 4096), (300, 520, 200)], ids=lambda s: "x".join(map(str, s)))
def test_qkv_gemm_entry_point(pkg, orc, cuda, shape, placement, with_bias, dtype):
    """ixk_gemm_qkv: three projections of one input (hgemm_impl.h:461-608), at the reference test's
    shape (example/qkv_fusion/test_qkv_fusion.py:37-51) and at a ragged one; outputs either stacked
    in one buffer (one launch, projection = batch index) or scattered (three launches)."""
    m, k, n = shape
    g = torch.Generator().manual_seed(29)
    x = torch.randn(m, k, generator=g).to(dtype)
    w = (torch.randn(3, k, n, generator=g) / (k ** 0.5)).to(dtype)
    b = torch.randn(3, n, generator=g).to(dtype) if with_bias else None
    if placement == "stacked":
        outs = None
    else:
        outs = tuple(torch.full((m, n), float("nan"), dtype=dtype, device=cuda) for _ in range(3))
        outs = (outs[2], outs[0], outs[1])     # no common spacing
    got = pkg.gemm_qkv(x.to(cuda), w.to(cuda), bias=b.to(cuda) if with_bias else None, outs=outs)
    odt = orc.BF16 if dtype == torch.bfloat16 else orc.F16
    want = orc.gemm_qkv(f32(x), f32(w), f32(b) if with_bias else None, dtype=odt)
    rtol, atol = TOL[dtype]
    for i in range(3):
        orc.check_close(f32(got[i]), want[i], rtol=rtol, atol=atol, what=f"qkv out{i}")


def test_qkv_gemm_rejections(pkg, cuda):
    x = torch.zeros(8, 64, dtype=torch.float32, device=cuda)
    w = torch.zeros(3, 64, 64, dtype=torch.float32, device=cuda)
    with pytest.raises((pkg.IxkError, KeyError)):
        pkg.gemm_qkv(x, w)                       # fp32 operands: BF16 / F16 only
    x = torch.zeros(8, 68, dtype=torch.bfloat16, device=cuda)   # pitch 136 bytes: not a multiple of 16
    w = torch.zeros(3, 68, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm_qkv(x, w)
    assert e.value.status == pkg.IXK_UNIMPLEMENTED


def test_block_n_variants_agree(pkg, orc, cuda, monkeypatch):
    M, K, N = 384, 320, 768
    g = torch.Generator().manual_seed(29)
    x = torch.randn(M, K, generator=g).bfloat16().to(cuda)
    w = (torch.randn(K, N, generator=g) * 0.1).bfloat16().to(cuda)
    outs = []
    for bn in ("64", "128", "256"):
        monkeypatch.setenv("IXK_GEMM_BLOCK_N", bn)
        outs.append(f32(pkg.gemm(x, w)))
    monkeypatch.delenv("IXK_GEMM_BLOCK_N")
    want = orc.round_bf16(f32(x) @ f32(w))
    for o in outs:
        orc.check_close(o, want, rtol=2e-2, atol=2e-2, what="block_n")
    # same k-order in every variant → bitwise identical
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])


def test_repeatable(pkg, cuda):
    g = torch.Generator().manual_seed(31)
    x = torch.randn(512, 512, generator=g).bfloat16().to(cuda)
    w = torch.randn(512, 1024, generator=g).bfloat16().to(cuda)
    a = pkg.gemm(x, w, epilogue="GELU")
    b = pkg.gemm(x, w, epilogue="GELU")
    assert torch.equal(a, b)


def test_linearity_at_full_size(pkg, cuda):
    """Configuration 1 at full size (8192x4096 . 4096x16384): too large for the CPU oracle in a
    test, so check a size-independent property — A.(B1 + B2) == A.B1 + A.B2 with operands chosen so
    every product and sum is exact in bf16/fp32 — plus a strip against the oracle's formula."""
    M, K, N = 8192, 4096, 16384
    g = torch.Generator(device="cuda").manual_seed(37)
    x = torch.randint(-2, 3, (M, K), generator=g, device=cuda).bfloat16()
    w1 = torch.randint(-2, 3, (K, N), generator=g, device=cuda).bfloat16()
    w2 = torch.randint(-2, 3, (K, N), generator=g, device=cuda).bfloat16()
    o1 = pkg.gemm(x, w1, out_dtype=torch.float32)
    o2 = pkg.gemm(x, w2, out_dtype=torch.float32)
    o12 = pkg.gemm(x, (w1 + w2), out_dtype=torch.float32)
    assert torch.equal(o12, o1 + o2)            # integers below 2^24: exact in fp32
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191], device=cuda)
    want = x[rows].float() @ w1.float()
    assert torch.equal(o1[rows], want)


def test_full_size_on_the_configuration_inputs(pkg, orc, cuda):
    """Configuration 1 on its own inputs and epilogue: X[8192,4096] ~ N(0,1), W[4096,16384] ~ N(0,0.02),
    bias ~ N(0,0.02), BIAS_GELU, bf16 out.  The oracle recomputes three 128-row blocks (first, one
    from the middle of a tile band, last) over all 16384 columns."""
    M, K, N = 8192, 4096, 16384
    g = torch.Generator().manual_seed(71)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(K, N, generator=g) * 0.02).bfloat16()
    b = (torch.randn(N, generator=g) * 0.02).bfloat16()
    out = pkg.gemm(x.to(cuda), w.to(cuda), bias=b.to(cuda), epilogue="BIAS_GELU")
    w32, b32 = f32(w), f32(b)
    for r0 in (0, 4480, M - 128):
        want = orc.gemm_epilogue(f32(x[r0:r0 + 128]) @ w32, b32, None, 0.0, "BIAS_GELU", orc.BF16)
        orc.check_close(f32(out[r0:r0 + 128]), want, rtol=2e-2, atol=2e-2, what=f"C1 rows {r0}..{r0 + 127}")


@pytest.mark.parametrize("alpha,beta", [(2.0, 0.0), (-0.5, 1.0), (0.25, -1.5)])
@pytest.mark.parametrize("shape", [(300, 136, 520), (2048, 512, 4096), (64, 4096, 3072)])
def test_alpha_scales_the_product_before_bias_and_residual(pkg, orc, cuda, shape, alpha, beta):
    """D = act(alpha*A.B + bias + beta*C) for any alpha (the reference CHECKs alpha == 1,
    onednn_matmul_utils.cc:438): single-CTA tiles, CTA pairs and the split-K path."""
    M, K, N = shape
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(K, N, generator=g) * 0.05).bfloat16()
    b = torch.randn(N, generator=g).bfloat16()
    c = torch.randn(M, N, generator=g).bfloat16()
    xd, wd = x.to(cuda), w.to(cuda)
    need = pkg.gemm_workspace_bytes(xd, wd)
    ws = torch.empty(need, dtype=torch.uint8, device=cuda) if need else None
    out = pkg.gemm(xd, wd, bias=b.to(cuda), c=c.to(cuda) if beta else None, beta=beta, alpha=alpha, epilogue="BIAS_GELU",
                   workspace=ws)
    want = orc.gemm_epilogue(f32(x) @ f32(w), f32(b), f32(c), beta, "BIAS_GELU", orc.BF16, alpha=alpha)
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2, what=f"alpha {alpha} beta {beta} {shape}")


@pytest.mark.parametrize("epilogue", ["GELU_AUX", "BIAS_GELU_AUX"])
@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32)])
@pytest.mark.parametrize("order", ["row", "col"])
def test_auxiliary_output_epilogues(pkg, orc, cuda, epilogue, dtype, out_dtype, order):
    """GELU_AUX / BIAS_GELU_AUX (onednn_matmul_utils.h:42-43): D = gelu(z) and the pre-activation z
    as a second result, for a small and a CTA-pair-sized problem, row- and column-major output."""
    for (M, K, N) in ((200, 136, 328), (2304, 256, 4352)):
        g = torch.Generator().manual_seed(N)
        x = torch.randn(M, K, generator=g).to(dtype)
        w = (torch.randn(K, N, generator=g) * 0.1).to(dtype)
        blen = N if order == "row" else M        # the bias follows the columns of the rewritten problem
        b = torch.randn(blen, generator=g).to(dtype) if "BIAS" in epilogue else None
        mk = (lambda: torch.full((M, N), float("nan"), dtype=out_dtype, device=cuda)) if order == "row" else \
             (lambda: torch.full((N, M), float("nan"), dtype=out_dtype, device=cuda).t())
        out, aux = mk(), mk()
        pkg.gemm(x.to(cuda), w.to(cuda), bias=None if b is None else b.to(cuda), epilogue=epilogue, out=out, aux=aux)
        acc = f32(x) @ f32(w)
        odt = {torch.bfloat16: orc.BF16, torch.float32: orc.F32}[out_dtype]
        if order == "row":
            want_d, want_aux = orc.gemm_epilogue(acc, None if b is None else f32(b), None, 0.0, epilogue, odt, with_aux=True)
        else:
            d_t, aux_t = orc.gemm_epilogue(acc.T, None if b is None else f32(b), None, 0.0, epilogue, odt, with_aux=True)
            want_d, want_aux = d_t.T, aux_t.T
        rtol, atol = TOL[out_dtype]
        orc.check_close(f32(aux), want_aux, rtol=rtol, atol=atol, what=f"{epilogue} aux {M}x{N} {order}")
        orc.check_close(f32(out), want_d, rtol=rtol, atol=atol, what=f"{epilogue} d {M}x{N} {order}")
    with pytest.raises(pkg.IxkError) as e:       # without the second buffer: the reference's answer
        pkg.gemm(x.to(cuda), w.to(cuda), epilogue="GELU_AUX")
    assert e.value.status == pkg.IXK_UNIMPLEMENTED


@pytest.mark.parametrize("shape", [(128, 64, 256), (200, 136, 328), (2304, 264, 4352), (16, 4096, 1024)])
@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_fp32_triple_runs_in_tf32(pkg, orc, cuda, shape, la, lb):
    """(F32,F32,F32) (onednn_matmul_utils.cc:609) on the tensor cores in TF32, the reference's
    XLA_FP32_MATH_MODE=TF32 (onednn_util.h:53-70).  Bound that holds for any TF32 implementation:
    each operand is off by < 2^-10 relative, so |D - A.B| <= 2^-9 (|A|.|B|); and the result must be
    the fp32 sum of products of operands cut to TF32 one way or the other (truncated or rounded)."""
    M, K, N = shape
    if (la == "col" and M % 4) or (lb == "row" and N % 4) or K % 4:
        pytest.skip("pitch not a multiple of 16 bytes")
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(K, N, generator=g) * 0.1
    b = torch.randn(N, generator=g)
    c = torch.randn(M, N, generator=g)
    out = pkg.gemm(as_layout(x.to(cuda), la), as_layout(w.to(cuda), lb), bias=b.to(cuda), c=c.to(cuda), beta=0.5,
                   alpha=2.0, epilogue="BIAS")
    assert out.dtype == torch.float32
    xn, wn = x.numpy(), w.numpy()
    exact = 2.0 * (xn.astype(np.float64) @ wn.astype(np.float64)) + b.numpy() + 0.5 * c.numpy()
    bound = 2.0 * 2.0 ** -9 * (np.abs(xn).astype(np.float64) @ np.abs(wn).astype(np.float64)) + 1e-4
    got = f32(out).astype(np.float64)
    assert np.all(np.abs(got - exact) <= bound), float(np.max(np.abs(got - exact) / bound))
    errs = []
    for mode in ("truncate", "round"):
        model = 2.0 * (orc.tf32_operand(xn, mode).astype(np.float64) @ orc.tf32_operand(wn, mode).astype(np.float64)) \
            + b.numpy() + 0.5 * c.numpy()
        errs.append(float(np.max(np.abs(got - model))))
    scale = float(np.max(np.abs(exact)))
    assert min(errs) <= 2e-5 * scale * np.sqrt(K / 64.0) + 1e-5, errs      # fp32 summation order only
    # GELU epilogue and a batch, against the oracle's epilogue chain on the TF32 model that matched
    mode = ("truncate", "round")[int(np.argmin(errs))]
    xb = torch.randn(3, 64, 96, generator=g)
    wb = torch.randn(3, 96, 40, generator=g) * 0.2
    outb = pkg.gemm(xb.to(cuda), wb.to(cuda), epilogue="GELU")
    for i in range(3):
        acc = orc.tf32_operand(xb[i].numpy(), mode) @ orc.tf32_operand(wb[i].numpy(), mode)
        want = orc.gemm_epilogue(acc, None, None, 0.0, "GELU", orc.F32)
        orc.check_close(f32(outb[i]), want, rtol=1e-3, atol=1e-3, what=f"tf32 batch {i}")


@pytest.mark.parametrize("shape", [(128, 128, 256), (200, 144, 336), (2304, 272, 4352), (16, 4096, 1024), (1, 16, 16)])
@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_int8_triple_is_exact(pkg, orc, cuda, shape, la, lb):
    """(S8,S8,S32) (onednn_matmul_utils.cc:610): integer products summed in 32 bits, bit for bit,
    over the whole signed 8-bit range."""
    M, K, N = shape
    if (la == "col" and M % 16) or (lb == "row" and N % 16) or K % 16:
        pytest.skip("pitch not a multiple of 16 bytes")
    g = torch.Generator().manual_seed(M * 7 + K * 3 + N)
    x = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int8)
    out = pkg.gemm(as_layout(x.to(cuda), la), as_layout(w.to(cuda), lb), out_dtype=torch.int32)
    assert out.dtype == torch.int32
    assert np.array_equal(out.cpu().numpy(), orc.gemm_s8(x.numpy(), w.numpy()))
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm(x.to(cuda), w.to(cuda), out_dtype=torch.int32, epilogue="RELU")
    assert e.value.status == pkg.IXK_UNIMPLEMENTED


def test_unaligned_pitch_is_rejected(pkg, cuda):
    x = torch.zeros(16, 20, dtype=torch.bfloat16, device=cuda)   # pitch 40 bytes
    w = torch.zeros(20, 16, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm(x, w)
    assert e.value.status == pkg.IXK_UNIMPLEMENTED
    with pytest.raises(pkg.IxkError) as e:       # a type triple outside RunGemm's list
        pkg.gemm(torch.zeros(16, 16, dtype=torch.float32, device=cuda), torch.zeros(16, 16, dtype=torch.float32, device=cuda),
                 out_dtype=torch.bfloat16)
    assert e.value.status == pkg.IXK_UNIMPLEMENTED


def test_empty_output_is_a_no_op(pkg, cuda):
    x = torch.zeros(0, 64, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(64, 32, dtype=torch.bfloat16, device=cuda)
    n0 = pkg.launch_count()
    out = pkg.gemm(x, w)
    assert out.shape == (0, 32) and pkg.launch_count() == n0


@pytest.mark.parametrize("shape", [(64, 3072, 12288), (64, 4096, 3072), (64, 24576, 3072), (8, 1024, 256), (128, 2048, 1536)])
@pytest.mark.parametrize("lb", ["row", "col"])
def test_split_k_skinny(pkg, orc, cuda, shape, lb):
    """Decode-shaped projections (M <= 128): with scratch the K range is split over CTAs and a
    second kernel reduces the partials and applies the epilogue; results must match the un-split
    path within accumulation-order noise, and the oracle within the usual tolerance."""
    M, K, N = shape
    g = torch.Generator().manual_seed(K + N)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(K, N, generator=g) * 0.03).bfloat16()
    b = torch.randn(N, generator=g).bfloat16()
    c = torch.randn(M, N, generator=g).bfloat16()
    xd, wd, bd, cd = x.to(cuda), as_layout(w.to(cuda), lb), b.to(cuda), c.to(cuda)
    need = pkg.gemm_workspace_bytes(xd, wd)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    n0 = pkg.launch_count()
    split = pkg.gemm(xd, wd, bias=bd, c=cd, beta=0.5, epilogue="BIAS_GELU", workspace=ws)
    assert pkg.launch_count() == n0 + 2            # partial GEMMs + reduce
    plain = pkg.gemm(xd, wd, bias=bd, c=cd, beta=0.5, epilogue="BIAS_GELU")
    assert pkg.launch_count() == n0 + 3
    want = orc.gemm_epilogue(f32(x) @ f32(w), f32(b), f32(c), 0.5, "BIAS_GELU", orc.BF16)
    orc.check_close(f32(split), want, rtol=2e-2, atol=2e-2, what=f"split-K {shape}")
    orc.check_close(f32(split), f32(plain), rtol=2e-2, atol=2e-2, what="split vs plain")
    # too little scratch: silently runs un-split
    n1 = pkg.launch_count()
    small = pkg.gemm(xd, wd, workspace=ws[:64])
    assert pkg.launch_count() == n1 + 1 and small.shape == (M, N)


@pytest.mark.parametrize("shape", [(64, 3072, 2 * 6144), (8, 512, 2 * 128), (128, 1024, 2 * 1024), (64, 3072, 2 * 24576)],
                         ids=lambda s: "M{}K{}N{}".format(*s))
def test_geglu_projection_in_one_product(pkg, orc, cuda, shape):
    """ixk_gemm_geglu: gate and up weights side by side, one GEMM (split along K where that helps) and
    one combining pass, against the three separate steps (gate GEMM with the GELU epilogue, up GEMM,
    elementwise product) and the oracle."""
    M, K, N2 = shape
    half = N2 // 2
    g = torch.Generator().manual_seed(M + K + N2)
    x = torch.randn(M, K, generator=g).bfloat16().to(cuda)
    w = (torch.randn(K, N2, generator=g) * 0.03).bfloat16().to(cuda)
    n0 = pkg.launch_count()
    got = pkg.gemm_geglu(x, w)
    assert pkg.launch_count() - n0 == 2 and got.shape == (M, half)
    gate = pkg.gemm(x, w[:, :half], epilogue="GELU")
    up = pkg.gemm(x, w[:, half:])
    # the same roundings in the same places; the products may differ in summation order (other K cuts)
    orc.check_close(f32(got), f32(gate * up), rtol=2e-2, atol=2e-3, what=f"geglu vs three steps {shape}")
    xf, wf = f32(x), f32(w)
    want = orc.round_bf16(orc.gemm_epilogue(xf @ wf[:, :half], None, None, 0.0, "GELU", orc.BF16) * orc.round_bf16(xf @ wf[:, half:]))
    orc.check_close(f32(got), want, rtol=2e-2, atol=2e-3, what=f"geglu vs oracle {shape}")
    # shapes it does not take
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm_geglu(torch.zeros(256, K, dtype=torch.bfloat16, device=cuda), w)
    assert e.value.status == pkg.IXK_UNIMPLEMENTED
    with pytest.raises(pkg.IxkError) as e:
        pkg.gemm_geglu(x, w, workspace=torch.empty(16, dtype=torch.uint8, device=cuda))
    assert e.value.status == pkg.IXK_WORKSPACE_TOO_SMALL
