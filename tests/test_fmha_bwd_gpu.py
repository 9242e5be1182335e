"""GPU parity of the attention backward (ixk_fmha_bwd) against the numpy oracle's statement of
fmha_backward.h, through the C ABI.  The forward runs on the GPU first; its output and log-sum-exp
rows are the inputs of both the kernel and the oracle, so that only the backward is compared.
Tolerance: the bf16 bound of the forward tests (rtol 2e-2, atol 2e-2) element-wise, plus a relative
Frobenius-norm bound of 1e-2 per gradient, which a structural error cannot meet."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def f32(t):
    return t.float().cpu().numpy()


def run_case(pkg, orc, cuda, *, B, N, F, T, H, causal=False, bias_shape=None, dtype=torch.bfloat16, seed=0,
             seq_major=False, launches_expected=3):
    g = torch.Generator().manual_seed(seed)

    def make(S):
        if seq_major:      # [B,S,N,H] storage handed over as a [B,N,S,H] view
            return torch.randn(B, S, N, H, generator=g).to(dtype).to(cuda).permute(0, 2, 1, 3)
        return torch.randn(B, N, S, H, generator=g).to(dtype).to(cuda)

    q, k, v, do = make(F), make(T), make(T), make(F)
    bias = None
    if bias_shape is not None:
        bias = (torch.randn(*bias_shape, F, T, generator=g) * 0.5).to(dtype).to(cuda)
    scale = 1.0 / math.sqrt(H)
    out = torch.empty_like(q)
    lse = torch.empty(B, N, F, dtype=torch.float32, device=cuda)
    pkg.fmha_forward_kernel(None, q, k, v, bias, None, 0.0, out, lse, scale, True, causal=causal)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    launches = pkg.launch_count()
    pkg.fmha_backward_kernel(None, q, k, v, out, bias, do, lse, dq, dk, dv, scale, causal=causal)
    torch.cuda.synchronize()
    assert pkg.launch_count() - launches == launches_expected
    assert pkg.device_status() == 0
    odt = orc.BF16 if dtype == torch.bfloat16 else orc.F16
    wq, wk, wv = orc.fmha_backward(f32(q), f32(k), f32(v), f32(out), f32(do), f32(lse),
                                   None if bias is None else f32(bias), head_scale=scale, causal=causal, dtype=odt)
    for name, got, want in (("dv", dv, wv), ("dk", dk, wk), ("dq", dq, wq)):
        got = f32(got)
        assert np.isfinite(got).all(), name
        # (a gradient that is zero up to rounding, e.g. dQ and dK of a single key, has no meaningful
        # relative error: the element-wise bound below still applies)
        if np.linalg.norm(want) > 1e-3 * math.sqrt(want.size):
            rel = np.linalg.norm(got - want) / np.linalg.norm(want)
            assert rel < 1e-2, f"{name}: relative error {rel:.3e}"
        orc.check_close(got, want, rtol=2e-2, atol=2e-2, what=name)


@pytest.mark.parametrize("H", [128, 64])
@pytest.mark.parametrize("causal", [False, True])
def test_one_block(pkg, orc, cuda, H, causal):
    run_case(pkg, orc, cuda, B=1, N=1, F=128, T=128, H=H, causal=causal, seed=1)


@pytest.mark.parametrize("F,T", [(256, 384), (384, 256), (200, 330), (130, 127), (640, 640), (5, 300), (300, 5), (1, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_several_blocks_and_ragged_edges(pkg, orc, cuda, F, T, causal):
    run_case(pkg, orc, cuda, B=2, N=3, F=F, T=T, H=128, causal=causal, seed=F + T)


@pytest.mark.parametrize("H", [64, 32, 96, 128])
def test_head_sizes(pkg, orc, cuda, H):
    run_case(pkg, orc, cuda, B=1, N=2, F=300, T=260, H=H, causal=True, seed=H)


@pytest.mark.parametrize("bias_shape", [(1, 1), (2, 1), (2, 2)])
def test_additive_bias(pkg, orc, cuda, bias_shape):
    run_case(pkg, orc, cuda, B=2, N=2, F=260, T=200, H=128, bias_shape=bias_shape, seed=7)


def test_fp16_and_sequence_major_storage(pkg, orc, cuda):
    run_case(pkg, orc, cuda, B=2, N=2, F=256, T=256, H=128, causal=True, dtype=torch.float16, seed=3)
    run_case(pkg, orc, cuda, B=2, N=4, F=384, T=384, H=64, causal=True, seq_major=True, seed=4)


@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
@pytest.mark.parametrize("case", [dict(B=1, N=1, F=128, T=128, H=256), dict(B=2, N=3, F=200, T=330, H=256),
                                  dict(B=1, N=2, F=300, T=77, H=160), dict(B=2, N=2, F=5, T=260, H=256),
                                  dict(B=1, N=4, F=384, T=384, H=256, seq_major=True),
                                  dict(B=2, N=2, F=260, T=200, H=256, bias_shape=(2, 1)),
                                  dict(B=1, N=2, F=256, T=256, H=192, dtype=torch.float16)],
                         ids=lambda c: "B{B}N{N}F{F}T{T}H{H}".format(**c) + ("sm" if c.get("seq_major") else "") +
                         ("b" if c.get("bias_shape") else "") + ("f16" if c.get("dtype") else ""))
def test_heads_wider_than_128(pkg, orc, cuda, case, causal):
    """Head sizes 129..256 (the reference's 64x128x256 backward policy, fmha_policy.h:107-116; both
    decoder-layer configurations have 256-wide heads): the GEMM-chain path, one group of heads per
    batch element here: prepare + 5 products + 2 score passes per group."""
    if case.get("bias_shape") and causal:
        pytest.skip("one mask at a time")
    run_case(pkg, orc, cuda, causal=causal, seed=case["F"] + case["H"], launches_expected=1 + 7 * case["B"], **case)


def test_wide_heads_in_several_groups(pkg, orc, cuda):
    """Scores of all heads that do not fit the per-group scratch budget (192 MB) are processed a
    group of heads at a time: 8 heads of 2304 x 2304 scores (32 MB each) run as groups of 6 and 2."""
    B, N, F, T, H = 1, 8, 2304, 2304, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda S: torch.randn(B, N, S, H, generator=g, device=cuda).bfloat16()
    q, k, v, do = mk(F), mk(T), mk(T), mk(F)
    scale = H ** -0.5
    out = torch.empty_like(q)
    lse = torch.empty(B, N, F, dtype=torch.float32, device=cuda)
    pkg.fmha_forward_kernel(None, q, k, v, None, None, 0.0, out, lse, scale, True, causal=True)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    n0 = pkg.launch_count()
    pkg.fmha_backward_kernel(None, q, k, v, out, None, do, lse, dq, dk, dv, scale, causal=True)
    assert pkg.launch_count() - n0 == 1 + 7 * 2 and pkg.device_status() == 0
    mask = torch.ones(F, T, dtype=torch.bool, device=cuda).tril()
    for n in (0, 7):
        qq, kk, vv = (t[:, n:n + 1].float().requires_grad_() for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=scale)
        ref.backward(do[:, n:n + 1].float())
        for name, got, want in (("dq", dq, qq.grad), ("dk", dk, kk.grad), ("dv", dv, vv.grad)):
            rel = ((got[:, n:n + 1].float() - want).norm() / want.norm()).item()
            assert rel < 1e-2, f"{name}[{n}]: relative error {rel:.3e}"


def test_rejections(pkg, cuda):
    lse = torch.zeros(1, 1, 128, device=cuda)
    q = torch.randn(1, 1, 128, 64, device=cuda).bfloat16()
    with pytest.raises(pkg.IxkError):      # gradient buffer of the wrong shape
        pkg.fmha_backward_kernel(None, q, q, q, q, None, q, lse, torch.empty(1, 1, 64, 64, device=cuda).bfloat16(),
                                 torch.empty_like(q), torch.empty_like(q), 1.0)
    with pytest.raises(pkg.IxkError):      # log-sum-exp rows missing
        pkg.fmha_backward_kernel(None, q, q, q, q, None, q, None, torch.empty_like(q), torch.empty_like(q),
                                 torch.empty_like(q), 1.0)


@pytest.mark.parametrize("fname", ["fmha_bwd_bf16.npz", "fmha_bwd_h256_bf16.npz"])
def test_golden_vectors(pkg, orc, cuda, fname):
    """Gradients made by autograd over fp32 attention on the CPU (tests/golden/make_golden.py),
    head size 64 (fused kernel) and 256 (GEMM-chain path)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", fname))
    t = lambda name: torch.from_numpy(g[name].view(np.int16)).view(torch.bfloat16).to(cuda)
    q, k, v, do, bias = (t(n) for n in ("q", "k", "v", "do", "bias"))
    scale = float(g["scale"])
    for name in ("causal", "bias"):
        b = bias if name == "bias" else None
        out = torch.empty_like(q)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=cuda)
        pkg.fmha_forward_kernel(None, q, k, v, b, None, 0.0, out, lse, scale, True, causal=name == "causal")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        pkg.fmha_backward_kernel(None, q, k, v, out, b, do, lse, dq, dk, dv, scale, causal=name == "causal")
        for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            orc.check_close(f32(got), g[f"{key}_{name}"], rtol=2e-2, atol=2e-2, what=f"golden {key} {name}")


@pytest.mark.parametrize("causal", [True, False])
def test_full_size_against_fp32_autograd(pkg, cuda, causal):
    """The benchmark's shape (B8 N16 S2048 H128): a few (batch, head) slices of all three gradients
    against autograd over fp32 attention on the same GPU; every element must also be finite."""
    B, N, S, H = 8, 16, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    mk = lambda: torch.randn(B, N, S, H, generator=g, device=cuda).bfloat16()
    q, k, v, do = mk(), mk(), mk(), mk()
    scale = H ** -0.5
    out = torch.empty_like(q)
    lse = torch.empty(B, N, S, dtype=torch.float32, device=cuda)
    pkg.fmha_forward_kernel(None, q, k, v, None, None, 0.0, out, lse, scale, True, causal=causal)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    pkg.fmha_backward_kernel(None, q, k, v, out, None, do, lse, dq, dk, dv, scale, causal=causal)
    assert pkg.device_status() == 0
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    mask = torch.ones(S, S, dtype=torch.bool, device=cuda).tril() if causal else None
    for b, n in ((0, 0), (3, 7), (7, 15)):
        qq, kk, vv = (t[b:b + 1, n:n + 1].float().requires_grad_() for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=scale)
        ref.backward(do[b:b + 1, n:n + 1].float())
        for name, got, want in (("dq", dq, qq.grad), ("dk", dk, kk.grad), ("dv", dv, vv.grad)):
            got = got[b:b + 1, n:n + 1].float()
            rel = ((got - want).norm() / want.norm()).item()
            assert rel < 1e-2, f"{name}[{b},{n}]: relative error {rel:.3e}"
            assert torch.allclose(got, want, rtol=2e-2, atol=2e-2), name
