"""GPU parity of the memory-bound steps between the custom calls (row normalisation, interleaved
rotary embedding, residual add) against the numpy layer oracle, through the C ABI.
Tolerances: outputs are O(1) values rounded once to the 16-bit type; a result may differ from the
oracle's by one rounding step where fp32 summation order differs, so 1 ulp of the type relative
(2^-7 for bf16, 2^-10 for fp16) plus the same absolute."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ULP = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}


def f32(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 264), (37, 3072), (64, 4096), (5, 8192), (300, 520)])
def test_row_norm(pkg, orc, cuda, dtype, kind, rows, cols):
    from oracle import layers_oracle
    g = torch.Generator().manual_seed(rows * 131 + cols)
    x = (torch.randn(rows, cols, generator=g) * 1.7 + 0.3).to(dtype)
    if kind == "layer":
        got = pkg.row_norm(x.to(cuda), kind=pkg.NORM_LAYER, eps=1e-5)
        xf = f32(x)
        mu = xf.mean(-1, keepdims=True)
        want = (xf - mu) / np.sqrt(((xf - mu) ** 2).mean(-1, keepdims=True) + 1e-5)
    else:
        got = pkg.row_norm(x.to(cuda), kind=pkg.NORM_RMS, eps=1e-6)
        xf = f32(x)
        want = xf / np.sqrt((xf * xf).mean(-1, keepdims=True) + 1e-6)
    assert got.dtype == dtype and got.shape == x.shape
    orc.check_close(f32(got), want, rtol=ULP[dtype], atol=ULP[dtype], what=f"row_norm {kind}")
    if dtype == torch.bfloat16:      # the layer oracle's own statement, bf16 storage
        ref = layers_oracle.layer_norm(xf) if kind == "layer" else layers_oracle.rms_norm(xf)
        orc.check_close(f32(got), ref, rtol=ULP[dtype], atol=ULP[dtype], what=f"row_norm {kind} vs layer oracle")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 3072), (5, 8192), (300, 520)])
def test_rms_norm_with_the_one_plus_w_scale(pkg, orc, cuda, dtype, rows, cols):
    """Gemma's RMSNorm: normalised * (1 + w), one rounding (and offset 0: the usual learned gain)."""
    from oracle import layers_oracle
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn(rows, cols, generator=g) * 1.7 + 0.3).to(dtype)
    w = (torch.randn(cols, generator=g) * 0.3).to(dtype)
    xf, wf = f32(x), f32(w)
    normed = xf / np.sqrt((xf * xf).mean(-1, keepdims=True) + 1e-6)
    got = pkg.row_norm(x.to(cuda), kind=pkg.NORM_RMS, eps=1e-6, gain=w.to(cuda), gain_offset=1.0)
    orc.check_close(f32(got), normed * (1.0 + wf), rtol=ULP[dtype], atol=ULP[dtype], what="rms norm (1 + w)")
    if dtype == torch.bfloat16:
        orc.check_close(f32(got), layers_oracle.rms_norm(xf, gain=wf), rtol=ULP[dtype], atol=ULP[dtype], what="vs layer oracle")
    got0 = pkg.row_norm(x.to(cuda), kind=pkg.NORM_RMS, eps=1e-6, gain=w.to(cuda))
    orc.check_close(f32(got0), normed * wf, rtol=ULP[dtype], atol=ULP[dtype], what="rms norm w")
    with pytest.raises(pkg.IxkError):
        pkg.row_norm(x.to(cuda), kind=pkg.NORM_RMS, gain=w[:-1].contiguous().to(cuda))     # wrong length


def test_row_norm_in_place_and_rejections(pkg, cuda):
    x = torch.randn(16, 256).bfloat16().to(cuda)
    want = pkg.row_norm(x)
    pkg.row_norm(x, out=x)
    assert torch.equal(x, want)
    with pytest.raises(pkg.IxkError):
        pkg.row_norm(torch.randn(4, 12).bfloat16().to(cuda))            # cols not a multiple of 8
    with pytest.raises(pkg.IxkError):
        pkg.row_norm(torch.randn(2, 8200).bfloat16().to(cuda))          # longer than 8192
    with pytest.raises(pkg.IxkError):
        pkg.row_norm(torch.randn(4, 16).to(cuda))                       # fp32 is not covered
    empty = pkg.row_norm(torch.empty(0, 64, dtype=torch.bfloat16, device=cuda))
    assert empty.shape == (0, 64)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,heads,hd,rot", [(2, 37, 2, 256, 64), (1, 1, 4, 256, 256), (3, 128, 3, 64, 64),
                                              (5, 1, 2, 128, 32), (1, 700, 1, 256, 8)])
def test_rotary_on_fused_qkv(pkg, orc, cuda, dtype, B, S, heads, hd, rot):
    """q and k slices of a fused [B,S,3,heads,hd] projection rotate; v and the tail of every head stay."""
    from oracle import layers_oracle
    layers = __import__("importlib").import_module("ixk_b200.layers")
    g = torch.Generator().manual_seed(B * 1000 + S)
    qkv = torch.randn(B, S, 3, heads, hd, generator=g).to(dtype)
    cos, sin = layers.rotary_tables(torch.arange(S), rot)
    dev = qkv.to(cuda)
    layers.KernelOps(pkg).rotary_qk_(dev, cos.to(cuda), sin.to(cuda), rot)
    xf = f32(qkv)
    assert torch.equal(dev[:, :, 2].cpu(), qkv[:, :, 2])
    assert torch.equal(dev[..., rot:].cpu(), qkv[..., rot:])
    for i in range(2):
        want = layers_oracle.rotary(xf[:, :, i], np.arange(S), rot) if dtype == torch.bfloat16 else None
        c, s = f32(cos)[:, None, :], f32(sin)[:, None, :]
        x1, x2 = xf[:, :, i, :, 0:rot:2], xf[:, :, i, :, 1:rot:2]
        exact = xf[:, :, i].copy()
        exact[..., 0:rot:2] = x1 * c - x2 * s
        exact[..., 1:rot:2] = x1 * s + x2 * c
        orc.check_close(f32(dev[:, :, i]), exact, rtol=ULP[dtype], atol=ULP[dtype], what="rotary")
        if want is not None:        # the oracle builds its own tables in numpy: table rounding adds an ulp
            orc.check_close(f32(dev[:, :, i]), want, rtol=2 * ULP[dtype], atol=2 * ULP[dtype], what="rotary vs layer oracle")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,heads,hd,rot", [(2, 37, 2, 256, 256), (1, 1, 4, 256, 256), (3, 128, 3, 64, 32),
                                              (5, 1, 2, 128, 128), (1, 700, 1, 256, 16)])
def test_rotary_half_split_on_fused_qkv(pkg, orc, cuda, dtype, B, S, heads, hd, rot):
    """The Gemma convention: element i pairs with element i + rot/2."""
    from oracle import layers_oracle
    layers = __import__("importlib").import_module("ixk_b200.layers")
    g = torch.Generator().manual_seed(B * 999 + S)
    qkv = torch.randn(B, S, 3, heads, hd, generator=g).to(dtype)
    cos, sin = layers.rotary_tables(torch.arange(S), rot)
    dev = qkv.to(cuda)
    layers.KernelOps(pkg).rotary_qk_(dev, cos.to(cuda), sin.to(cuda), rot, half_split=True)
    xf = f32(qkv)
    assert torch.equal(dev[:, :, 2].cpu(), qkv[:, :, 2])
    assert torch.equal(dev[..., rot:].cpu(), qkv[..., rot:])
    half = rot // 2
    for i in range(2):
        c, s = f32(cos)[:, None, :], f32(sin)[:, None, :]
        x1, x2 = xf[:, :, i, :, :half], xf[:, :, i, :, half:rot]
        exact = xf[:, :, i].copy()
        exact[..., :half] = x1 * c - x2 * s
        exact[..., half:rot] = x2 * c + x1 * s
        orc.check_close(f32(dev[:, :, i]), exact, rtol=ULP[dtype], atol=ULP[dtype], what="rotary, half-split")
        if dtype == torch.bfloat16:
            want = layers_oracle.rotary_half(xf[:, :, i], np.arange(S), rot)
            orc.check_close(f32(dev[:, :, i]), want, rtol=2 * ULP[dtype], atol=2 * ULP[dtype], what="vs layer oracle")
    # the torch stand-in the CPU tests use computes the same thing
    ref = qkv.clone()
    layers._rotary_qk_torch_(ref, cos, sin, rot, half_split=True)
    orc.check_close(f32(dev), f32(ref), rtol=ULP[dtype], atol=ULP[dtype], what="kernel vs torch stand-in")
    with pytest.raises(pkg.IxkError):
        pkg.rotary_half_(dev.view(B * S, 3 * heads, hd), cos[:, :4].contiguous().to(cuda), sin[:, :4].contiguous().to(cuda), S, 8)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", ["btnh", "bnth"])
def test_kv_append(pkg, cuda, dtype, layout):
    """The step's keys and values land at `position` of both caches, nothing else changes; the new
    rows are slices of a fused QKV projection (strided views), the cache in either layout."""
    B, T, N, H, pos = 3, 37, 4, 256, 21
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, 1, 3, N, H, generator=g).to(dtype).to(cuda)
    if layout == "btnh":
        kc, vc = (torch.randn(B, T, N, H, generator=g).to(dtype).to(cuda) for _ in range(2))
    else:
        kc, vc = (torch.randn(B, N, T, H, generator=g).to(dtype).to(cuda).permute(0, 2, 1, 3) for _ in range(2))
    want_k, want_v = kc.clone(), vc.clone()
    want_k[:, pos] = qkv[:, 0, 1]
    want_v[:, pos] = qkv[:, 0, 2]
    n0 = pkg.launch_count()
    pkg.kv_append_(kc, vc, qkv[:, 0, 1], qkv[:, 0, 2], pos)
    assert pkg.launch_count() == n0 + 1
    assert torch.equal(kc, want_k) and torch.equal(vc, want_v)
    with pytest.raises(pkg.IxkError):
        pkg.kv_append_(kc, vc, qkv[:, 0, 1], qkv[:, 0, 2], T)                 # position outside the cache
    with pytest.raises(pkg.IxkError):
        pkg.kv_append_(kc, vc, qkv[:, 0, 1, :2], qkv[:, 0, 2, :2], pos)       # head count differs


def test_rotary_rejections(pkg, cuda):
    x = torch.randn(8, 2, 64).bfloat16().to(cuda)
    cos = torch.ones(8, 16, device=cuda)
    with pytest.raises(pkg.IxkError):
        pkg.rotary_interleaved_(x, cos, cos, 8, 36)                      # table shape does not match rotary_dim
    with pytest.raises(pkg.IxkError):
        pkg.rotary_interleaved_(x, cos[:3].contiguous(), cos[:3].contiguous(), 3, 32)   # 8 tokens, seq_len 3
    with pytest.raises(pkg.IxkError):
        pkg.rotary_interleaved_(x, cos.double(), cos.double(), 8, 32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("rows,cols", [(1, 8), (33, 3072), (640, 4096), (7, 520)])
def test_residual_add(pkg, cuda, dtype, with_bias, rows, cols):
    """Bit-exact: both roundings are defined (inner sum to the type, then the residual add)."""
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    p = torch.randn(rows, cols, generator=g).to(dtype)
    b = torch.randn(cols, generator=g).to(dtype) if with_bias else None
    got = pkg.residual_add(x.to(cuda), p.to(cuda), b.to(cuda) if with_bias else None)
    inner = (p.float() + b.float()).to(dtype) if with_bias else p
    want = (x.float() + inner.float()).to(dtype)
    assert torch.equal(got.cpu(), want)


def test_residual_add_aliasing_and_rejections(pkg, cuda):
    x = torch.randn(40, 64).bfloat16().to(cuda)
    p = torch.randn(40, 64).bfloat16().to(cuda)
    want = pkg.residual_add(x, p)
    pkg.residual_add(x, p, out=p)
    assert torch.equal(p, want)
    with pytest.raises(pkg.IxkError):
        pkg.residual_add(x, p[:, :32].contiguous())
    with pytest.raises(pkg.IxkError):
        pkg.residual_add(x, p, torch.zeros(32, dtype=torch.bfloat16, device=cuda))
