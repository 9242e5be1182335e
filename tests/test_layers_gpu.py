"""GPU parity: the decoder-layer drivers (GEMM + attention kernels + torch glue) on one GPU against
the un-sharded numpy layer oracle, at reduced sizes the oracle finishes in seconds.
Tolerance: activations are O(1) and stored in bf16 between kernels, so 6e-2 absolute (a few bf16
ulps accumulated over the block), plus the bf16 relative bound 2e-2."""
import importlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def f32(t):
    return t.float().cpu().numpy()


def test_gptj_block_prefill(pkg, orc, cuda):
    from oracle import layers_oracle
    layers = importlib.import_module("ixk_b200.layers")
    hidden, heads, hd, rot, ffn, B, S = 512, 2, 256, 64, 1024, 2, 320
    g = torch.Generator().manual_seed(1)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.02).bfloat16()
    full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "w1": r(hidden, ffn), "b1": r(ffn),
            "w2": r(ffn, hidden), "b2": r(hidden)}
    x = torch.randn(B, S, hidden, generator=g).bfloat16()
    w = layers.GptJLayerWeights.shard({k: v.to(cuda) for k, v in full.items()}, heads, hd, rot, 0, 1)
    y = layers.gptj_layer_prefill(x.to(cuda), w, layers.KernelOps(pkg))
    want = layers_oracle.gptj_layer_prefill(f32(x), {k: f32(v) for k, v in full.items()}, heads, hd, rot)
    orc.check_close(f32(y), want, rtol=2e-2, atol=6e-2, what="gptj block")


def test_gemma_decode_step(pkg, orc, cuda):
    from oracle import layers_oracle
    layers = importlib.import_module("ixk_b200.layers")
    hidden, heads, hd, ffn, B, T = 384, 2, 256, 768, 5, 700
    g = torch.Generator().manual_seed(2)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.02).bfloat16()
    full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "wgate": r(hidden, ffn),
            "wup": r(hidden, ffn), "wdown": r(ffn, hidden),
            "norm_attn": r(hidden), "norm_mlp": r(hidden)}
    x = torch.randn(B, 1, hidden, generator=g).bfloat16()
    kc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
    vc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
    w = layers.GemmaLayerWeights.shard({k: v.to(cuda) for k, v in full.items()}, heads, hd, 0, 1)
    kd, vd = kc.to(cuda), vc.to(cuda)
    y = layers.gemma_decode_step(x.to(cuda), w, kd, vd, T - 1, layers.KernelOps(pkg))
    want = layers_oracle.gemma_decode_step(f32(x), {k: f32(v) for k, v in full.items()}, f32(kc), f32(vc), T - 1, heads, hd)
    orc.check_close(f32(y), want, rtol=2e-2, atol=6e-2, what="gemma decode")
    assert not torch.equal(kd[:, T - 1].cpu(), kc[:, T - 1])      # the new key was written into the cache


def test_gptj_block_at_full_width(pkg, orc, cuda):
    """Configuration 4's layer at its real widths (hidden 4096, 16 heads x 256, rotary 64, MLP 16384,
    weights ~ N(0, 0.02)), with batch and sequence cut to what the numpy oracle finishes in seconds
    (2 x 320 tokens instead of 4 x 2048; 320 is not a multiple of the 128-row tiles)."""
    from oracle import layers_oracle
    layers = importlib.import_module("ixk_b200.layers")
    hidden, heads, hd, rot, ffn, B, S = 4096, 16, 256, 64, 16384, 2, 320
    g = torch.Generator().manual_seed(3)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.02).bfloat16()
    full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "w1": r(hidden, ffn), "b1": r(ffn),
            "w2": r(ffn, hidden), "b2": r(hidden)}
    x = torch.randn(B, S, hidden, generator=g).bfloat16()
    w = layers.GptJLayerWeights.shard({k: v.to(cuda) for k, v in full.items()}, heads, hd, rot, 0, 1)
    y = layers.gptj_layer_prefill(x.to(cuda), w, layers.KernelOps(pkg))
    want = layers_oracle.gptj_layer_prefill(f32(x), {k: f32(v) for k, v in full.items()}, heads, hd, rot)
    orc.check_close(f32(y), want, rtol=2e-2, atol=6e-2, what="gptj block, full width")


def test_gemma_decode_step_at_full_width(pkg, orc, cuda):
    """Configuration 5's step at its real widths (hidden 3072, 16 heads x 256, GeGLU 24576: the
    K = 24576 down projection runs split along K), 8 sequences against a cache of 1100 keys
    instead of 64 against 4096."""
    from oracle import layers_oracle
    layers = importlib.import_module("ixk_b200.layers")
    hidden, heads, hd, ffn, B, T = 3072, 16, 256, 24576, 8, 1100
    g = torch.Generator().manual_seed(4)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.02).bfloat16()
    full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "wgate": r(hidden, ffn),
            "wup": r(hidden, ffn), "wdown": r(ffn, hidden),
            "norm_attn": r(hidden), "norm_mlp": r(hidden)}
    x = torch.randn(B, 1, hidden, generator=g).bfloat16()
    kc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
    vc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
    w = layers.GemmaLayerWeights.shard({k: v.to(cuda) for k, v in full.items()}, heads, hd, 0, 1)
    ops = layers.KernelOps(pkg, gemm_workspace=torch.empty(32 << 20, dtype=torch.uint8, device=cuda))
    n0 = pkg.launch_count()
    y = layers.gemma_decode_step(x.to(cuda), w, kc.to(cuda), vc.to(cuda), T - 1, ops)
    assert pkg.launch_count() - n0 >= 5 * 2 + 2       # every projection split along K (+ reduce), attention + combine
    want = layers_oracle.gemma_decode_step(f32(x), {k: f32(v) for k, v in full.items()}, f32(kc), f32(vc), T - 1, heads, hd)
    orc.check_close(f32(y), want, rtol=2e-2, atol=6e-2, what="gemma decode, full width")
