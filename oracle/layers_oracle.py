"""CPU oracle for the two decoder-layer configurations (TEST INFRASTRUCTURE — never the product
path): an independent numpy float32 statement of the GPT-J prefill block and the Gemma decode
step, un-sharded, against which the tensor-parallel CUDA drivers are compared.

PARITY UNPINNED: the layers are the benchmark's own composition of the three custom calls (shapes
from example/gptj/jax_gptj.py and example/gemma/keras_nlp.patch:53-63, random-init weights); the
reference has no golden outputs for them.  Intermediate activations are rounded to bf16 where the
CUDA path stores them in bf16, so that the comparison isolates kernel error from storage rounding.
"""
from __future__ import annotations

import math

import numpy as np

from . import ixk_oracle as orc


def _r(x):
    return orc.round_bf16(np.asarray(x, np.float32))


def layer_norm(x, eps=1e-5):
    x = np.asarray(x, np.float32)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return _r((x - mu) / np.sqrt(var + eps))


def rms_norm(x, eps=1e-6, gain=None):
    """`gain`: the learned scale w of Gemma's RMSNorm, applied as (1 + w) before the one rounding."""
    x = np.asarray(x, np.float32)
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return _r(y if gain is None else y * (1.0 + np.asarray(gain, np.float32)))


def rotary(x, positions, rotary_dim, base=10000.0):
    """Interleaved-pair rotary on the first rotary_dim elements; x [..., S, heads, head_dim]."""
    x = np.array(x, np.float32)
    inv = 1.0 / (base ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / rotary_dim))
    ang = np.asarray(positions, np.float32)[:, None] * inv[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x1, x2 = x[..., 0:rotary_dim:2].copy(), x[..., 1:rotary_dim:2].copy()
    x[..., 0:rotary_dim:2] = x1 * c - x2 * s
    x[..., 1:rotary_dim:2] = x1 * s + x2 * c
    return _r(x)


def rotary_half(x, positions, rotary_dim, base=10000.0):
    """Half-split rotary (Gemma): element i < rotary_dim/2 pairs with i + rotary_dim/2; the published
    form of keras_nlp's CachedGemmaAttention._apply_rope, which the reference's Gemma example runs
    (example/gemma/keras_nlp.patch:6-23 calls it; keras_nlp itself is not part of the reference)."""
    x = np.array(x, np.float32)
    half = rotary_dim // 2
    inv = 1.0 / (base ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / rotary_dim))
    ang = np.asarray(positions, np.float32)[:, None] * inv[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x1, x2 = x[..., :half].copy(), x[..., half:rotary_dim].copy()
    x[..., :half] = x1 * c - x2 * s
    x[..., half:rotary_dim] = x2 * c + x1 * s
    return _r(x)


def gptj_layer_prefill(x, w, num_heads, head_dim, rotary_dim):
    """y = x + Attn(LN(x)) + MLP(LN(x)); x [B,S,hidden]; w: dict of full (un-sharded) float32 weights
    holding bf16-representable values."""
    B, S, hidden = x.shape
    h = layer_norm(x).reshape(B * S, hidden)
    qkv = _r(h @ w["wqkv"]).reshape(B, S, 3, num_heads, head_dim)
    pos = np.arange(S)
    q = rotary(qkv[:, :, 0], pos, rotary_dim).transpose(0, 2, 1, 3)
    k = rotary(qkv[:, :, 1], pos, rotary_dim).transpose(0, 2, 1, 3)
    v = qkv[:, :, 2].transpose(0, 2, 1, 3)
    ctx, _ = orc.fmha_forward(q, k, v, None, head_scale=1.0 / math.sqrt(head_dim), causal=True)
    ctx = ctx.transpose(0, 2, 1, 3).reshape(B * S, num_heads * head_dim)
    attn = ctx @ w["wo"]
    up = orc.gemm_epilogue(h @ w["w1"], w["b1"], None, 0.0, "BIAS_GELU", orc.BF16)
    partial = attn + up @ w["w2"]
    return _r(np.asarray(x, np.float32) + (partial + w["b2"][None, :]).reshape(B, S, hidden))


def gemma_decode_step(x, w, k_cache, v_cache, position, num_heads, head_dim):
    """x [B,1,hidden]; caches [B,T,heads,head_dim] (updated copies are used, inputs untouched)."""
    B, _, hidden = x.shape
    h = rms_norm(x, gain=w.get("norm_attn")).reshape(B, hidden)
    qkv = _r(h @ w["wqkv"]).reshape(B, 1, 3, num_heads, head_dim)
    pos = np.array([position])
    q = rotary_half(qkv[:, :, 0], pos, head_dim).transpose(0, 2, 1, 3)
    k_new = rotary_half(qkv[:, :, 1], pos, head_dim)[:, 0]
    k_cache = np.array(k_cache, np.float32)
    v_cache = np.array(v_cache, np.float32)
    k_cache[:, position] = k_new
    v_cache[:, position] = qkv[:, 0, 2]
    T = position + 1
    ctx, _ = orc.fmha_forward(q, k_cache[:, :T].transpose(0, 2, 1, 3), v_cache[:, :T].transpose(0, 2, 1, 3), None,
                              head_scale=1.0 / math.sqrt(head_dim))
    ctx = ctx.transpose(0, 2, 1, 3).reshape(B, num_heads * head_dim)
    x1 = _r(np.asarray(x, np.float32) + _r(ctx @ w["wo"]).reshape(B, 1, hidden))
    h2 = rms_norm(x1, gain=w.get("norm_mlp")).reshape(B, hidden)
    gate = orc.gemm_epilogue(h2 @ w["wgate"], None, None, 0.0, "GELU", orc.BF16)
    up = _r(h2 @ w["wup"])
    down = _r(_r(gate * up) @ w["wdown"])
    return _r(x1 + down.reshape(B, 1, hidden))
