"""Decoder-layer drivers built from the three custom calls: the shapes the reference's examples
run (GPT-J prefill, example/gptj/jax_gptj.py; Gemma decode with a [B,T,N,H] KV cache,
example/gemma/keras_nlp.patch:53-63), tensor-parallel the way the Gemma example lays it out
(example/gemma/finetune.py:136-153): QKV and the MLP up-projection split by heads / columns with
no exchange, attention by heads, the row-parallel projections (attention output, MLP down) ending
in one all-reduce.

The GEMMs and the attention go through libixk (`KernelOps`), and so do the steps between them
that XLA would emit as fusions: row normalisation, rotary embedding and the residual adds are one
pass over HBM each (csrc/glue_sm100.cu).  `ops` is injectable so that the sharding and reduction
logic can be exercised on CPU ranks with a stand-in implementation of the two calls; an `ops`
without the glue methods gets the plain torch versions defined below.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------- kernel calls

class KernelOps:
    """The custom calls as the layers use them, bound to libixk.so."""

    def __init__(self, pkg, gemm_workspace=None):
        self.pkg = pkg
        self.gemm_workspace = gemm_workspace   # scratch for split-K of skinny (decode) GEMMs; may be None

    def gemm(self, x, w, *, bias=None, c=None, beta=0.0, epilogue="DEFAULT", out=None):
        return self.pkg.gemm(x, w, bias=bias, c=c, beta=beta, epilogue=epilogue, out=out,
                             workspace=self.gemm_workspace)

    def gemm_geglu(self, x, w_gate_up):
        """gelu(x @ gate) * (x @ up) with [gate | up] as one weight: one GEMM + one combining pass (decode
        shapes; needs the scratch).  None when the library does not take the shape."""
        if x.shape[-2] > 128 or self.gemm_workspace is None:
            return None
        try:
            return self.pkg.gemm_geglu(x, w_gate_up, workspace=self.gemm_workspace)
        except self.pkg.IxkError as ex:
            if ex.status in (self.pkg.IXK_UNIMPLEMENTED, self.pkg.IXK_WORKSPACE_TOO_SMALL):
                return None
            raise

    def attention(self, q, k, v, out, *, scale, causal, workspace=None):
        """q/out [B,N,F,H] views, k/v [B,N,T,H] views."""
        self.pkg.fmha_forward_kernel(None, q, k, v, None, None, 0.0, out, None, scale, False, causal=causal,
                                     workspace=workspace)
        return out

    def layer_norm(self, x, eps=1e-5):
        return self.pkg.row_norm(x, kind=self.pkg.NORM_LAYER, eps=eps)

    def rms_norm(self, x, eps=1e-6, gain=None):
        """`gain`: Gemma's learned scale w, applied as (1 + w)."""
        return self.pkg.row_norm(x, kind=self.pkg.NORM_RMS, eps=eps, gain=gain, gain_offset=1.0)

    def rotary_qk_(self, qkv, cos, sin, rotary_dim, half_split=False):
        """qkv [B, S, 3, heads_local, head_dim] dense: rotates the q and k slices in place (they are
        2 * heads_local consecutive heads of every token)."""
        B, S, _, hl, hd = qkv.shape
        qk = qkv.view(B * S, 3 * hl, hd)[:, :2 * hl]
        self.pkg.rotary_interleaved_(qk, cos, sin, S, rotary_dim, half_split=half_split)
        return qkv

    def residual_add(self, x, partial, bias=None, out=None):
        return self.pkg.residual_add(x, partial, bias, out=out)

    def kv_append_(self, k_cache, v_cache, k_new, v_new, position):
        self.pkg.kv_append_(k_cache, v_cache, k_new, v_new, position)


def _glue(ops, name, fallback):
    return getattr(ops, name, None) or fallback


# ----------------------------------------------------------------------------- sharding

def shard_range(total: int, rank: int, world: int):
    """Contiguous [begin, end) share of `total` units for `rank`; total must divide evenly."""
    if total % world != 0:
        raise ValueError(f"{total} units do not split evenly over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def shard_qkv_weight(wqkv: torch.Tensor, num_heads: int, head_dim: int, rank: int, world: int) -> torch.Tensor:
    """Fused QKV weight [hidden, 3*num_heads*head_dim] (q | k | v blocks, heads inside each) →
    the columns of this rank's heads, still as q | k | v."""
    hidden = wqkv.shape[0]
    h0, h1 = shard_range(num_heads, rank, world)
    w = wqkv.view(hidden, 3, num_heads, head_dim)[:, :, h0:h1, :]
    return w.reshape(hidden, 3 * (h1 - h0) * head_dim).contiguous()


def shard_columns(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    c0, c1 = shard_range(w.shape[-1], rank, world)
    return w[..., c0:c1].contiguous()


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    r0, r1 = shard_range(w.shape[0], rank, world)
    return w[r0:r1].contiguous()


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the row-parallel partials over the tensor-parallel group (NCCL on GPUs)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


# ----------------------------------------------------------------------------- glue

def layer_norm(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm with unit gain and zero shift (the benchmark's random-init convention)."""
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = xf.var(-1, keepdim=True, unbiased=False)
    return ((xf - mu) * torch.rsqrt(var + eps)).to(x.dtype)


def rms_norm(x: torch.Tensor, eps: float = 1e-6, gain: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm; `gain` is Gemma's learned scale w, applied as (1 + w) before the one rounding."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y if gain is None else y * (1.0 + gain.float())).to(x.dtype)


def rotary_tables(positions: torch.Tensor, rotary_dim: int, base: float = 10000.0):
    """cos/sin [len(positions), rotary_dim/2] in fp32."""
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, device=positions.device, dtype=torch.float32) / rotary_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rotary_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """In place, GPT-J convention: interleaved pairs (2i, 2i+1) of the first rotary_dim elements of
    every head.  x [..., S, heads, head_dim]; cos/sin [S, rotary_dim/2]."""
    rot = x[..., :rotary_dim].float()
    x1, x2 = rot[..., 0::2], rot[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1).flatten(-2)
    x[..., :rotary_dim] = out.to(x.dtype)
    return x


def apply_rotary_half_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """In place, Gemma convention: element i < rotary_dim/2 pairs with element i + rotary_dim/2
    (keras_nlp's CachedGemmaAttention._apply_rope, which example/gemma/keras_nlp.patch:6-23 calls)."""
    half = rotary_dim // 2
    x1, x2 = x[..., :half].float(), x[..., half:rotary_dim].float()
    c, s = cos[:, None, :], sin[:, None, :]
    x[..., :half] = (x1 * c - x2 * s).to(x.dtype)
    x[..., half:rotary_dim] = (x2 * c + x1 * s).to(x.dtype)
    return x


def _rotary_qk_torch_(qkv, cos, sin, rotary_dim, half_split=False):
    fn = apply_rotary_half_ if half_split else apply_rotary_
    fn(qkv[:, :, 0], cos, sin, rotary_dim)
    fn(qkv[:, :, 1], cos, sin, rotary_dim)
    return qkv


def _kv_append_torch_(k_cache, v_cache, k_new, v_new, position):
    k_cache[:, position] = k_new
    v_cache[:, position] = v_new


def _residual_add_torch(x, partial, bias=None, out=None):
    t = partial if bias is None else (partial.float() + bias.float()).to(x.dtype)
    return x + t.view(x.shape)


# ----------------------------------------------------------------------------- GPT-J prefill layer

@dataclass
class GptJLayerWeights:
    """This rank's shard.  Full shapes: wqkv [4096, 12288], wo [4096, 4096], w1 [4096, 16384],
    b1 [16384], w2 [16384, 4096], b2 [4096]."""
    wqkv: torch.Tensor
    wo: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor
    heads_local: int
    head_dim: int
    rotary_dim: int

    @staticmethod
    def shard(full: dict, num_heads: int, head_dim: int, rotary_dim: int, rank: int, world: int):
        return GptJLayerWeights(
            wqkv=shard_qkv_weight(full["wqkv"], num_heads, head_dim, rank, world),
            wo=shard_rows(full["wo"], rank, world),          # rows follow the heads
            w1=shard_columns(full["w1"], rank, world),
            b1=shard_columns(full["b1"], rank, world),
            w2=shard_rows(full["w2"], rank, world),
            b2=full["b2"],
            heads_local=num_heads // world, head_dim=head_dim, rotary_dim=rotary_dim)


def gptj_layer_prefill(x: torch.Tensor, w: GptJLayerWeights, ops, group=None, rope=None, reduce=None,
                       comm=None, fused_exchange: bool = False) -> torch.Tensor:
    """GPT-J block, prefill: y = x + Attn(LN(x)) + MLP(LN(x)), x [B, S, hidden] replicated on every
    rank.  The attention-output and MLP-down partial sums are added locally (the second GEMM takes
    the first as its C operand with beta = 1), so the block needs ONE all-reduce.  `rope` may carry
    precomputed (cos, sin) tables for positions 0..S-1, which keeps the step free of host work (and
    capturable in a CUDA graph).  `reduce(t, group)` replaces the all-reduce call (a caller that
    records the step in pieces around the exchange passes its own).  With `comm` (a
    comm.Communicator) the partial sum is produced straight into the NVLink exchange buffer and
    reduced there by libixk's own all-reduce kernel: no NCCL call, so the whole step is one stream of
    kernel launches that a CUDA graph can hold.  With `fused_exchange` as well, the down projection
    stores each row block of its result into the exchange buffer of the rank that owns it while it
    computes the next tiles, and the rest of the exchange (sum of the slots, bias, residual add,
    rows written to every rank) is one more kernel; the result is then a view of the exchange buffer
    (valid until the next step) with the same bits as the other paths."""
    B, S, hidden = x.shape
    hl, hd = w.heads_local, w.head_dim
    rows = B * S
    fused = comm is not None and fused_exchange and comm.world > 1
    h = _glue(ops, "layer_norm", layer_norm)(x).view(rows, hidden)
    qkv = ops.gemm(h, w.wqkv).view(B, S, 3, hl, hd)
    cos, sin = rope if rope is not None else rotary_tables(torch.arange(S, device=x.device), w.rotary_dim)
    _glue(ops, "rotary_qk_", _rotary_qk_torch_)(qkv, cos, sin, w.rotary_dim)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))        # [B, hl, S, hd] views, no copies
    ctx = torch.empty(B, S, hl, hd, dtype=x.dtype, device=x.device)
    ops.attention(q, k, v, ctx.permute(0, 2, 1, 3), scale=1.0 / math.sqrt(hd), causal=True)
    slot = comm.view(0, (rows, hidden), x.dtype) if comm is not None and not fused else None
    attn_partial = ops.gemm(ctx.view(rows, hl * hd), w.wo, out=slot)
    up = ops.gemm(h, w.w1, bias=w.b1, epilogue="BIAS_GELU")
    if fused:
        nbytes = rows * hidden * x.element_size()
        comm.gemm_scatter(up, w.w2, 0, c=attn_partial, beta=1.0)          # slots at [0, nbytes) of every rank's buffer
        y = comm.all_reduce_scattered(0, comm.view(nbytes, (rows, hidden), x.dtype), x=x.view(rows, hidden), bias=w.b2)
        return y.view(B, S, hidden)
    partial = ops.gemm(up, w.w2, c=attn_partial, beta=1.0, out=attn_partial)   # in place: C aliases D
    if comm is not None:
        partial = comm.all_reduce(partial)              # in place in the exchange buffer
    else:
        partial = (reduce or all_reduce_sum)(partial, group)
    return _glue(ops, "residual_add", _residual_add_torch)(x, partial, w.b2)


def gptj_layer_flops(B, S, hidden=4096, heads=16, head_dim=256, ffn=16384):
    m = B * S
    return (2.0 * m * hidden * 3 * heads * head_dim + 4.0 * B * heads * head_dim * S * (S + 1) / 2 +
            2.0 * m * heads * head_dim * hidden + 2.0 * m * hidden * ffn * 2)


# ----------------------------------------------------------------------------- Gemma decode step

@dataclass
class GemmaLayerWeights:
    """This rank's shard.  Full shapes: wqkv [3072, 12288], wo [4096, 3072], wgate/wup [3072, 24576],
    wdown [24576, 3072]; norm_attn / norm_mlp [3072]: the learned scales w of the two RMSNorms,
    applied as (1 + w), replicated on every rank (None = unit gain).  The gate and up shards are
    kept side by side in one matrix (wgateup [3072, 2 * columns]: one GEMM serves both); wgate and
    wup are its two halves as views."""
    wqkv: torch.Tensor
    wo: torch.Tensor
    wgateup: torch.Tensor
    wdown: torch.Tensor
    heads_local: int
    head_dim: int
    norm_attn: Optional[torch.Tensor] = None
    norm_mlp: Optional[torch.Tensor] = None

    @property
    def wgate(self) -> torch.Tensor:
        return self.wgateup[:, :self.wgateup.shape[1] // 2]

    @property
    def wup(self) -> torch.Tensor:
        return self.wgateup[:, self.wgateup.shape[1] // 2:]

    @staticmethod
    def shard(full: dict, num_heads: int, head_dim: int, rank: int, world: int):
        return GemmaLayerWeights(
            wqkv=shard_qkv_weight(full["wqkv"], num_heads, head_dim, rank, world),
            wo=shard_rows(full["wo"], rank, world),
            wgateup=torch.cat((shard_columns(full["wgate"], rank, world), shard_columns(full["wup"], rank, world)), dim=1),
            wdown=shard_rows(full["wdown"], rank, world),
            heads_local=num_heads // world, head_dim=head_dim,
            norm_attn=full.get("norm_attn"), norm_mlp=full.get("norm_mlp"))


def gemma_decode_step(x: torch.Tensor, w: GemmaLayerWeights, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      position: int, ops, group=None, workspace=None, rope=None, reduce=None, comm=None) -> torch.Tensor:
    """One new token per sequence: x [B, 1, hidden]; k_cache / v_cache [B, T, heads_local, head_dim]
    (this rank's heads) are updated in place at `position` and attended over [0, position].
    Two all-reduces: after the attention output projection and after the MLP down projection.
    `rope` may carry the precomputed (cos, sin) row for `position` (no host work in the step).
    With `comm` (a comm.Communicator) each row-parallel projection writes its partial into the
    NVLink exchange buffer and one libixk kernel does the exchange and the residual add that
    follows it (the two partials use different offsets, so the second exchange never waits for
    readers of the first).  Numerics are the Gemma block's: RMSNorm with the (1 + w) scale,
    rotary embedding on half-split pairs over the whole head, GeGLU with the tanh GELU."""
    B, _, hidden = x.shape
    hl, hd = w.heads_local, w.head_dim
    norm = _glue(ops, "rms_norm", rms_norm)
    add = _glue(ops, "residual_add", _residual_add_torch)
    h = norm(x, gain=w.norm_attn).view(B, hidden)
    qkv = ops.gemm(h, w.wqkv).view(B, 1, 3, hl, hd)
    cos, sin = rope if rope is not None else rotary_tables(torch.tensor([position], device=x.device), hd)
    _glue(ops, "rotary_qk_", _rotary_qk_torch_)(qkv, cos, sin, hd, half_split=True)
    _glue(ops, "kv_append_", _kv_append_torch_)(k_cache, v_cache, qkv[:, 0, 1], qkv[:, 0, 2], position)
    T = position + 1
    q = qkv[:, :, 0].permute(0, 2, 1, 3)                                   # [B, hl, 1, hd]
    ctx = torch.empty(B, 1, hl, hd, dtype=x.dtype, device=x.device)
    ops.attention(q, k_cache[:, :T].permute(0, 2, 1, 3), v_cache[:, :T].permute(0, 2, 1, 3),
                  ctx.permute(0, 2, 1, 3), scale=1.0 / math.sqrt(hd), causal=False, workspace=workspace)
    reduce = reduce or all_reduce_sum
    if comm is not None:
        nbytes = (B * hidden * x.element_size() + 255) // 256 * 256
        part = ops.gemm(ctx.view(B, hl * hd), w.wo, out=comm.view(0, (B, hidden), x.dtype))
        x1 = comm.all_reduce_residual(part, x)
    else:
        x1 = add(x, reduce(ops.gemm(ctx.view(B, hl * hd), w.wo), group))
    h2 = norm(x1, gain=w.norm_mlp).view(B, hidden)
    fused = getattr(ops, "gemm_geglu", None)
    act = fused(h2, w.wgateup) if fused is not None else None     # one GEMM for gate and up, GeGLU in its second pass
    if act is None:
        act = ops.gemm(h2, w.wgate, epilogue="GELU") * ops.gemm(h2, w.wup)
    if comm is not None:
        part = ops.gemm(act, w.wdown, out=comm.view(nbytes, (B, hidden), x.dtype))
        return comm.all_reduce_residual(part, x1)
    return add(x1, reduce(ops.gemm(act, w.wdown), group))


def gemma_decode_bytes(B, T, hidden=3072, heads=16, head_dim=256, ffn=24576, elem=2):
    """Algorithmic HBM bytes of one decode step: K and V once, every weight once."""
    attn = 2.0 * B * heads * T * head_dim * elem + 2.0 * B * heads * head_dim * elem
    weights = (hidden * 3 * heads * head_dim + heads * head_dim * hidden + 2 * hidden * ffn + ffn * hidden) * elem
    return attn + weights
