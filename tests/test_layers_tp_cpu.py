"""CPU, two gloo ranks: the tensor-parallel layer drivers — sharding by heads / columns / rows, the
local partial-sum fusion and the all-reduce — against the un-sharded layer oracle.  The two custom
calls are stood in for by the CPU oracle here (this is a test of the host-side logic; the CUDA
kernels have their own GPU tests)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleOps:
    """gemm / attention with the package's call signature, evaluated by the CPU oracle."""

    def __init__(self, orc):
        self.orc = orc

    def gemm(self, x, w, *, bias=None, c=None, beta=0.0, epilogue="DEFAULT", out=None):
        f = lambda t: None if t is None else t.float().numpy()
        res = self.orc.gemm_epilogue(f(x) @ f(w), f(bias), f(c), beta, epilogue, self.orc.BF16)
        res = torch.from_numpy(res).to(x.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def attention(self, q, k, v, out, *, scale, causal, workspace=None):
        f = lambda t: t.float().numpy()
        o, _ = self.orc.fmha_forward(f(q), f(k), f(v), None, head_scale=scale, causal=causal)
        out.copy_(torch.from_numpy(o).to(out.dtype))
        return out


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_weights(seed, hidden, heads, head_dim, ffn, gemma):
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: (torch.randn(*shape, generator=g) * 0.05).bfloat16()
    if gemma:
        return {"wqkv": r(hidden, 3 * heads * head_dim), "wo": r(heads * head_dim, hidden), "wgate": r(hidden, ffn),
                "wup": r(hidden, ffn), "wdown": r(ffn, hidden),
            "norm_attn": r(hidden), "norm_mlp": r(hidden)}
    return {"wqkv": r(hidden, 3 * heads * head_dim), "wo": r(heads * head_dim, hidden), "w1": r(hidden, ffn),
            "b1": r(ffn), "w2": r(ffn, hidden), "b2": r(hidden)}


def _worker(rank, world, port, result_queue):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = entry.load_package()
        orc = entry.load_oracle()
        from oracle import layers_oracle
        import importlib
        layers = importlib.import_module("ixk_b200.layers")
        ops = OracleOps(orc)
        f = lambda t: t.float().numpy()

        # ---- GPT-J block, prefill
        hidden, heads, hd, rot, ffn, B, S = 64, 4, 16, 8, 128, 2, 24
        full = _make_weights(1, hidden, heads, hd, ffn, gemma=False)
        g = torch.Generator().manual_seed(2)
        x = torch.randn(B, S, hidden, generator=g).bfloat16()
        w = layers.GptJLayerWeights.shard(full, heads, hd, rot, rank, world)
        assert w.wqkv.shape == (hidden, 3 * heads * hd // world) and w.wo.shape == (heads * hd // world, hidden)
        y = layers.gptj_layer_prefill(x, w, ops)
        # the exchange call is pluggable (a caller that records the step in pieces passes its own)
        calls = []
        y_hook = layers.gptj_layer_prefill(x, w, ops, reduce=lambda t, group=None: (calls.append(tuple(t.shape)),
                                                                                    layers.all_reduce_sum(t, group))[1])
        assert calls == [(B * S, hidden)] and torch.equal(y, y_hook)
        want = layers_oracle.gptj_layer_prefill(f(x), {k: f(v) for k, v in full.items()}, heads, hd, rot)
        err_gptj = float(np.abs(f(y) - want).max())

        # ---- Gemma decode step
        hidden, heads, hd, ffn, B, T = 48, 4, 16, 96, 3, 40
        full = _make_weights(3, hidden, heads, hd, ffn, gemma=True)
        x = torch.randn(B, 1, hidden, generator=g).bfloat16()
        kc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
        vc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
        h0, h1 = layers.shard_range(heads, rank, world)
        w = layers.GemmaLayerWeights.shard(full, heads, hd, rank, world)
        k_loc, v_loc = kc[:, :, h0:h1].contiguous(), vc[:, :, h0:h1].contiguous()
        y = layers.gemma_decode_step(x, w, k_loc, v_loc, T - 1, ops)
        calls = []
        y_hook = layers.gemma_decode_step(x, w, k_loc.clone(), v_loc.clone(), T - 1, ops,
                                          reduce=lambda t, group=None: (calls.append(tuple(t.shape)),
                                                                        layers.all_reduce_sum(t, group))[1])
        assert len(calls) == 2 and torch.equal(y, y_hook)
        want = layers_oracle.gemma_decode_step(f(x), {k: f(v) for k, v in full.items()}, f(kc), f(vc), T - 1, heads, hd)
        err_gemma = float(np.abs(f(y) - want).max())
        cache_written = bool((k_loc[:, T - 1] != kc[:, T - 1, h0:h1]).any())
        result_queue.put((rank, err_gptj, err_gemma, cache_written))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_tensor_parallel_layers_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err_gptj, err_gemma, cache_written in results:
        # bf16 storage of activations of O(1): a few ulps of 2^-8 after the partial sums are reduced
        assert err_gptj < 6e-2, (rank, err_gptj)
        assert err_gemma < 6e-2, (rank, err_gemma)
        assert cache_written


def test_shard_helpers(pkg):
    import importlib
    layers = importlib.import_module("ixk_b200.layers")
    assert layers.shard_range(16, 3, 8) == (6, 8)
    with pytest.raises(ValueError):
        layers.shard_range(10, 0, 4)
    w = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).view(2, 3 * 4 * 5)       # hidden 2, 4 heads x dim 5
    s = layers.shard_qkv_weight(w, 4, 5, rank=1, world=2)                          # heads 2,3 of q | k | v
    full = w.view(2, 3, 4, 5)
    assert torch.equal(s.view(2, 3, 2, 5), full[:, :, 2:4])
    assert torch.equal(layers.shard_columns(w, 0, 4), w[:, :15])
    assert torch.equal(layers.shard_rows(w.t().contiguous(), 1, 2), w.t()[30:])
    assert layers.gptj_layer_flops(4, 2048) == pytest.approx(3.4360e12, rel=1e-3)
    assert layers.gemma_decode_bytes(64, 4096) == pytest.approx(4.2960e9 + 553.6e6, rel=2e-3)
