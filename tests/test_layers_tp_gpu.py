"""GPU, two ranks over NCCL (skipped on a single-GPU machine): the tensor-parallel layer drivers
with the real kernels — TP=2 must agree with the un-sharded numpy layer oracle, and the
all-reduce must leave both ranks with the same bits."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import importlib
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = entry.load_package()
        orc = entry.load_oracle()
        from oracle import layers_oracle
        layers = importlib.import_module("ixk_b200.layers")
        f = lambda t: t.float().cpu().numpy()
        hidden, heads, hd, rot, ffn, B, S = 512, 4, 128, 64, 1024, 2, 384
        g = torch.Generator().manual_seed(1)
        r = lambda *s: (torch.randn(*s, generator=g) * 0.02).bfloat16()
        full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "w1": r(hidden, ffn), "b1": r(ffn),
                "w2": r(ffn, hidden), "b2": r(hidden)}
        x = torch.randn(B, S, hidden, generator=g).bfloat16()
        w = layers.GptJLayerWeights.shard({k: v.to(dev) for k, v in full.items()}, heads, hd, rot, rank, world)
        y = layers.gptj_layer_prefill(x.to(dev), w, layers.KernelOps(pkg))
        want = layers_oracle.gptj_layer_prefill(f(x), {k: f(v) for k, v in full.items()}, heads, hd, rot)
        err = float(np.abs(f(y) - want).max())
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        q.put((rank, err, same, pkg.device_status()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_gptj_block_tp2_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=480) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err, same, status in results:
        assert err < 6e-2, (rank, err)
        assert same and status == 0
