"""GPU, two ranks, one process per GPU (skipped on a single-GPU machine): the tensor-parallel layer
drivers with the real kernels.  TP=2 must agree with the un-sharded numpy layer oracle and leave
both ranks with the same bits, with the exchange done by NCCL and by libixk's own NVLink
all-reduce (exchange buffers shared through CUDA IPC); the two must agree bit for bit at two
ranks (a sum of two 16-bit values is exact in fp32 and rounded once either way).  The all-reduce
itself is checked against ncclAllReduce on integer data, one-shot and two-shot."""
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
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # a rank sits an exchange out below: no NVLink multicast objects around it
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

        # ---- libixk's all-reduce against ncclAllReduce, bit for bit on integers
        comm_mod = importlib.import_module("ixk_b200.comm")
        comm = comm_mod.Communicator(pkg, rank, world, 32 << 20)
        checks = {}
        gi = torch.Generator(device=dev).manual_seed(100 + rank)
        for name, n in (("one_shot", 64 * 3072), ("two_shot", 3 * 1024 * 1024 + 8), ("tail", 1000 + 3)):
            for dt in (torch.bfloat16, torch.float32):
                v = torch.randint(-60, 60, (n,), generator=gi, device=dev).to(dt)
                slot = comm.view(0, (n,), dt)
                slot.copy_(v)
                want_ar = v.clone()
                dist.all_reduce(want_ar)
                priv = torch.empty_like(v)
                comm.all_reduce(slot, out=priv)                # result to a private buffer: one-shot
                torch.cuda.synchronize()
                ok_priv = torch.equal(priv, want_ar)
                comm.all_reduce(slot)                          # in place in the exchange buffer: two-shot when large
                torch.cuda.synchronize()
                checks[f"{name}_{dt}"] = ok_priv and torch.equal(slot, want_ar)
        # the two halves as calls of their own, against NCCL's
        n = 8 * 4096
        v = torch.randint(-60, 60, (world * n,), generator=gi, device=dev).to(torch.bfloat16)
        slot = comm.view(0, (world * n,), torch.bfloat16)
        slot.copy_(v)
        mine = torch.empty(n, dtype=torch.bfloat16, device=dev)
        comm.reduce_scatter(slot, mine)
        want_rs = torch.empty(n, dtype=torch.bfloat16, device=dev)
        dist.reduce_scatter_tensor(want_rs, v)
        gathered = comm.view(8 << 20, (world * n,), torch.bfloat16)
        comm.all_gather(mine, gathered)
        want_ag = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(want_ag, want_rs)
        torch.cuda.synchronize()
        checks["reduce_scatter"] = torch.equal(mine, want_rs)
        checks["all_gather"] = torch.equal(gathered, want_ag)
        # many calls back to back (the flags' generation counters, no host sync in between)
        slot = comm.view(0, (4096,), torch.float32)
        slot.fill_(1.0)
        for _ in range(20):
            comm.all_reduce(slot)
        torch.cuda.synchronize()
        checks["repeat"] = bool((slot == float(world) ** 20).all())

        # ---- the GPT-J block again, exchange through libixk
        y2 = layers.gptj_layer_prefill(x.to(dev), w, layers.KernelOps(pkg), comm=comm)
        checks["gptj_comm_equals_nccl"] = torch.equal(y, y2)
        # the projection that scatters its result + one exchange kernel (needs the CTA-pair GEMM: a wider case)
        hidden2, ffn2, B2, S2 = 2048, 2048, 2, 1280
        g2 = torch.Generator().manual_seed(5)
        r2 = lambda *s: (torch.randn(*s, generator=g2) * 0.02).bfloat16()
        full2 = {"wqkv": r2(hidden2, 3 * 16 * 128), "wo": r2(16 * 128, hidden2), "w1": r2(hidden2, ffn2), "b1": r2(ffn2),
                 "w2": r2(ffn2, hidden2), "b2": r2(hidden2)}
        w2 = layers.GptJLayerWeights.shard({k_: v_.to(dev) for k_, v_ in full2.items()}, 16, 128, rot, rank, world)
        x2 = (torch.randn(B2, S2, hidden2, generator=torch.Generator().manual_seed(6)) * 0.5).bfloat16().to(dev)
        y_unfused = layers.gptj_layer_prefill(x2, w2, layers.KernelOps(pkg), comm=comm).clone()
        # The scattered stores of the fused form land in the peers' buffers with no handshake (that is
        # the point), in the range the unfused step above still reads after its exchange: the ranks
        # meet before the range changes hands.  Steps of one form need no such meeting.
        torch.cuda.synchronize()
        dist.barrier()
        y_fused = layers.gptj_layer_prefill(x2, w2, layers.KernelOps(pkg), comm=comm, fused_exchange=True).clone()
        y_fused2 = layers.gptj_layer_prefill(x2, w2, layers.KernelOps(pkg), comm=comm, fused_exchange=True).clone()
        torch.cuda.synchronize()
        dist.barrier()
        checks["gptj_fused_exchange_twice_in_a_row"] = torch.equal(y_fused, y_fused2)
        torch.cuda.synchronize()
        checks["gptj_fused_exchange_equals_unfused"] = torch.equal(y_unfused, y_fused)
        checks["gptj_fused_exchange_finite"] = bool(torch.isfinite(y_fused.float()).all())

        # ---- Gemma decode step, TP=2: NCCL exchange, libixk exchange, CUDA-graph replay of the latter
        hidden, heads, hd, ffn, B, T = 384, 4, 256, 768, 6, 900
        g = torch.Generator().manual_seed(2)
        full = {"wqkv": r(hidden, 3 * heads * hd), "wo": r(heads * hd, hidden), "wgate": r(hidden, ffn),
                "wup": r(hidden, ffn), "wdown": r(ffn, hidden),
            "norm_attn": r(hidden), "norm_mlp": r(hidden)}
        xg = torch.randn(B, 1, hidden, generator=g).bfloat16()
        kc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
        vc = torch.randn(B, T, heads, hd, generator=g).bfloat16()
        h0, h1 = layers.shard_range(heads, rank, world)
        wg = layers.GemmaLayerWeights.shard({k: v.to(dev) for k, v in full.items()}, heads, hd, rank, world)
        want = layers_oracle.gemma_decode_step(f(xg), {k: f(v) for k, v in full.items()}, f(kc), f(vc), T - 1, heads, hd)
        ops = layers.KernelOps(pkg)
        local = lambda c: c[:, :, h0:h1].contiguous().to(dev)
        y_nccl = layers.gemma_decode_step(xg.to(dev), wg, local(kc), local(vc), T - 1, ops)
        y_comm = layers.gemma_decode_step(xg.to(dev), wg, local(kc), local(vc), T - 1, ops, comm=comm)
        err_gemma = float(np.abs(f(y_nccl) - want).max())
        checks["gemma_comm_equals_nccl"] = torch.equal(y_nccl, y_comm)
        # the step with its two exchanges inside one CUDA graph, replayed three times
        kd, vd, xd = local(kc), local(vc), xg.to(dev)
        ws = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
        rope = layers.rotary_tables(torch.tensor([T - 1], device=dev), hd)
        step = lambda: layers.gemma_decode_step(xd, wg, kd, vd, T - 1, ops, workspace=ws, rope=rope, comm=comm)
        step()
        torch.cuda.synchronize()
        dist.barrier()
        cap = torch.cuda.Stream()
        cap.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap):
            with torch.cuda.graph(graph, stream=cap, capture_error_mode="thread_local"):
                y_graph = step()
        torch.cuda.current_stream().wait_stream(cap)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        checks["gemma_graph_equals_eager"] = torch.equal(y_graph, y_comm)
        # the same step with the promise that consecutive exchanges never share a range (its two use
        # two offsets): the one-shot kernels then leave without their second meeting; 40 replays back
        # to back, where a rank that runs ahead would be caught rewriting a range still being read
        # (the promise is read when a call is issued: a new capture)
        comm.set_alternating(True)
        torch.cuda.synchronize()
        dist.barrier()
        cap.wait_stream(torch.cuda.current_stream())
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap):
            with torch.cuda.graph(graph2, stream=cap, capture_error_mode="thread_local"):
                y_alt = step()
        torch.cuda.current_stream().wait_stream(cap)
        for _ in range(40):
            graph2.replay()
        torch.cuda.synchronize()
        checks["gemma_alternating_equals_eager"] = torch.equal(y_alt, y_comm) and pkg.device_status() == 0
        comm.set_alternating(False)
        dist.barrier()
        # ---- a peer that does not show up: rank 1 sits this exchange out (it is between steps, nothing
        # of its own in flight); rank 0's kernel gives up after its cycle budget, reports where, and
        # the GPU stays usable.  The ranks then meet on the host and take the communicator down.
        torch.cuda.synchronize()
        dist.barrier()
        comm.set_wait_limit(20_000_000)                # about 10 ms
        if rank == 0:
            comm.all_reduce(comm.view(0, (4096,), torch.float32), out=torch.empty(4096, device=dev))
            try:
                pkg.device_status()
                checks["absent_peer_times_out"] = False
            except pkg.IxkError as e:
                checks["absent_peer_times_out"] = e.status == pkg.IXK_DEVICE_TIMEOUT and "301" in str(e)
            xs = torch.ones(64, 64, dtype=torch.bfloat16, device=dev)
            checks["usable_after_timeout"] = bool((pkg.gemm(xs, xs) == 64).all()) and pkg.device_status() == 0
        comm.close()
        q.put((rank, err, same, pkg.device_status(), err_gemma, checks))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_layers_and_all_reduce_tp2():
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
    for rank, err, same, status, err_gemma, checks in results:
        assert err < 6e-2, (rank, err)
        assert err_gemma < 6e-2, (rank, err_gemma)
        assert same and status == 0
        assert all(checks.values()), (rank, {k: v for k, v in checks.items() if not v})
