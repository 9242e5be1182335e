"""GPU (one device): libixk's NVLink all-reduce kernels and the bounded waits around them.

Two ranks that wait for each other must never run as separate launches on ONE GPU, so the
two-rank cases here are arranged so that no kernel ever waits: both "ranks" are communicators on
the same device, connected by plain pointers (the way ranks that share a process connect), and
the flags a rank would wait for are written from the host before its kernel is launched.  Rank 0
runs to completion, then rank 1 (whose flags rank 0's kernel has set by then).  The real
two-process, two-GPU run is tests/test_layers_tp_gpu.py.

Sums of two 16-bit values are exact in fp32 and rounded once, so results are compared bit for bit
with (a.float() + b.float()).to(dtype)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
HEADER_BYTES = 8192          # flags in front of the exchange buffer (csrc/comm_sm100.cu: Flags)
MAX_BLOCKS, MAX_RANKS = 64, 8


class RawComm:
    """ixk_comm_* through ctypes, without torch.distributed."""

    def __init__(self, pkg, rank, world, nbytes, cuda):
        self.pkg, self.lib, self.rank, self.world, self.nbytes = pkg, pkg.load_library(), rank, world, nbytes
        self.h = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        pkg._check(self.lib.ixk_comm_create(rank, world, nbytes, ctypes.byref(self.h), handle))
        self.base = self.lib.ixk_comm_base(self.h)
        from importlib import import_module
        raw = import_module("ixk_b200.comm")._RawCudaMemory(self.base, HEADER_BYTES + nbytes)
        self.mem = torch.as_tensor(raw, device=cuda)
        self.flags = self.mem[:2 * MAX_BLOCKS * MAX_RANKS * 4].view(torch.int32).view(2, MAX_BLOCKS, MAX_RANKS)
        self.data = self.mem[HEADER_BYTES:]

    def connect(self, others):
        arr = (ctypes.c_void_p * self.world)(*[c.base for c in others])
        self.pkg._check(self.lib.ixk_comm_connect_pointers(self.h, arr))

    def view(self, offset, n, dtype):
        return self.data[offset:offset + n * torch.empty((), dtype=dtype).element_size()].view(dtype)

    def all_reduce(self, dtype, offset, out, count, kind=0):
        return self.lib.ixk_all_reduce(self.h, self.pkg._TORCH_TO_IXK[dtype], kind, offset, out.data_ptr(), count,
                                       torch.cuda.current_stream().cuda_stream)

    def close(self):
        torch.cuda.synchronize()
        self.flags = self.data = self.mem = None
        self.pkg._check(self.lib.ixk_comm_destroy(self.h))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_single_rank_is_a_copy_and_the_epilogue(pkg, cuda, dtype):
    n = 4096 * 3 + 5                    # a tail behind the last whole 16-byte vector
    c = RawComm(pkg, 0, 1, 1 << 20, cuda)
    try:
        g = torch.Generator(device="cuda").manual_seed(1)
        src = torch.randn(n, generator=g, device=cuda).to(dtype)
        c.view(256, n, dtype).copy_(src)
        out = torch.zeros(n, dtype=dtype, device=cuda)
        assert c.all_reduce(dtype, 256, out, n) == pkg.IXK_OK
        assert torch.equal(out, src)
        # fused residual add with a bias row: out = x + round(sum + bias)
        rows, cols = 24, 512
        x = torch.randn(rows, cols, generator=g, device=cuda).to(dtype)
        bias = torch.randn(cols, generator=g, device=cuda).to(dtype)
        part = torch.randn(rows, cols, generator=g, device=cuda).to(dtype)
        c.view(0, rows * cols, dtype).copy_(part.flatten())
        got = torch.empty_like(x)
        st = c.lib.ixk_all_reduce_residual(c.h, pkg._TORCH_TO_IXK[dtype], 0, x.data_ptr(), bias.data_ptr(), got.data_ptr(),
                                           rows, cols, torch.cuda.current_stream().cuda_stream)
        assert st == pkg.IXK_OK
        want = (x.float() + (part.float() + bias.float()).to(dtype).float()).to(dtype)
        assert torch.equal(got, want)
        if dtype != torch.float32:       # the stand-alone residual add takes 16-bit types only
            assert torch.equal(got, pkg.residual_add(x, part, bias))
    finally:
        c.close()


@pytest.mark.parametrize("algo", ["one-shot", "two-shot"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
def test_two_ranks_on_one_device_without_any_wait(pkg, cuda, monkeypatch, algo, dtype):
    monkeypatch.setenv("IXK_ALLREDUCE_ALGO", "2" if algo == "two-shot" else "1")
    n = 300000 + 3                                  # several CTAs, an uneven split, a tail
    nbytes = 4 << 20
    a, b = RawComm(pkg, 0, 2, nbytes, cuda), RawComm(pkg, 1, 2, nbytes, cuda)
    try:
        a.connect([a, b])
        b.connect([a, b])
        g = torch.Generator(device="cuda").manual_seed(2)
        va = torch.randint(-50, 50, (n,), generator=g, device=cuda).to(dtype)
        vb = torch.randint(-50, 50, (n,), generator=g, device=cuda).to(dtype)
        in_off, out_off = 0, 2 << 20
        for gen in (1, 2):                          # two calls in a row: the generation counters advance
            va, vb = va + 1, vb * 2
            a.view(in_off, n, dtype).copy_(va)
            b.view(in_off, n, dtype).copy_(vb)
            a.view(out_off, n, dtype).zero_()
            b.view(out_off, n, dtype).zero_()
            want = (va.float() + vb.float()).to(dtype)
            # rank 0 finds rank 1's flags already there (written by the host): it never waits
            a.flags[:, :, 1] = gen
            torch.cuda.synchronize()
            assert a.all_reduce(dtype, in_off, a.view(out_off, n, dtype), n) == pkg.IXK_OK
            torch.cuda.synchronize()
            assert pkg.device_status() == 0
            # rank 1 runs after rank 0 has finished, which has set rank 1's flags for every CTA it used
            assert b.all_reduce(dtype, in_off, b.view(out_off, n, dtype), n) == pkg.IXK_OK
            torch.cuda.synchronize()
            assert pkg.device_status() == 0
            assert torch.equal(a.view(out_off, n, dtype), want), f"rank 0, call {gen}"
            assert torch.equal(b.view(out_off, n, dtype), want), f"rank 1, call {gen}"
        # other reduction kinds (ccl_ops.cc:656-779), one-shot to a private buffer
        if algo == "one-shot":
            for kind, fn in ((1, torch.mul), (2, torch.minimum), (3, torch.maximum)):
                a.flags[:, :, 1] = 3 + kind - 1
                torch.cuda.synchronize()
                out = torch.empty(n, dtype=dtype, device=cuda)
                assert a.all_reduce(dtype, in_off, out, n, kind=kind) == pkg.IXK_OK
                assert torch.equal(out, fn(va.float(), vb.float()).to(dtype))
                # keep rank 1's counters in step with rank 0's
                assert b.all_reduce(dtype, in_off, torch.empty(n, dtype=dtype, device=cuda), n, kind=kind) == pkg.IXK_OK
                torch.cuda.synchronize()
    finally:
        a.close()
        b.close()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
def test_reduce_scatter_and_all_gather_two_ranks_without_any_wait(pkg, cuda, dtype):
    """The two halves of the two-shot all-reduce as calls of their own (ccl_ops.cc:518-559, :268-294),
    with the same no-wait arrangement: flags written from the host, rank 0 first, then rank 1."""
    per_rank = 40000                                     # elements per rank: whole 16-byte vectors
    a, b = RawComm(pkg, 0, 2, 4 << 20, cuda), RawComm(pkg, 1, 2, 4 << 20, cuda)
    try:
        a.connect([a, b])
        b.connect([a, b])
        lib, k = a.lib, pkg._TORCH_TO_IXK[dtype]
        stream = torch.cuda.current_stream().cuda_stream
        g = torch.Generator(device="cuda").manual_seed(3)
        va = torch.randint(-50, 50, (2 * per_rank,), generator=g, device=cuda).to(dtype)
        vb = torch.randint(-50, 50, (2 * per_rank,), generator=g, device=cuda).to(dtype)
        a.view(0, 2 * per_rank, dtype).copy_(va)
        b.view(0, 2 * per_rank, dtype).copy_(vb)
        want = (va.float() + vb.float()).to(dtype)
        oa = torch.zeros(per_rank, dtype=dtype, device=cuda)
        ob = torch.zeros(per_rank, dtype=dtype, device=cuda)
        a.flags[:, :, 1] = 1                             # generation 1: reduce-scatter
        torch.cuda.synchronize()
        assert lib.ixk_reduce_scatter(a.h, k, 0, 0, oa.data_ptr(), per_rank, stream) == pkg.IXK_OK
        torch.cuda.synchronize()
        assert lib.ixk_reduce_scatter(b.h, k, 0, 0, ob.data_ptr(), per_rank, stream) == pkg.IXK_OK
        torch.cuda.synchronize()
        assert torch.equal(oa, want[:per_rank]) and torch.equal(ob, want[per_rank:])
        # generation 2: all-gather of the two reduced pieces = the all-reduce result on both ranks
        off = 2 << 20
        a.flags[:, :, 1] = 2
        torch.cuda.synchronize()
        assert lib.ixk_all_gather(a.h, k, oa.data_ptr(), off, per_rank, stream) == pkg.IXK_OK
        torch.cuda.synchronize()
        assert lib.ixk_all_gather(b.h, k, ob.data_ptr(), off, per_rank, stream) == pkg.IXK_OK
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        assert torch.equal(a.view(off, 2 * per_rank, dtype), want) and torch.equal(b.view(off, 2 * per_rank, dtype), want)
        # a piece that is not a whole number of vectors, and a local buffer inside the exchanged range
        assert lib.ixk_reduce_scatter(a.h, k, 0, 0, oa.data_ptr(), 3, stream) == pkg.IXK_UNIMPLEMENTED
        inside = a.view(0, per_rank, dtype)
        assert lib.ixk_reduce_scatter(a.h, k, 0, 0, inside.data_ptr(), per_rank, stream) == pkg.IXK_INVALID_ARGUMENT
    finally:
        a.close()
        b.close()


def test_projection_scattered_into_the_owners_slots_then_reduced_two_ranks_without_any_wait(pkg, cuda):
    """ixk_gemm_scatter + ixk_all_reduce_scattered against ixk_gemm + sum + ixk_residual_add, bit for
    bit.  Both ranks' projections run first (they wait for nobody), then the second halves in the
    no-wait arrangement."""
    M, N, K = 2560, 2048, 512                       # 10 x 8 tiles of 256 x 256: the CTA-pair kernel
    slots_off, out_off = 0, M * N * 2
    a, b = RawComm(pkg, 0, 2, 2 * M * N * 2, cuda), RawComm(pkg, 1, 2, 2 * M * N * 2, cuda)
    try:
        a.connect([a, b])
        b.connect([a, b])
        g = torch.Generator(device="cuda").manual_seed(4)
        rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=g, device=cuda) * s).bfloat16()
        lhs, rhs, add = [rnd(M, K), rnd(M, K)], [rnd(K, N, s=0.05), rnd(K, N, s=0.05)], [rnd(M, N), rnd(M, N)]
        x, bias = rnd(M, N), rnd(N)
        stream = torch.cuda.current_stream().cuda_stream
        for c in (a, b):
            c.data.zero_()
        for r, c in enumerate((a, b)):
            attrs = pkg.gemm_attrs_for(lhs[r], rhs[r], torch.empty((M, N), device="meta", dtype=torch.bfloat16), 1.0)
            d = pkg.gemm_desc_from_attrs(attrs, "DEFAULT")
            st = c.lib.ixk_gemm_scatter(c.h, ctypes.byref(d), lhs[r].data_ptr(), rhs[r].data_ptr(), add[r].data_ptr(), None,
                                        slots_off, stream)
            assert st == pkg.IXK_OK, a.lib.ixk_last_error().decode()
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        part = [pkg.gemm(lhs[r], rhs[r], c=add[r], beta=1.0) for r in range(2)]
        half = M // 2
        # rank o's slot s = rows [o * half, (o + 1) * half) of rank s's partial
        for o, c in enumerate((a, b)):
            for src in range(2):
                slot = c.view(slots_off + src * half * N * 2, half * N, torch.bfloat16).view(half, N)
                assert torch.equal(slot, part[src][o * half:(o + 1) * half]), f"slot {src} of rank {o}"
        total = (part[0].float() + part[1].float()).bfloat16()
        want = pkg.residual_add(x, total, bias)
        k = pkg._TORCH_TO_IXK[torch.bfloat16]
        a.flags[:, :, 1] = 1
        torch.cuda.synchronize()
        for c in (a, b):
            assert c.lib.ixk_all_reduce_scattered(c.h, k, slots_off, x.data_ptr(), bias.data_ptr(), out_off, M, N,
                                                  stream) == pkg.IXK_OK, a.lib.ixk_last_error().decode()
            torch.cuda.synchronize()
            assert pkg.device_status() == 0
        for c in (a, b):
            assert torch.equal(c.view(out_off, M * N, torch.bfloat16).view(M, N), want)
        # without the residual: the plain sum
        a.flags[:, :, 1] = 2
        torch.cuda.synchronize()
        for c in (a, b):
            assert c.lib.ixk_all_reduce_scattered(c.h, k, slots_off, None, None, out_off, M, N, stream) == pkg.IXK_OK
            torch.cuda.synchronize()
        assert torch.equal(a.view(out_off, M * N, torch.bfloat16).view(M, N), total)
        assert torch.equal(b.view(out_off, M * N, torch.bfloat16).view(M, N), total)
        # shapes the scattered store does not take; ranges that do not fit
        small = pkg.gemm_desc_from_attrs(pkg.gemm_attrs_for(lhs[0][:256], rhs[0], torch.empty((256, N), device="meta",
                                                                                             dtype=torch.bfloat16)), "DEFAULT")
        assert a.lib.ixk_gemm_scatter(a.h, ctypes.byref(small), lhs[0].data_ptr(), rhs[0].data_ptr(), None, None, 0,
                                      stream) == pkg.IXK_UNIMPLEMENTED
        assert a.lib.ixk_gemm_scatter(a.h, ctypes.byref(d), lhs[0].data_ptr(), rhs[0].data_ptr(), add[0].data_ptr(), None,
                                      out_off + 16, stream) == pkg.IXK_INVALID_ARGUMENT
        assert a.lib.ixk_all_reduce_scattered(a.h, k, slots_off, None, None, out_off - 16, M, N, stream) == pkg.IXK_INVALID_ARGUMENT
        assert a.lib.ixk_gemm_scatter(None, ctypes.byref(d), lhs[0].data_ptr(), rhs[0].data_ptr(), None, None, 0,
                                      stream) == pkg.IXK_INVALID_ARGUMENT
    finally:
        a.close()
        b.close()


def test_eight_ranks_on_one_device_without_any_wait(pkg, cuda):
    """The widest communicator (8 ranks: the unrolled kernels, the slice and slot arithmetic, eight
    output tensor maps of the scattered projection), as eight communicators on one device run one
    after the other with every flag written from the host beforehand, so that no kernel waits."""
    world = 8
    M, N, K = 2048, 2560, 256                       # 8 x 10 tiles of 256 x 256: the CTA-pair kernel; 256 rows per rank
    slots_off, out_off = 0, M * N * 2
    ranks = [RawComm(pkg, r, world, 2 * M * N * 2, cuda) for r in range(world)]
    try:
        for c in ranks:
            c.connect(ranks)
        stream = torch.cuda.current_stream().cuda_stream
        k = pkg._TORCH_TO_IXK[torch.bfloat16]
        g = torch.Generator(device="cuda").manual_seed(8)

        def preset():
            """Every CTA slot of every rank finds every peer at the generation it is about to use
            (one more than the slot's own counter, which sits behind the flags in the header; the
            ranks have made the same calls, so their counters agree)."""
            for c in ranks:
                counters = c.mem[2 * MAX_BLOCKS * MAX_RANKS * 4:2 * MAX_BLOCKS * MAX_RANKS * 4 + MAX_BLOCKS * 4].view(torch.int32)
                c.flags[:, :, :] = (counters + 1)[None, :, None]
            torch.cuda.synchronize()

        def in_rank_order(parts):                    # fp32 sum in rank order, rounded once: what the kernels compute
            acc = parts[0].float()
            for p_ in parts[1:]:
                acc = acc + p_.float()
            return acc

        # one-shot (a decode step's partial) with the residual epilogue, and the plain sum to a private buffer
        rows, cols = 64, 3072
        parts = [torch.randn(rows, cols, generator=g, device=cuda).bfloat16() for _ in range(world)]
        x = torch.randn(rows, cols, generator=g, device=cuda).bfloat16()
        for c, p_ in zip(ranks, parts):
            c.view(0, rows * cols, torch.bfloat16).copy_(p_.flatten())
        total = in_rank_order(parts).bfloat16()
        preset()
        for c in ranks:
            got = torch.empty_like(x)
            assert c.lib.ixk_all_reduce_residual(c.h, k, 0, x.data_ptr(), None, got.data_ptr(), rows, cols, stream) == pkg.IXK_OK
            torch.cuda.synchronize()
            assert torch.equal(got, (x.float() + total.float()).bfloat16()), f"one-shot, rank {c.rank}"
        # two-shot, in place: rank r reduces slice r and writes it into every rank's buffer
        n = 3 * 1024 * 1024 + 8 * 5                  # the last rank's slice is longer than the others'
        big = [torch.randint(-20, 20, (n,), generator=g, device=cuda).bfloat16() for _ in range(world)]
        for c, p_ in zip(ranks, big):
            c.view(0, n, torch.bfloat16).copy_(p_)
        preset()
        for c in ranks:
            assert c.all_reduce(torch.bfloat16, 0, c.view(0, n, torch.bfloat16), n) == pkg.IXK_OK
            torch.cuda.synchronize()
        want = in_rank_order(big).bfloat16()
        for c in ranks:
            assert torch.equal(c.view(0, n, torch.bfloat16), want), f"two-shot, rank {c.rank}"
        assert pkg.device_status() == 0

        # the projection scattered over eight owners, then the second half with bias and residual
        lhs = [torch.randn(M, K, generator=g, device=cuda).bfloat16() for _ in range(world)]
        rhs = [(torch.randn(K, N, generator=g, device=cuda) * 0.06).bfloat16() for _ in range(world)]
        xr = torch.randn(M, N, generator=g, device=cuda).bfloat16()
        bias = torch.randn(N, generator=g, device=cuda).bfloat16()
        for c in ranks:
            c.data.zero_()
        for c in ranks:
            attrs = pkg.gemm_attrs_for(lhs[c.rank], rhs[c.rank], torch.empty((M, N), device="meta", dtype=torch.bfloat16))
            d = pkg.gemm_desc_from_attrs(attrs, "DEFAULT")
            assert c.lib.ixk_gemm_scatter(c.h, ctypes.byref(d), lhs[c.rank].data_ptr(), rhs[c.rank].data_ptr(), None, None,
                                          slots_off, stream) == pkg.IXK_OK, c.lib.ixk_last_error().decode()
        torch.cuda.synchronize()
        part = [pkg.gemm(lhs[r], rhs[r]) for r in range(world)]
        per = M // world
        for o, c in enumerate(ranks):                # rank o's slot s = rows [o * per, (o + 1) * per) of rank s's partial
            for src in (0, 3, 7):
                slot = c.view(slots_off + src * per * N * 2, per * N, torch.bfloat16).view(per, N)
                assert torch.equal(slot, part[src][o * per:(o + 1) * per]), f"slot {src} of rank {o}"
        want = pkg.residual_add(xr, in_rank_order(part).bfloat16(), bias)
        preset()
        for c in ranks:
            assert c.lib.ixk_all_reduce_scattered(c.h, k, slots_off, xr.data_ptr(), bias.data_ptr(), out_off, M, N,
                                                  stream) == pkg.IXK_OK, c.lib.ixk_last_error().decode()
            torch.cuda.synchronize()
        for c in ranks:
            assert torch.equal(c.view(out_off, M * N, torch.bfloat16).view(M, N), want), f"scattered, rank {c.rank}"
        assert pkg.device_status() == 0
    finally:
        for c in ranks:
            c.close()


def test_a_peer_that_never_arrives_ends_in_a_timeout_status(pkg, cuda):
    """The wait for a peer is bounded: with nobody on the other side the kernel gives up after its
    cycle budget, reports where, and leaves the device usable."""
    a, b = RawComm(pkg, 0, 2, 1 << 20, cuda), RawComm(pkg, 1, 2, 1 << 20, cuda)
    try:
        a.connect([a, b])
        pkg._check(a.lib.ixk_comm_set_wait_limit(a.h, 2_000_000))          # about a millisecond
        out = torch.zeros(1024, dtype=torch.bfloat16, device=cuda)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert a.all_reduce(torch.bfloat16, 0, out, 1024) == pkg.IXK_OK   # the launch itself succeeds
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 100.0                                 # ms: it gave up, it did not hang
        with pytest.raises(pkg.IxkError) as e:
            pkg.device_status()
        assert e.value.status == pkg.IXK_DEVICE_TIMEOUT and "301" in str(e.value)
        assert pkg.device_status() == 0                                    # read once, cleared
        x = torch.ones(64, 64, dtype=torch.bfloat16, device=cuda)
        assert torch.equal(pkg.gemm(x, x), torch.full((64, 64), 64.0, dtype=torch.bfloat16, device=cuda))
    finally:
        a.close()
        b.close()


def test_bounded_mbarrier_wait_gives_up_and_reports(pkg, cuda):
    """The wait every tensor-core kernel uses (mbarrier try_wait loop with a cycle budget), made to
    run out on purpose: site code 901 from the first warp, the second warp leaves through the
    CTA's abort flag, the kernel returns, the status word clears, the next launch is clean."""
    lib = pkg.load_library()
    cycles = torch.zeros(1, dtype=torch.int64, device=cuda)
    assert lib.ixk_selftest_bounded_wait(2_000_000, cycles.data_ptr(), torch.cuda.current_stream().cuda_stream) == pkg.IXK_OK
    torch.cuda.synchronize()
    spent = int(cycles.item())
    assert 2_000_000 <= spent < 50_000_000          # the first wait ran its budget, the second did not run its own (2e9)
    with pytest.raises(pkg.IxkError) as e:
        pkg.device_status()
    assert e.value.status == pkg.IXK_DEVICE_TIMEOUT and "901" in str(e.value)
    assert pkg.device_status() == 0
    assert lib.ixk_selftest_bounded_wait(0, None, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_selftest_bounded_wait(10 ** 9, None, None) == pkg.IXK_INVALID_ARGUMENT
    q = torch.randn(1, 1, 128, 64, device=cuda).bfloat16()
    o = torch.empty_like(q)
    pkg.fmha_forward_kernel(None, q, q, q, None, None, 0.0, o, None, 0.125, False)
    assert pkg.device_status() == 0 and bool(torch.isfinite(o.float()).all())


def test_argument_checks(pkg, cuda):
    lib = pkg.load_library()
    h = ctypes.c_void_p()
    assert lib.ixk_comm_create(2, 2, 1 << 20, ctypes.byref(h), None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_comm_create(0, 9, 1 << 20, ctypes.byref(h), None) == pkg.IXK_INVALID_ARGUMENT
    c = RawComm(pkg, 0, 2, 1 << 20, cuda)
    try:
        out = torch.zeros(16, dtype=torch.bfloat16, device=cuda)
        assert c.all_reduce(torch.bfloat16, 0, out, 16) == pkg.IXK_INVALID_ARGUMENT       # not connected
        c.connect([c, c])
        assert c.all_reduce(torch.bfloat16, 8, out, 16) == pkg.IXK_INVALID_ARGUMENT       # offset % 16
        assert c.all_reduce(torch.bfloat16, 0, out, (1 << 20)) == pkg.IXK_INVALID_ARGUMENT  # past the buffer
        assert c.all_reduce(torch.bfloat16, 0, out, 16, kind=7) == pkg.IXK_INVALID_ARGUMENT
        assert c.all_reduce(torch.bfloat16, 0, out, 0) == pkg.IXK_OK                        # empty: nothing launched
    finally:
        c.close()
