"""GPU: the attention entry point that allocates nothing (ixk_fmha_fwd_static_scratch).

Some hosts of this library cannot give it scratch memory and cannot let it allocate: a custom
call bound without a scratch allocator, or a process whose framework already owns the GPU's
memory pool.  For them the split-key decode path keeps its partials in a fixed array inside the
library.  This file checks, through the C ABI, that the result is the one the ordinary entry point
(caller-provided workspace) produces — bit for bit, since both run the same kernels — on two calls
in a row (the second one finds the first one's partials still in the array), that an oversized
problem is refused, and that the call really allocates nothing.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It also passes when run alone in a fresh process."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(cuda, B, N, F, T, H, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, N, F, H, generator=g).bfloat16().to(cuda)
    k = torch.randn(B, T, N, H, generator=g).bfloat16().to(cuda).permute(0, 2, 1, 3)   # cache layout [B,T,N,H]
    v = torch.randn(B, T, N, H, generator=g).bfloat16().to(cuda).permute(0, 2, 1, 3)
    return q, k, v


def _call_static(pkg, q, k, v, out, lse, causal=False):
    """Straight through the C ABI: descriptor + raw pointers, no torch allocation in between."""
    d = pkg._fmha_desc(q, k, v, None, out, q.shape[-1] ** -0.5, causal, 0.0)
    lib = pkg.load_library()
    return lib.ixk_fmha_fwd_static_scratch(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                           out.data_ptr(), lse.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_matches_the_workspace_entry_point_twice_in_a_row(pkg, cuda):
    lib = pkg.load_library()
    # two different problems, both on the split-key path (workspace > 0), run back to back
    cases = [(_inputs(cuda, 2, 4, 1, 4096, 256, seed=1), False), (_inputs(cuda, 3, 2, 2, 1500, 128, seed=2), True)]
    for round_ in range(2):
        for (q, k, v), causal in cases:
            B, N, F, H = q.shape
            d = pkg._fmha_desc(q, k, v, None, torch.empty_like(q), H ** -0.5, causal, 0.0)
            need = lib.ixk_fmha_fwd_workspace_bytes(ctypes.byref(d))
            assert 0 < need <= pkg.STATIC_SCRATCH_BYTES

            want = torch.full_like(q, float("nan"))
            want_lse = torch.full((B, N, F), float("nan"), dtype=torch.float32, device=cuda)
            ws = torch.empty(need, dtype=torch.uint8, device=cuda)
            pkg.fmha_forward_kernel(None, q, k, v, None, None, 0.0, want, want_lse, H ** -0.5, True, causal=causal,
                                    workspace=ws)

            got = torch.full_like(q, float("nan"))
            got_lse = torch.full((B, N, F), float("nan"), dtype=torch.float32, device=cuda)
            if round_ == 0:
                # The very first call on a device may be the one that makes the CUDA runtime load the
                # part of the library image that holds the array (module loading is lazy), so the
                # steady state is what is measured: one untimed call first.
                assert _call_static(pkg, q, k, v, got, got_lse, causal) == pkg.IXK_OK
            gc.collect()                                         # tensors of earlier tests that sit in reference cycles go now, not mid-measurement
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()           # the driver's view: sees any cudaMalloc, whoever makes it
            torch_before = torch.cuda.memory_allocated()
            assert _call_static(pkg, q, k, v, got, got_lse, causal) == pkg.IXK_OK
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before                     # no device memory was taken (or given back) by the call
            assert torch.cuda.memory_allocated() == torch_before  # and nothing went through torch's allocator either

            # same kernels, same split count → identical bits; the suite's tolerance (2e-2) as the outer bound
            assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
            assert torch.equal(got, want), f"round {round_}"
            assert torch.equal(got_lse, want_lse)


def test_python_wrapper_and_prefill_pass_through(pkg, orc, cuda):
    """The wrapper gives the oracle's answer; a prefill-sized problem (no scratch needed) also goes through."""
    q, k, v = _inputs(cuda, 1, 2, 1, 700, 64, seed=3)
    out = torch.empty_like(q)
    lse = torch.empty(1, 2, 1, dtype=torch.float32, device=cuda)
    pkg.fmha_forward_kernel_static_scratch(None, q, k, v, None, out, lse, 64 ** -0.5)
    f32 = lambda t: t.float().cpu().numpy()
    want, want_lse = orc.fmha_forward(f32(q), f32(k), f32(v), None, head_scale=64 ** -0.5)
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2, what="static scratch decode")
    orc.check_close(f32(lse), want_lse, rtol=2e-3, atol=2e-3, what="static scratch lse")

    g = torch.Generator().manual_seed(4)
    q = torch.randn(1, 2, 256, 128, generator=g).bfloat16().to(cuda)
    out = torch.empty_like(q)
    pkg.fmha_forward_kernel_static_scratch(None, q, q, q, None, out, None, 128 ** -0.5, causal=True)
    want, _ = orc.fmha_forward(f32(q), f32(q), f32(q), None, head_scale=128 ** -0.5, causal=True)
    orc.check_close(f32(out), want, rtol=2e-2, atol=2e-2, what="static scratch prefill")


def test_oversized_problem_is_refused_before_launch(pkg, cuda):
    # 2367 (batch, head) rows -> 2 key splits -> 2 x 2367 x 258 floats = 4.89 MB of partials > 4 MiB
    B, N, T, H = 263, 9, 512, 256
    q = torch.zeros(B, N, 1, H, dtype=torch.bfloat16, device=cuda)
    kv = torch.zeros(1, 1, T, H, dtype=torch.bfloat16, device=cuda).expand(B, N, T, H)   # stride-0 view: tiny
    out = torch.zeros_like(q)
    assert pkg.fmha_workspace_bytes(q, kv, kv, None, out, 1.0) == 2 * 2367 * 258 * 4 > pkg.STATIC_SCRATCH_BYTES
    n0 = pkg.launch_count()
    with pytest.raises(pkg.IxkError) as e:
        pkg.fmha_forward_kernel_static_scratch(None, q, kv, kv, None, out, None, 1.0)
    assert e.value.status == pkg.IXK_WORKSPACE_TOO_SMALL
    assert "built-in scratch holds 4194304" in str(e.value)
    assert pkg.launch_count() == n0
    # the ordinary entry point still takes it, with a workspace of the caller's own
    pkg.fmha_forward_kernel(None, q, kv, kv, None, None, 0.0, out, None, 1.0, False)
    assert pkg.launch_count() == n0 + 2
