"""GPU: attention forward from host tensors (ixk_b200.host_io.HostAttention): the pipelined copy /
kernel / copy-back over the batch gives the bits of the plain device-buffer call, call after call."""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal,with_bias,chunk", [(True, False, 1), (False, True, 2), (False, False, 4)])
def test_host_pipeline_matches_the_device_call(pkg, cuda, causal, with_bias, chunk):
    host_io = importlib.import_module("ixk_b200.host_io")
    B, N, S, H = 4, 3, 384, 128
    g = torch.Generator().manual_seed(31)
    pipe = host_io.HostAttention(pkg, B, N, S, S, H, causal=causal, bias=with_bias, chunk=chunk)
    for call in range(3):                       # staging buffers are reused: later calls must not see earlier data
        q, k, v = (torch.randn(B, N, S, H, generator=g).bfloat16().pin_memory() for _ in range(3))
        bias = torch.randn(B, 1, S, S, generator=g).bfloat16().pin_memory() if with_bias else None
        out = torch.full((B, N, S, H), float("nan"), dtype=torch.bfloat16).pin_memory()
        pipe(q, k, v, out, bias)
        torch.cuda.current_stream().synchronize()
        want = torch.empty(B, N, S, H, dtype=torch.bfloat16, device=cuda)
        pkg.fmha_forward_kernel(None, q.to(cuda), k.to(cuda), v.to(cuda), None if bias is None else bias.to(cuda), None, 0.0,
                                want, None, H ** -0.5, False, causal=causal)
        assert torch.equal(out, want.cpu()), f"call {call}"
    assert pkg.device_status() == 0


def test_host_pipeline_rejections(pkg, cuda):
    host_io = importlib.import_module("ixk_b200.host_io")
    with pytest.raises(pkg.IxkError):
        host_io.HostAttention(pkg, 3, 1, 128, 128, 64, chunk=2)              # chunk does not divide the batch
    pipe = host_io.HostAttention(pkg, 2, 1, 128, 128, 64)
    q = torch.zeros(2, 1, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError):
        pipe(q, q, q, torch.zeros(2, 1, 64, 64, dtype=torch.bfloat16))       # out of another shape
    with pytest.raises(pkg.IxkError):
        pipe(q, q, q, q.clone(), bias=torch.zeros(2, 1, 128, 128, dtype=torch.bfloat16))   # built without a bias
    with pytest.raises(pkg.IxkError):
        pipe(q.to(cuda), q, q, q.clone())                                    # a device tensor
