"""Attention forward for callers whose tensors live in HOST memory.

The custom call itself takes device buffers (the reference's runner is handed device pointers by
XLA, xla/service/gpu/xetla_gpu_fused_mha_runner.cc); a host of the library that starts from host
arrays pays a PCIe transfer that is 30 x longer than the kernel.  Done as "copy everything, run,
copy back" the three legs add up.  `HostAttention` cuts the call along the batch dimension and
runs the legs as a pipeline on three streams: while batch b's inputs are on their way to the
device, batch b-1 is in the kernel and batch b-2's result is on its way back, so the call costs
about as much as its largest leg (the input copy), and consecutive calls overlap too (call i+1's
input copies run under call i's last result copies).

Host tensors should be pinned (`torch.Tensor.pin_memory()`): pageable memory makes the copies
synchronous and the pipeline degenerates to the sequential form.  Results are bit-identical to
the device-buffer call: the same kernel runs on the same values, one batch element at a time.
"""
from __future__ import annotations

from typing import Optional

import torch


class HostAttention:
    """Staging buffers, streams and events for one attention shape.  Not thread-safe; one object
    per caller thread and device."""

    def __init__(self, pkg, B: int, N: int, F: int, T: int, H: int, dtype=torch.bfloat16, *, causal: bool = False,
                 bias: bool = False, device=None, chunk: int = 1):
        if B % chunk != 0:
            raise pkg.IxkError(pkg.IXK_INVALID_ARGUMENT, "chunk must divide the batch size")
        self.pkg, self.causal, self.chunk = pkg, causal, chunk
        self.shape = (B, N, F, T, H)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        dev = self.device
        self.q = torch.empty(B, N, F, H, dtype=dtype, device=dev)
        self.k = torch.empty(B, N, T, H, dtype=dtype, device=dev)
        self.v = torch.empty(B, N, T, H, dtype=dtype, device=dev)
        self.bias = torch.empty(B, 1, F, T, dtype=dtype, device=dev) if bias else None
        self.out = torch.empty(B, N, F, H, dtype=dtype, device=dev)
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(device=dev) for _ in range(3))
        n = B // chunk
        # per chunk: inputs arrived / kernel done / result back on the host (the last two also guard
        # the staging buffers against the NEXT call: inputs are overwritten only after the kernel
        # that read them, the result only after the copy that read it)
        self.arrived = [torch.cuda.Event() for _ in range(n)]
        self.computed = [torch.cuda.Event() for _ in range(n)]
        self.returned = [torch.cuda.Event() for _ in range(n)]
        self.used = False

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
        """q [B,N,F,H], k/v [B,N,T,H], bias [B,1,F,T] or None, out [B,N,F,H]: host tensors.  Returns
        `out`; it is complete once the work queued on the current stream up to here has completed
        (`torch.cuda.current_stream().synchronize()`, or an event recorded after the call)."""
        pkg = self.pkg
        B, N, F, T, H = self.shape
        if q.shape != (B, N, F, H) or k.shape != (B, N, T, H) or v.shape != k.shape or out.shape != q.shape:
            raise pkg.IxkError(pkg.IXK_INVALID_ARGUMENT, "shapes differ from the ones this pipeline was built for")
        if (bias is None) != (self.bias is None):
            raise pkg.IxkError(pkg.IXK_INVALID_ARGUMENT, "bias must be given exactly when the pipeline was built with one")
        for t in (q, k, v, out, bias):
            if t is not None and (t.is_cuda or t.dtype != self.q.dtype):
                raise pkg.IxkError(pkg.IXK_INVALID_ARGUMENT, "host tensors of the pipeline's type are expected")
        scale = H ** -0.5 if scale is None else scale
        c = self.chunk
        for i in range(B // c):
            s = slice(i * c, (i + 1) * c)
            with torch.cuda.stream(self.h2d):
                if self.used:
                    self.h2d.wait_event(self.computed[i])      # the previous call's kernel has read this chunk
                self.q[s].copy_(q[s], non_blocking=True)
                self.k[s].copy_(k[s], non_blocking=True)
                self.v[s].copy_(v[s], non_blocking=True)
                if bias is not None:
                    self.bias[s].copy_(bias[s], non_blocking=True)
                self.arrived[i].record(self.h2d)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(self.arrived[i])
                if self.used:
                    self.compute.wait_event(self.returned[i])  # the previous call's result has left this chunk
                pkg.fmha_forward_kernel(None, self.q[s], self.k[s], self.v[s], None if bias is None else self.bias[s],
                                        None, 0.0, self.out[s], None, scale, False, causal=self.causal)
                self.computed[i].record(self.compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(self.computed[i])
                out[s].copy_(self.out[s], non_blocking=True)
                self.returned[i].record(self.d2h)
        self.used = True
        torch.cuda.current_stream(self.device).wait_event(self.returned[-1])   # copies of one stream finish in order
        return out
