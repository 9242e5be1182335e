"""Benchmark of the kernel-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the chosen custom call over one batch of synthetic, seeded input with
the shapes and distributions of the benchmark configuration.  The default workload is the fused
attention forward, causal, B=8 N=16 S=2048 H=128 bf16.  Rank 0 prints ONE JSON line:

  value      device-timed throughput, inputs resident in HBM (CUDA events on the launch stream,
             one event pair per step, L2 flushed between steps, max over ranks)
  e2e        the same metric through the C ABI with HOST (pinned) buffers: H2D of the step's
             inputs and D2H of its result inside the timed region
  roofline   algorithmic FLOPs (or bytes) per launch / measured launch duration, against the
             measured peak in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle timed on this machine's cores on a bounded sample (reported only)

With --gpus N > 1 (launched by torch.distributed.run) every rank runs the headline workload on its
own batch (the custom calls have no cross-GPU exchange: independent batches/heads), and `value` is
the sum of the work over all ranks divided by the slowest rank's time.  The same line carries,
under `others`, every other benchmark configuration: at N = 1 the single-GPU ones (each with its
own e2e and cpu_baseline), and at every N the two decoder-layer configurations run
tensor-parallel over the N GPUs (strong scaling; the exchange after the row-parallel projections
is libixk's NVLink all-reduce, or NCCL where the exchange buffers cannot be shared), each checked
once against the un-sharded layer on the same inputs.  `--impl reference` times the CPU
restatement of the reference's algorithm (oracle/) on the host cores with the same JSON schema.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np
import torch

import __graft_entry__ as entry

ROOT = os.path.dirname(os.path.abspath(__file__))
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's dominant kernel, from
# one ncu capture of that kernel at this size (absent: no capture of that kernel exists).
NCU_TRAFFIC_BYTES = {
    "fmha_causal": 267.1e6,
    "fmha_bias": 319.8e6,
    "fmha_bwd_causal": 829.4e6,    # the main kernel of the three
    "fmha_bwd_full": 626.8e6,
    "gemm_bias_gelu": 0.985e9,
    "gemm_fp8": 1.137e9,
    "gemm_fp8_e5m2": 1.137e9,      # same kernel and shape; captured with e4m3 x e4m3
    "decode_attn": 4.30e9,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


# ------------------------------------------------------------------------------- workloads
# Every workload: make(dev, gen) -> dict of host (pinned) inputs; to_device; run(pkg, dev_inputs,
# out); work per step; a CPU sample.

class FmhaWorkload:
    """Fused attention forward (configuration 2): Q,K,V ~ N(0,1) bf16 [B,N,S,H], scale 1/sqrt(H);
    causal, or non-causal with an additive bias [B,1,S,S] ~ N(0,1)."""

    def __init__(self, causal: bool, B=8, N=16, S=2048, H=128):
        self.causal, self.B, self.N, self.S, self.H = causal, B, N, S, H
        self.name = f"fmha_fwd_{'causal' if causal else 'bias'}_B{B}_N{N}_S{S}_H{H}_bf16"
        self.metric = "fused-MHA forward TFLOP/s, whole job (bf16, %s)" % ("causal" if causal else "additive bias")
        self.unit = "TFLOP/s"
        self.bound = "tensor"
        self.dtype = "bf16"
        self.kernel = "fmha_prefill_kernel"
        if causal:
            self.work = 4.0 * B * N * H * S * (S + 1) / 2   # masked half not counted
        else:
            self.work = 4.0 * B * N * S * S * H
        self.scale_div = 1e12

    def make(self, seed):
        g = torch.Generator().manual_seed(seed)
        shape = (self.B, self.N, self.S, self.H)
        t = {"q": torch.randn(shape, generator=g).bfloat16(), "k": torch.randn(shape, generator=g).bfloat16(),
             "v": torch.randn(shape, generator=g).bfloat16()}
        if not self.causal:
            t["bias"] = torch.randn(self.B, 1, self.S, self.S, generator=g).bfloat16()
        return t

    def alloc_out(self, dev):
        return torch.empty(self.B, self.N, self.S, self.H, dtype=torch.bfloat16, device=dev)

    def run(self, pkg, d, out):
        pkg.fmha_forward_kernel(None, d["q"], d["k"], d["v"], d.get("bias"), None, 0.0, out, None,
                                self.H ** -0.5, False, causal=self.causal)

    def host_runner(self, pkg, dev):
        """The call a user with host tensors makes: copy-in, kernel and copy-back pipelined over
        the batch on three streams (host_io.HostAttention)."""
        import importlib
        pipe = importlib.import_module(pkg.__name__ + ".host_io").HostAttention(
            pkg, self.B, self.N, self.S, self.S, self.H, causal=self.causal, bias=not self.causal, device=dev,
            chunk=max(1, self.B // 2))   # two pieces: fewest copies that still hide the kernel and the copy-back
        run = lambda host_in, host_out: pipe(host_in["q"], host_in["k"], host_in["v"], host_out, host_in.get("bias"))
        return run, "host_io.HostAttention: H2D / kernel / D2H pipelined over two halves of the batch on three streams"

    def cpu_units(self):
        return self.B * self.N  # independent (batch, head) problems

    def cpu_run(self, orc, host, idx):
        b, n = divmod(idx, self.N)
        f = lambda t: t[b:b + 1, n:n + 1].float().numpy()
        bias = None if self.causal else host["bias"][b:b + 1].float().numpy()
        orc.fmha_forward(f(host["q"]), f(host["k"]), f(host["v"]), bias, head_scale=self.H ** -0.5, causal=self.causal)


class FmhaBwdWorkload:
    """Fused attention backward on configuration 2's shape: dQ, dK, dV from Q, K, V, O, dO and the
    forward's log-sum-exp rows (the forward runs once, outside the timed steps).  Five matrix
    products per tile against the forward's two: 2.5 x the forward's flops."""

    def __init__(self, causal: bool, bias: bool = False, B=8, N=16, S=2048, H=128):
        self.causal, self.bias, self.B, self.N, self.S, self.H = causal, bias, B, N, S, H
        kind = "causal" if causal else ("bias" if bias else "full")
        self.name = f"fmha_bwd_{kind}_B{B}_N{N}_S{S}_H{H}_bf16"
        self.metric = "fused-MHA backward TFLOP/s, whole job (bf16, %s)" % (
            "causal" if causal else ("additive bias" if bias else "non-causal"))
        self.unit = "TFLOP/s"
        self.bound = "tensor"
        self.dtype = "bf16"
        self.kernel = "fmha_bwd_kernel"
        self.work = 10.0 * B * N * H * S * ((S + 1) / 2 if causal else S)
        self.scale_div = 1e12

    def make(self, seed):
        g = torch.Generator().manual_seed(seed)
        shape = (self.B, self.N, self.S, self.H)
        t = {name: torch.randn(shape, generator=g).bfloat16() for name in ("q", "k", "v", "do")}
        if self.bias:
            t["bias"] = torch.randn(self.B, 1, self.S, self.S, generator=g).bfloat16()
        return t

    def alloc_out(self, dev):
        return torch.empty(self.B, self.N, self.S, self.H, dtype=torch.bfloat16, device=dev)   # dQ

    def run(self, pkg, d, out):
        scale = self.H ** -0.5
        if "_o" not in d:
            d["_o"] = torch.empty_like(d["q"])
            d["_lse"] = torch.empty(self.B, self.N, self.S, dtype=torch.float32, device=out.device)
            pkg.fmha_forward_kernel(None, d["q"], d["k"], d["v"], d.get("bias"), None, 0.0, d["_o"], d["_lse"], scale,
                                    True, causal=self.causal)
            d["_dk"], d["_dv"] = torch.empty_like(d["k"]), torch.empty_like(d["v"])
            need = pkg.fmha_backward_workspace_bytes(d["q"], d["k"], d["v"], d["_o"], d.get("bias"), d["do"], out, d["_dk"],
                                                     d["_dv"], scale, self.causal)
            d["_ws"] = torch.empty(need, dtype=torch.uint8, device=out.device)
        pkg.fmha_backward_kernel(None, d["q"], d["k"], d["v"], d["_o"], d.get("bias"), d["do"], d["_lse"], out, d["_dk"],
                                 d["_dv"], scale, causal=self.causal, workspace=d["_ws"])

    def cpu_units(self):
        return self.B * self.N

    def cpu_run(self, orc, host, idx):
        b, n = divmod(idx, self.N)
        f = lambda t: t[b:b + 1, n:n + 1].float().numpy()
        scale = self.H ** -0.5
        bias = host["bias"][b:b + 1].float().numpy() if self.bias else None
        o, lse = orc.fmha_forward(f(host["q"]), f(host["k"]), f(host["v"]), bias, head_scale=scale, causal=self.causal)
        orc.fmha_backward(f(host["q"]), f(host["k"]), f(host["v"]), o, f(host["do"]), lse, bias, head_scale=scale,
                          causal=self.causal)


class GemmWorkload:
    """bf16 GEMM + bias + GELU(tanh) (configuration 1): X[8192x4096] ~ N(0,1), W[4096x16384] ~
    N(0,0.02), bias ~ N(0,0.02), fp32 accumulate, bf16 out."""

    def __init__(self, M=8192, K=4096, N=16384):
        self.M, self.K, self.N = M, K, N
        self.name = f"gemm_bias_gelu_M{M}_K{K}_N{N}_bf16"
        self.metric = "bf16 GEMM+bias+GELU TFLOP/s, whole job"
        self.unit, self.bound, self.dtype, self.kernel = "TFLOP/s", "tensor", "bf16", "gemm_pair_kernel"
        self.work = 2.0 * M * N * K
        self.scale_div = 1e12

    def make(self, seed):
        g = torch.Generator().manual_seed(seed)
        return {"x": torch.randn(self.M, self.K, generator=g).bfloat16(),
                "w": (torch.randn(self.K, self.N, generator=g) * 0.02).bfloat16(),
                "b": (torch.randn(self.N, generator=g) * 0.02).bfloat16()}

    def alloc_out(self, dev):
        return torch.empty(self.M, self.N, dtype=torch.bfloat16, device=dev)

    def run(self, pkg, d, out):
        pkg.gemm(d["x"], d["w"], bias=d["b"], epilogue="BIAS_GELU", out=out)

    library_name = "cuBLAS bf16 matmul through torch.matmul (no bias, no GELU)"

    def library_run(self, d, out):
        torch.matmul(d["x"], d["w"], out=out)

    def cpu_units(self):
        return self.M // 128  # row blocks

    def cpu_run(self, orc, host, idx):
        x = host["x"][idx * 128:(idx + 1) * 128].float().numpy()
        if "w32" not in host:
            host["w32"] = host["w"].float().numpy()
            host["b32"] = host["b"].float().numpy()
        orc.gemm_epilogue(x @ host["w32"], host["b32"], None, 0.0, "BIAS_GELU", orc.BF16)


class Fp8GemmWorkload:
    """fp8 scaled GEMM (configuration 3): A[16384x8192], B[8192x8192] ~ N(0,1) quantised per tensor
    (scale = max_finite/amax), A e4m3, B e4m3 or e5m2; fp32 accumulate; bf16 out."""

    def __init__(self, b_e5m2=False, M=16384, K=8192, N=8192):
        self.M, self.K, self.N, self.b_e5m2 = M, K, N, b_e5m2
        self.name = f"gemm_fp8_e4m3x{'e5m2' if b_e5m2 else 'e4m3'}_M{M}_K{K}_N{N}"
        self.metric = "fp8 scaled GEMM TFLOP/s, whole job"
        self.unit, self.bound, self.dtype, self.kernel = "TFLOP/s", "tensor", "fp8", "gemm_pair_kernel"
        self.work = 2.0 * M * N * K
        self.scale_div = 1e12

    def make(self, seed):
        pkg = entry.load_package()
        g = torch.Generator().manual_seed(seed)
        a, sa = pkg.quantize_fp8(torch.randn(self.M, self.K, generator=g), torch.float8_e4m3fn)
        b, sb = pkg.quantize_fp8(torch.randn(self.K, self.N, generator=g),
                                 torch.float8_e5m2 if self.b_e5m2 else torch.float8_e4m3fn)
        self.inv = (1.0 / sa, 1.0 / sb)
        return {"a": a, "b": b}

    def alloc_out(self, dev):
        return torch.empty(self.M, self.N, dtype=torch.bfloat16, device=dev)

    def run(self, pkg, d, out):
        pkg.gemm_fp8(d["a"], d["b"], self.inv[0], self.inv[1], out=out)

    library_name = "cuBLASLt fp8 matmul through torch._scaled_mm (B repacked column-major beforehand)"

    def library_run(self, d, out):
        if "b_col" not in d:
            d["b_col"] = d["b"].t().contiguous().t()   # cuBLASLt wants the fp8 B operand column-major
            d["sa"] = torch.tensor(self.inv[0], device=out.device)
            d["sb"] = torch.tensor(self.inv[1], device=out.device)
        torch._scaled_mm(d["a"], d["b_col"], scale_a=d["sa"], scale_b=d["sb"], out_dtype=torch.bfloat16, out=out)

    def cpu_units(self):
        return self.M // 128

    def cpu_run(self, orc, host, idx):
        a = host["a"][idx * 128:(idx + 1) * 128].view(torch.uint8).numpy()
        if "b_codes" not in host:
            host["b_codes"] = host["b"].view(torch.uint8).numpy()
        orc.fp8_scaled_gemm(a, orc.F8E4M3, 1.0 / self.inv[0], host["b_codes"],
                            orc.F8E5M2 if self.b_e5m2 else orc.F8E4M3, 1.0 / self.inv[1])


class DecodeWorkload:
    """Decode attention of configuration 5: batch 64, one query per sequence against a KV cache of
    4096 keys, 16 heads x 256, cache stored [B,T,N,H]; HBM-bound, reported in GB/s of K+V+q+o."""

    def __init__(self, B=64, N=16, T=4096, H=256):
        self.B, self.N, self.T, self.H = B, N, T, H
        self.name = f"fmha_decode_B{B}_N{N}_T{T}_H{H}_bf16"
        self.metric = "decode attention GB/s, whole job (bf16 KV cache)"
        self.unit, self.bound, self.dtype, self.kernel = "GB/s", "hbm", "bf16", "fmha_decode_kernel"
        self.work = 2.0 * B * N * T * H * 2 + 2.0 * B * N * H * 2
        self.scale_div = 1e9

    def make(self, seed):
        g = torch.Generator().manual_seed(seed)
        return {"q": torch.randn(self.B, self.N, 1, self.H, generator=g).bfloat16(),
                "k": torch.randn(self.B, self.T, self.N, self.H, generator=g).bfloat16(),
                "v": torch.randn(self.B, self.T, self.N, self.H, generator=g).bfloat16()}

    def alloc_out(self, dev):
        self.ws = None
        return torch.empty(self.B, self.N, 1, self.H, dtype=torch.bfloat16, device=dev)

    def run(self, pkg, d, out):
        k, v = d["k"].permute(0, 2, 1, 3), d["v"].permute(0, 2, 1, 3)
        if self.ws is None:
            need = pkg.fmha_workspace_bytes(d["q"], k, v, None, out, self.H ** -0.5)
            self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device=out.device)
        pkg.fmha_forward_kernel(None, d["q"], k, v, None, None, 0.0, out, None, self.H ** -0.5, False,
                                workspace=self.ws)

    def cpu_units(self):
        return self.B

    def cpu_run(self, orc, host, idx):
        f = lambda t: t[idx:idx + 1].float().numpy()
        k = host["k"][idx:idx + 1].permute(0, 2, 1, 3).float().numpy()
        v = host["v"][idx:idx + 1].permute(0, 2, 1, 3).float().numpy()
        orc.fmha_forward(f(host["q"]), k, v, None, head_scale=self.H ** -0.5)


WORKLOADS = {
    "fmha_causal": lambda: FmhaWorkload(True),
    "fmha_bias": lambda: FmhaWorkload(False),
    "fmha_bwd_causal": lambda: FmhaBwdWorkload(True),
    "fmha_bwd_full": lambda: FmhaBwdWorkload(False),
    "fmha_bwd_bias": lambda: FmhaBwdWorkload(False, bias=True),
    "gemm_bias_gelu": lambda: GemmWorkload(),
    "gemm_fp8": lambda: Fp8GemmWorkload(False),
    "gemm_fp8_e5m2": lambda: Fp8GemmWorkload(True),
    "decode_attn": lambda: DecodeWorkload(),
}
LAYER_WORKLOADS = ("gptj_layer", "gemma_decode")   # tensor-parallel over --gpus N, strong scaling
DEFAULT_WORKLOAD = "fmha_causal"
OTHERS = ["fmha_bias", "fmha_bwd_causal", "gemm_bias_gelu", "gemm_fp8", "gemm_fp8_e5m2", "decode_attn"]


# ------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(device_index).uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------- measurement

def flush_l2(buf):
    buf.add_(1)  # read+write of a buffer twice the size of L2


def time_device(pkg, wl, dev_in, out, steps, warmup, flush_buf):
    """K event-bracketed steps with an L2 flush between them; returns per-step ms list."""
    for _ in range(warmup):
        wl.run(pkg, dev_in, out)
        flush_l2(flush_buf)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        # the flush goes first: every timed step, the first included, starts from a flushed L2, and
        # the host has the flush's run time to enqueue the step behind it (an idle GPU would add
        # the host's launch latency to the first event pair)
        flush_l2(flush_buf)
        starts[i].record()
        wl.run(pkg, dev_in, out)
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def time_library(wl, dev_in, out, steps, warmup, flush_buf):
    """The vendor library's kernel for the same product, timed the same way (context for the
    roofline fraction; not on the product path).  None when the library refuses the operands."""
    try:
        for _ in range(warmup):
            wl.library_run(dev_in, out)
            flush_l2(flush_buf)
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush_l2(flush_buf)
            starts[i].record()
            wl.library_run(dev_in, out)
            ends[i].record()
        torch.cuda.synchronize()
        ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, ends)]))
        return {"name": wl.library_name, "value": wl.work / (ms * 1e-3) / wl.scale_div, "unit": wl.unit, "ms": ms}
    except Exception as e:  # noqa: BLE001 - any refusal of the library is reported, not fatal
        return {"name": wl.library_name, "unavailable": str(e).splitlines()[0][:200]}


def time_e2e(pkg, wl, host_in, dev_in, out, host_out, steps, warmup, dev=None):
    """Steps through the public API with host buffers: H2D inputs, kernel, D2H result, every step.
    Returns (ms per step, which API ran).  The end event is recorded on the current stream after
    the last call, which every call makes wait for its own last copy-back."""
    api = "device-buffer call between torch copies on one stream (H2D, kernel, D2H in sequence)"
    if hasattr(wl, "host_runner"):
        run_host, api = wl.host_runner(pkg, dev)
        one = lambda: run_host(host_in, host_out)
    else:
        def one():
            for k, t in host_in.items():
                dev_in[k].copy_(t, non_blocking=True)
            wl.run(pkg, dev_in, out)
            host_out.copy_(out, non_blocking=True)
    for _ in range(max(1, min(warmup, 3))):
        one()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        one()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps, api


def cpu_baseline(wl, orc, host, budget_s=15.0, threads=None):
    """Times the CPU oracle on a bounded sample: independent units of the workload spread over
    a thread pool (BLAS held to one thread per worker)."""
    from concurrent.futures import ThreadPoolExecutor
    threads = threads or os.cpu_count() or 1
    def body():
        t0 = time.perf_counter()
        wl.cpu_run(orc, host, 0)  # also warms caches / lazily converted operands
        one = max(time.perf_counter() - t0, 1e-4)
        total = wl.cpu_units()
        count = int(max(threads, min(total, budget_s / one * threads)))
        count = min(count, total)
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(lambda i: wl.cpu_run(orc, host, i), range(count)))
        return count, total, time.perf_counter() - t0

    try:
        from threadpoolctl import threadpool_limits
        with threadpool_limits(limits=1):
            n, total_units, dt = body()
    except ImportError:
        n, total_units, dt = body()
    frac = n / total_units
    return {"value": wl.work * frac / dt / wl.scale_div, "unit": wl.unit, "cores": threads, "kind": "port",
            "sample": f"{n} of {total_units} independent units of {wl.name} ({dt:.1f} s)"}, dt


def headline_config(wl):
    """`config` of the JSON line; the same dictionary in both arms."""
    return {"workload": wl.name, "per_gpu": "one full batch per GPU, no cross-GPU exchange",
            "l2": "L2 flushed (512 MB read+write) between timed steps; inputs also exceed L2"}


def probe_xla_cpu():
    """BASELINE.json names "the same HLO on JAX's XLA CPU backend" as the reference semantics.  This
    looks for it on the machine the bench runs on and says what it found."""
    try:
        import jax  # noqa: F401
        return "jax %s is importable here" % getattr(jax, "__version__", "?")
    except Exception as e:  # noqa: BLE001
        return "XLA CPU: unavailable on this box (%s)" % (str(e).splitlines()[0][:120] if str(e) else type(e).__name__)


def xla_cpu_sample(wl, host):
    """If jax is present, time the headline attention on its CPU backend on one (batch, head) unit;
    returns a dict or None.  Any failure is reported, never fatal."""
    try:
        import jax
        import jax.numpy as jnp
    except Exception:  # noqa: BLE001
        return None
    try:
        if not isinstance(wl, FmhaWorkload):
            return {"note": "jax present; XLA-CPU timing is implemented for the attention workloads only"}
        cpu = jax.devices("cpu")[0]
        f = lambda t: jax.device_put(jnp.asarray(t[:1, :1].float().numpy()).transpose(0, 2, 1, 3), cpu)   # [B,S,N,H]
        q, k, v = f(host["q"]), f(host["k"]), f(host["v"])
        bias = None if wl.causal else jax.device_put(jnp.asarray(host["bias"][:1].float().numpy()), cpu)
        fn = jax.jit(lambda q, k, v: jax.nn.dot_product_attention(q, k, v, bias=bias, scale=wl.H ** -0.5,
                                                                  is_causal=wl.causal), device=cpu)
        fn(q, k, v).block_until_ready()
        best = 1e30
        for _ in range(3):
            t0 = time.perf_counter()
            fn(q, k, v).block_until_ready()
            best = min(best, time.perf_counter() - t0)
        unit_work = wl.work / (wl.B * wl.N)
        return {"value": unit_work / best / wl.scale_div, "unit": wl.unit, "kind": "xla-cpu",
                "sample": "1 of %d (batch, head) units, best of 3" % (wl.B * wl.N), "cores": os.cpu_count()}
    except Exception as e:  # noqa: BLE001
        return {"error": str(e).splitlines()[0][:200]}


def measure_fp8_peak(dev, flush_buf):
    """Dense fp8 throughput of the vendor library on this GPU, measured the way the bf16 figure in
    MEASURED_PEAKS.json was (8192^3 product, best of 10): cuBLASLt e4m3 x e4m3 through
    torch._scaled_mm.  None if the library refuses."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t().contiguous().t()
        one = torch.tensor(1.0, device=dev)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e30
        for _ in range(10):
            flush_l2(flush_buf)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # noqa: BLE001
        return None


def run_ours(args, rank, world):
    pkg = entry.load_package()
    pkg.load_library()
    orc = entry.load_oracle()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    flush_buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
    want_others = not args.no_others and args.workload not in LAYER_WORKLOADS
    fp8_peak = measure_fp8_peak(dev, flush_buf) if (world == 1 and want_others) or "fp8" in args.workload else None

    def measure(name, full, cpu_budget):
        wl = WORKLOADS[name]()
        host = {k: t.pin_memory() for k, t in wl.make(seed=1000 * rank + 17).items()}
        dev_in = {k: t.to(dev, non_blocking=True) for k, t in host.items()}
        out = wl.alloc_out(dev)
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()
        n0 = pkg.launch_count()
        with ClockSampler(local) as clk:
            ms = time_device(pkg, wl, dev_in, out, args.steps, args.warmup, flush_buf)
        launches = (pkg.launch_count() - n0) * args.steps // (args.steps + args.warmup)
        total_ms = float(sum(ms))
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([total_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            total_ms = float(t.item())
        torch.cuda.synchronize()
        status = pkg.device_status()
        ms_per_step = total_ms / args.steps
        value = wl.work * world / (ms_per_step * 1e-3) / wl.scale_div
        kernel_ms = float(np.mean(ms))  # one dominant kernel per step
        achieved = wl.work / (kernel_ms * 1e-3) / wl.scale_div
        extra = {}
        if wl.bound == "tensor" and wl.dtype == "fp8":
            assumed = 2.0 * peaks["bf16_tflops"]
            if fp8_peak is not None:
                peak, peak_note = fp8_peak, "cuBLASLt e4m3 8192^3 burst measured in this run (no fp8 figure in MEASURED_PEAKS.json)"
            else:
                peak, peak_note = assumed, f"2 x {peaks['source']} bf16 burst peak (assumed)"
            extra = {"frac_of_2x_bf16_peak": achieved / assumed}
        elif wl.bound == "tensor":
            peak, peak_note = peaks["bf16_tflops"], f"{peaks['source']} bf16 burst peak"
        else:
            peak, peak_note = peaks["hbm_gbs"], f"{peaks['source']} HBM copy bandwidth"
        res = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "ms_per_step": ms_per_step,
            "min_ms": float(min(ms)), "workload": wl.name, "device_status": status,
            "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": wl.unit,
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(name), "kernel": wl.kernel,
                         "peak_source": peak_note, **extra},
            "clocks": clk.summary(), "gpu_launches": int(launches),
        }
        if hasattr(wl, "library_run") and world == 1:
            res["library"] = time_library(wl, dev_in, out, max(3, min(args.steps, 10)), 3, flush_buf)
        if full:
            host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
            host_in = {k: v for k, v in host.items()}
            e2e_ms, e2e_api = time_e2e(pkg, wl, host_in, dev_in, out, host_out, max(3, min(args.steps, 10)), args.warmup, dev)
            if world > 1:
                import torch.distributed as dist
                t = torch.tensor([e2e_ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                e2e_ms = float(t.item())
            h2d = sum(t.numel() * t.element_size() for t in host_in.values())
            d2h = host_out.numel() * host_out.element_size()
            res["e2e"] = {"value": wl.work * world / (e2e_ms * 1e-3) / wl.scale_div, "unit": wl.unit,
                          "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms,
                          "api": e2e_api}
            if rank == 0 and world == 1:
                cb, _ = cpu_baseline(wl, orc, {k: v for k, v in host.items()}, budget_s=cpu_budget)
                res["cpu_baseline"] = cb
        del dev_in, out
        torch.cuda.empty_cache()
        return res, wl, host

    if args.workload in LAYER_WORKLOADS:
        line = run_layer(args, rank, world, pkg, dev, local, peaks, flush_buf, with_cpu=not args.kernel_only)
    else:
        main, wl, host = measure(args.workload, full=not args.kernel_only, cpu_budget=12.0)
        line = {
            "metric": main["metric"], "value": main["value"], "unit": main["unit"], "n_gpus": world,
            "per_gpu_value": main["value"] / world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic (seeded N(0,1) tensors of the configuration's shapes)",
            "config": headline_config(wl),
            "clocks": main["clocks"], "e2e": main.get("e2e"), "gpu_launches": main["gpu_launches"],
            "roofline": main["roofline"], "device_status": main["device_status"],
        }
        if "cpu_baseline" in main:
            line["cpu_baseline"] = main["cpu_baseline"]
            line["cpu_baseline"]["xla_cpu"] = probe_xla_cpu()
            sample = xla_cpu_sample(wl, host)
            if sample is not None:
                line["cpu_baseline"]["xla_cpu_sample"] = sample
        del host
    if want_others:
        others = []
        keys = ("value", "unit", "ms_per_step", "roofline", "gpu_launches", "e2e", "cpu_baseline", "library", "clocks")
        if world == 1:
            for name in OTHERS:
                if name == args.workload:
                    continue
                try:
                    r, w, _ = measure(name, full=not args.kernel_only, cpu_budget=6.0)
                    others.append({"workload": w.name, "metric": w.metric, **{k: r[k] for k in keys if k in r}})
                except Exception as ex:  # a failing side workload must not hide the headline
                    others.append({"workload": name, "error": repr(ex)})
        for lname in LAYER_WORKLOADS:
            try:
                largs = argparse.Namespace(**{**vars(args), "workload": lname})
                r = run_layer(largs, rank, world, pkg, dev, local, peaks, flush_buf, with_cpu=not args.kernel_only)
                others.append({"workload": r["config"]["workload"], "metric": r["metric"], "n_gpus": world,
                               "scaling": r["scaling"], "config": r["config"], "tp_check": r.get("tp_check"),
                               **{k: r[k] for k in keys if k in r}})
            except Exception as ex:  # noqa: BLE001
                if world > 1:
                    raise      # a rank that leaves a collective workload alone would strand the others
                others.append({"workload": lname, "error": repr(ex)})
        if world > 1 and not args.nccl:
            try:
                others.append(run_all_reduce(rank, world, pkg, dev))
            except Exception as ex:  # noqa: BLE001 - e.g. CUDA IPC refused: every rank fails at the same (collective) point
                others.append({"workload": "all_reduce", "error": repr(ex)[:300]})
        line["others"] = others
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the reference's algorithm (oracle/) on the host
    cores.  The reference's own kernels are SYCL/ESIMD for Intel GPUs on XeTLA and oneDNN and cannot
    be built or run here, so `kind` is "port".  Rank 0 alone runs."""
    if rank != 0:
        return
    if args.workload in LAYER_WORKLOADS:
        print(json.dumps(layer_reference(args, full_line=True)))
        return
    orc = entry.load_oracle()
    wl = WORKLOADS[args.workload]()
    host = wl.make(seed=17)
    threads = os.cpu_count() or 1
    # size the per-step sample so that steps+warmup passes stay within ~2 minutes
    budget = max(1.0, 100.0 / (args.steps + args.warmup))
    times, sample = [], None
    for i in range(args.warmup + args.steps):
        cb, dt = cpu_baseline(wl, orc, host, budget_s=budget, threads=threads)
        sample = cb["sample"]
        if i >= args.warmup:
            times.append((cb["value"], dt))
    value = float(np.mean([v for v, _ in times]))
    ms = float(np.mean([d for _, d in times])) * 1e3
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic (seeded N(0,1) tensors of the configuration's shapes)",
        "config": headline_config(wl),
        "note": "each step is a bounded sample of the workload; arithmetic in fp32 on bf16-rounded inputs",
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample,
                         "xla_cpu": probe_xla_cpu()},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------- layer configs

def _layer_weights(name, seed=7):
    """Random-init weights ~ N(0, 0.02) in bf16, identical on every rank (same seed)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: (torch.randn(*shape, generator=g) * 0.02).bfloat16()
    if name == "gptj_layer":   # hidden 4096, 16 heads x 256, MLP 16384
        return {"wqkv": r(4096, 12288), "wo": r(4096, 4096), "w1": r(4096, 16384), "b1": r(16384),
                "w2": r(16384, 4096), "b2": r(4096)}
    return {"wqkv": r(3072, 12288), "wo": r(4096, 3072), "wgate": r(3072, 24576), "wup": r(3072, 24576),
            "wdown": r(24576, 3072),   # Gemma-7B shape: hidden 3072, 16 heads x 256, GeGLU 24576
            "norm_attn": r(3072), "norm_mlp": r(3072)}   # the RMSNorm scales w, applied as (1 + w)


LAYER_METRIC = {
    "gptj_layer": "GPT-J-6B-shaped decoder layer prefill TFLOP/s (bf16, tensor-parallel, whole job)",
    "gemma_decode": "Gemma-7B-shaped decode step GB/s of algorithmic bytes (bf16, tensor-parallel, whole job)",
}


def layer_config(name, world):
    if name == "gptj_layer":
        wname = f"gptj_layer_prefill_B4_S2048_hidden4096_heads16x256_mlp16384_tp{world}"
    else:
        wname = f"gemma_decode_B64_T4096_hidden3072_heads16x256_mlp24576_tp{world}"
    return {"workload": wname, "parallelism": f"tp{world} by heads / MLP columns, all-reduce after row-parallel GEMMs",
            "l2": "L2 flushed (512 MB read+write) between timed steps"}


def run_all_reduce(rank, world, pkg, dev, calls=40):
    """The exchange of the tensor-parallel layers on its own: libixk's NVLink all-reduce at the two
    message sizes of configurations 5 and 4 (393 KB: one-shot to a private buffer; 67 MB: two-shot in
    place), `calls` back to back between one pair of CUDA events, max over ranks, with
    ncclAllReduce timed the same way beside it.  Bus bandwidth = 2 (N - 1) / N x bytes / time."""
    import importlib
    import torch.distributed as dist
    comm_mod = importlib.import_module(entry.PKG_NAME + ".comm")
    sizes = (("393 KB (decode partial), one-shot", 64 * 3072), ("67 MB (prefill partial), two-shot in place", 8192 * 4096))
    comm = comm_mod.Communicator(pkg, rank, world, sizes[-1][1] * 2)
    rows = []
    try:
        for label, n in sizes:
            slot = comm.view(0, (n,), torch.bfloat16)
            slot.normal_()
            private = torch.empty(n, dtype=torch.bfloat16, device=dev)
            mine = (lambda: comm.all_reduce(slot, out=private)) if n * 2 < (1 << 20) else (lambda: comm.all_reduce(slot))
            ref_t = torch.randn(n, device=dev).bfloat16()
            theirs = lambda: dist.all_reduce(ref_t)
            out = {}
            for name, fn in (("libixk", mine), ("nccl", theirs)):
                for _ in range(5):
                    fn()
                torch.cuda.synchronize()
                dist.barrier()
                s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s_ev.record()
                for _ in range(calls):
                    fn()
                e_ev.record()
                torch.cuda.synchronize()
                t = torch.tensor([s_ev.elapsed_time(e_ev) / calls], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                us = float(t.item()) * 1e3
                out[name] = {"us_per_call": us, "bus_gbs": 2.0 * (world - 1) / world * n * 2 / (us * 1e-6) / 1e9}
            rows.append({"message": label, "bytes": n * 2, **out})
        status = pkg.device_status()
    finally:
        comm.close()
    return {"workload": f"all_reduce_bf16_{world}_ranks", "metric": "all-reduce time per call, back to back (us) and bus bandwidth (GB/s)",
            "n_gpus": world, "sizes": rows, "device_status": status,
            "note": "NVLink peer loads / stores with device-side flags (libixk) against ncclAllReduce, same buffers sizes and timing"}


def run_layer(args, rank, world, pkg, dev, local, peaks, flush_buf, with_cpu=True):
    """Configurations 4 and 5: one decoder layer, tensor-parallel over `world` GPUs by heads / MLP
    columns, one exchange after the row-parallel projections.  Total work is fixed (strong scaling).
      gptj_layer    prefill, batch 4 x seq 2048, reported in TFLOP/s of the layer's GEMM+attention FLOPs
      gemma_decode  one token for 64 sequences against a 4096-entry KV cache, reported in GB/s of the
                    algorithmic bytes (K, V and every weight once)
    Returns the JSON line as a dictionary (every rank; rank 0's is the one printed)."""
    import importlib
    import torch.distributed as dist
    layers = importlib.import_module(entry.PKG_NAME + ".layers")
    comm_mod = importlib.import_module(entry.PKG_NAME + ".comm")
    ops = layers.KernelOps(pkg, gemm_workspace=torch.empty(32 << 20, dtype=torch.uint8, device=dev))
    full = _layer_weights(args.workload)
    g = torch.Generator().manual_seed(11)
    ident = lambda t, group=None: t
    tol_abs, tol_rel = 6e-2, 2e-2      # the layer tests' bound: bf16 activations of O(1) through a block

    def to_dev(w):
        for k, v in vars(w).items():
            if torch.is_tensor(v):
                setattr(w, k, v.to(dev))
        return w

    # ---- exchange: libixk's NVLink all-reduce where the buffers can be shared, else NCCL
    comm, comm_note = None, None
    if world > 1 and not args.nccl:
        nbytes = 2 * 4 * 2048 * 4096 * 2 if args.workload == "gptj_layer" else 1 << 20   # GPT-J: the slots + the result
        nbytes += 4096                                  # + the slot of the per-step alignment exchange (see the timed loop)
        try:
            comm = comm_mod.Communicator(pkg, rank, world, nbytes)
        except Exception as ex:  # noqa: BLE001 - e.g. CUDA IPC not permitted between the ranks' containers
            comm_note = "libixk exchange buffers could not be shared (%s): NCCL all-reduce" % str(ex).splitlines()[0][:160]
        ok = torch.tensor([1 if comm is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0 and comm is not None:
            comm.close()
            comm, comm_note = None, "a peer could not share its exchange buffer: NCCL all-reduce"

    tp_check = None
    if args.workload == "gptj_layer":
        B, S = 4, 2048
        w = to_dev(layers.GptJLayerWeights.shard(full, 16, 256, 64, rank, world))
        x_host = torch.randn(B, S, 4096, generator=g).bfloat16().pin_memory()
        x = x_host.to(dev)
        rope = layers.rotary_tables(torch.arange(S, device=dev), 64)
        step = lambda reduce=None: layers.gptj_layer_prefill(x, w, ops, rope=rope, reduce=reduce, comm=comm,
                                                             fused_exchange=not args.unfused_exchange)
        work, div, unit, bound = layers.gptj_layer_flops(B, S), 1e12, "TFLOP/s", "tensor"
        peak = peaks["bf16_tflops"] * world
        if world > 1:   # once, outside the timed region: the sharded step against the un-sharded layer, same inputs
            w_full = to_dev(layers.GptJLayerWeights.shard(full, 16, 256, 64, 0, 1))
            y_ref = layers.gptj_layer_prefill(x, w_full, ops, rope=rope, reduce=ident).float()
            del w_full
    else:
        B, T = 64, 4096
        w = to_dev(layers.GemmaLayerWeights.shard(full, 16, 256, rank, world))
        hl = 16 // world
        x_host = torch.randn(B, 1, 3072, generator=g).bfloat16().pin_memory()
        x = x_host.to(dev)
        # the full cache from one seed on every rank (same device generator, same values); a rank keeps its heads
        gk = torch.Generator(device=dev).manual_seed(13)
        k_full = torch.randn(B, T, 16, 256, generator=gk, device=dev, dtype=torch.bfloat16)
        v_full = torch.randn(B, T, 16, 256, generator=gk, device=dev, dtype=torch.bfloat16)
        h0 = rank * hl
        k_cache = k_full[:, :, h0:h0 + hl].contiguous() if world > 1 else k_full
        v_cache = v_full[:, :, h0:h0 + hl].contiguous() if world > 1 else v_full
        ws = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
        rope = layers.rotary_tables(torch.tensor([T - 1], device=dev), 256)
        if comm is not None:
            comm.set_alternating(True)   # the step's two exchanges (and the alignment one) use three different ranges in turn
        step = lambda reduce=None: layers.gemma_decode_step(x, w, k_cache, v_cache, T - 1, ops, workspace=ws, rope=rope,
                                                            reduce=reduce, comm=comm)
        work, div, unit, bound = layers.gemma_decode_bytes(B, T), 1e9, "GB/s", "hbm"
        peak = peaks["hbm_gbs"] * world
        if world > 1:
            w_full = to_dev(layers.GemmaLayerWeights.shard(full, 16, 256, 0, 1))
            y_ref = layers.gemma_decode_step(x, w_full, k_full, v_full, T - 1, ops, workspace=ws, rope=rope,
                                             reduce=ident).float()
            del w_full
        del k_full, v_full
    del full
    torch.cuda.empty_cache()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def warm_up_and_check():
        """Warm-up steps, then (N > 1) the sharded result against the un-sharded layer and the device
        status word; the outcome is the same on every rank."""
        for _ in range(args.warmup):
            out = step()
            flush_l2(flush_buf)
        barrier()
        check, why = None, ""
        try:
            pkg.device_status()          # a bounded wait that gave up shows here (and is cleared)
        except pkg.IxkError as ex:
            why = str(ex).splitlines()[0][:160]
        if world > 1:
            err = (out.float() - y_ref).abs()
            bad = int((err > tol_abs + tol_rel * y_ref.abs()).sum().item())
            check = {"against": "the un-sharded layer on this GPU, same weights and inputs", "max_abs_err": float(err.max().item()),
                     "tolerance": f"{tol_abs} + {tol_rel} * |ref|", "elements_outside": bad, "ok": bad == 0}
            flag = torch.tensor([1 if (bad or why) else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            failed = int(flag.item()) != 0
            if failed and not why:
                why = f"{bad} elements outside the tolerance on this rank" if bad else "a peer reported a failure"
        else:
            failed = bool(why)
        return out, check, failed, why

    y, tp_check, failed, why = warm_up_and_check()
    if failed and comm is not None:
        # libixk's exchange did not pass on this machine: say so and measure with NCCL's instead
        comm_note = f"libixk exchange failed its check ({why}): NCCL all-reduce"
        try:
            comm.close()
        except Exception:  # noqa: BLE001 - a communicator whose wait ran out may refuse; it is abandoned either way
            pass
        comm = None
        y, tp_check, failed, why = warm_up_and_check()
    if failed:
        raise RuntimeError(f"tensor-parallel {args.workload} disagrees with the un-sharded layer: {tp_check} {why}")
    if world > 1:
        del y_ref
    y_eager = y.clone()      # the checked result, to be met again by the last timed (replayed) step
    # A layer step is a fixed sequence of ~10-15 library kernels: it is captured once into a CUDA
    # graph and replayed, which removes the launch gaps (the decode step is launch-bound otherwise).
    # With libixk's all-reduce the exchange is an ordinary kernel inside that graph.  With NCCL the
    # pieces of the step between the all-reduces are captured as separate graphs and the
    # all-reduces stay eager calls between the replays (NCCL is never captured here).
    launches_per_step = None
    launch_mode = "eager"
    whole_graph = not args.no_graph and (world == 1 or comm is not None)
    segmented = not args.no_graph and world > 1 and comm is None
    if whole_graph:
        n_before = pkg.launch_count()
        cap_stream = torch.cuda.Stream()
        cap_stream.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap_stream):
            with torch.cuda.graph(graph, stream=cap_stream, capture_error_mode="thread_local"):
                y = step()
        torch.cuda.current_stream().wait_stream(cap_stream)
        launches_per_step = pkg.launch_count() - n_before
        y_graph = y
        step = lambda: (graph.replay(), y_graph)[1]
        launch_mode = "CUDA graph replay of the whole step" + (" (libixk NVLink all-reduce inside)" if comm is not None else "")
    elif segmented:
        n_before = pkg.launch_count()
        cap_stream = torch.cuda.Stream()
        cap_stream.wait_stream(torch.cuda.current_stream())
        pool = torch.cuda.graph_pool_handle()
        plan = []
        eager = step
        with torch.cuda.stream(cap_stream):
            cur = torch.cuda.CUDAGraph()
            cur.capture_begin(pool=pool, capture_error_mode="thread_local")

            def cut(t, group=None):
                nonlocal cur
                cur.capture_end()
                plan.append(cur)
                plan.append(t)
                dist.all_reduce(t)
                cur = torch.cuda.CUDAGraph()
                cur.capture_begin(pool=pool, capture_error_mode="thread_local")
                return t

            y_seg = eager(cut)
            cur.capture_end()
            plan.append(cur)
        torch.cuda.current_stream().wait_stream(cap_stream)
        launches_per_step = pkg.launch_count() - n_before

        def step():
            for item in plan:
                if isinstance(item, torch.cuda.CUDAGraph):
                    item.replay()
                else:
                    dist.all_reduce(item)
            return y_seg
        launch_mode = "CUDA graphs of the pieces between eager NCCL all-reduces"
    if whole_graph or segmented:
        y_before = y.clone() if not whole_graph else None
        for _ in range(2):
            y = step()
        barrier()
    n0 = pkg.launch_count()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    # N > 1: the L2 flush between steps takes a slightly different time on every GPU, and a rank that
    # is through earlier would otherwise spend the difference waiting inside its step's first
    # exchange, i.e. inside its timed region.  A tiny exchange after the flush lines the ranks up
    # before the start event; it is not part of the step and not timed.
    if world > 1:
        if comm is not None:
            align_slot = comm.view(comm.buffer_bytes - 4096, (1024,), torch.float32)
            align_slot.zero_()
            align_out = torch.empty(1024, dtype=torch.float32, device=dev)
            align = lambda: comm.all_reduce(align_slot, out=align_out)
        else:
            align_t = torch.zeros(1024, device=dev)
            align = lambda: dist.all_reduce(align_t)
        barrier()
    else:
        align = lambda: None
    with ClockSampler(local) as clk:
        for i in range(args.steps):
            flush_l2(flush_buf)      # first, so that the host enqueues the step while the flush runs
            align()
            starts[i].record()
            y = step()
            ends[i].record()
        torch.cuda.synchronize()
    launches = pkg.launch_count() - n0 - (args.steps if (world > 1 and comm is not None) else 0)   # without the alignment launches
    if launches_per_step is not None:
        launches = launches_per_step * args.steps   # replayed from the graph
    total_ms = float(sum(s.elapsed_time(e) for s, e in zip(starts, ends)))
    # the steps are deterministic (fixed inputs, sums in rank order): the last timed step, launched the
    # way the timed steps are, must reproduce the checked warm-up result bit for bit
    same = torch.tensor([1 if torch.equal(y, y_eager) else 0], device=dev)
    if world > 1:
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
    timed_equals_checked = bool(int(same.item()))
    del y_eager
    # end to end: host x in, host y out
    y_host = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s_ev.record()
    for _ in range(e2e_steps):
        x.copy_(x_host, non_blocking=True)
        y = step()
        y_host.copy_(y, non_blocking=True)
    e_ev.record()
    torch.cuda.synchronize()
    e2e_ms = s_ev.elapsed_time(e_ev) / e2e_steps
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0].item()), float(t[1].item())
    status = pkg.device_status()
    ms_per_step = total_ms / args.steps
    value = work / (ms_per_step * 1e-3) / div
    config = layer_config(args.workload, world)
    config["launch"] = launch_mode
    config["exchange"] = ("none (one GPU)" if world == 1 else
                          "libixk NVLink all-reduce (peer loads/stores, device-side flags)" if comm is not None else
                          (comm_note or "NCCL all-reduce"))
    if comm is not None and args.workload == "gptj_layer" and not args.unfused_exchange:
        config["exchange"] += "; the down projection stores its row blocks into the owners' buffers as it computes"
    line = {
        "metric": LAYER_METRIC[args.workload], "value": value, "unit": unit, "n_gpus": world, "per_gpu_value": value / world,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random-init weights ~N(0,0.02), activations ~N(0,1), seeded)",
        "config": config, "clocks": clk.summary(),
        "e2e": {"value": work / (e2e_ms * 1e-3) / div, "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(x_host.numel() * 2), "d2h_bytes_per_step": int(y_host.numel() * 2)},
        "gpu_launches": int(launches),
        "roofline": {"bound": bound, "achieved": value, "peak": peak, "unit": unit, "frac": value / peak, "traffic": None,
                     "kernel": "whole layer step (libixk GEMM, attention, glue and exchange kernels)",
                     "peak_source": f"{world} x {peaks['source']} single-GPU peak"},
        "device_status": status,
    }
    line["config"]["timed_step_equals_checked_step"] = timed_equals_checked
    if tp_check is not None:
        line["tp_check"] = tp_check
    if with_cpu and rank == 0 and world == 1:
        ref = layer_reference(args, full_line=False)
        line["cpu_baseline"] = ref
    if comm is not None:
        comm.close()
    return line


def layer_reference(args, full_line):
    """CPU arm of the layer configurations: the un-sharded numpy layer oracle on the host cores, on
    a bounded sample of the batch.  Returns the cpu_baseline object, or the whole reference-arm line."""
    import importlib
    from oracle import layers_oracle
    layers = importlib.import_module(entry.PKG_NAME + ".layers")
    full = {k: v.float().numpy() for k, v in _layer_weights(args.workload).items()}
    g = torch.Generator().manual_seed(11)
    times = []
    if args.workload == "gptj_layer":
        B, S = 4, 2048
        x = torch.randn(B, S, 4096, generator=g).bfloat16().float().numpy()[:1]
        work, div, unit, frac = layers.gptj_layer_flops(1, S), 1e12, "TFLOP/s", "1 of 4 sequences"
        fn = lambda: layers_oracle.gptj_layer_prefill(x, full, 16, 256, 64)
    else:
        B, T = 64, 4096
        nb = 8
        x = torch.randn(B, 1, 3072, generator=g).bfloat16().float().numpy()[:nb]
        kc = np.random.default_rng(0).standard_normal((nb, T, 16, 256), dtype=np.float32)
        vc = np.random.default_rng(1).standard_normal((nb, T, 16, 256), dtype=np.float32)
        work, div, unit, frac = layers.gemma_decode_bytes(nb, T), 1e9, "GB/s", f"{nb} of 64 sequences (weights read once per sample)"
        fn = lambda: layers_oracle.gemma_decode_step(x, full, kc, vc, T - 1, 16, 256)
    passes = (args.warmup + args.steps) if full_line else 2
    warm = args.warmup if full_line else 1
    for i in range(passes):
        t0 = time.perf_counter()
        fn()
        if i >= warm:
            times.append(time.perf_counter() - t0)
        if sum(times) > 120:
            break
    dt = float(np.mean(times))
    value = work / dt / div
    cores = os.cpu_count() or 1
    cb = {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": frac + " (%.1f s per pass)" % dt}
    if not full_line:
        return cb
    world = int(os.environ.get("WORLD_SIZE", 1))
    return {
        "impl": "reference", "metric": LAYER_METRIC[args.workload], "value": value, "unit": unit, "n_gpus": world,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random-init weights ~N(0,0.02), activations ~N(0,1), seeded)",
        "config": layer_config(args.workload, world), "note": "each step is a bounded sample of the workload: " + frac,
        "cpu_baseline": {**cb, "xla_cpu": probe_xla_cpu()},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + list(LAYER_WORKLOADS))
    ap.add_argument("--no-others", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-graph", action="store_true", help="layer workloads: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--nccl", action="store_true",
                    help="layer workloads at N > 1: exchange through NCCL instead of libixk's NVLink all-reduce")
    ap.add_argument("--unfused-exchange", action="store_true",
                    help="GPT-J layer at N > 1 with libixk's exchange: down projection, all-reduce and residual add as "
                         "three launches instead of the projection that scatters its result + one exchange kernel")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-timed steps only (no e2e, no CPU baseline): the command profiled under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        if world != args.gpus and world == 1 and args.gpus > 1:
            print(json.dumps({"error": "launch with torch.distributed.run for --gpus > 1"}))
            sys.exit(2)
        run_ours(args, rank, world)


if __name__ == "__main__":
    main()
