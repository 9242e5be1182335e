"""Host side of libixk's NVLink all-reduce (ixk_comm_* / ixk_all_reduce* in include/ixk.h), the
exchange step the reference runs through sycl_allreduce (xla/service/gpu/ccl_ops.cc:604-789).

One `Communicator` per rank (one process per GPU).  torch.distributed is used once, at set-up, to
pass the IPC handles of the exchange buffers around and to make the ranks meet; after that an
all-reduce is one kernel launch on the caller's stream with no host synchronisation, so a layer
step that contains it can be captured into a CUDA graph.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

REDUCE_KINDS = ("SUM", "PRODUCT", "MIN", "MAX")   # ReductionKind, ccl_ops.cc:656-779


class _RawCudaMemory:
    """Lets torch alias device memory owned by the library (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Communicator:
    def __init__(self, pkg, rank: int, world: int, buffer_bytes: int, group=None, device=None):
        """Creates this rank's exchange buffer on the current device and connects it to the peers'
        (handles travel through torch.distributed's `group`).  Collective: every rank of the
        group must call it."""
        import torch.distributed as dist
        self.pkg, self.rank, self.world, self.group = pkg, rank, world, group
        self.lib = pkg.load_library()
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        handle = (ctypes.c_ubyte * 64)()
        comm = ctypes.c_void_p()
        pkg._check(self.lib.ixk_comm_create(rank, world, buffer_bytes, ctypes.byref(comm), handle))
        self._comm = comm
        self.buffer_bytes = buffer_bytes
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle), group=group)
            blob = b"".join(handles)
            pkg._check(self.lib.ixk_comm_connect_ipc(self._comm, blob))
            dist.barrier(group=group)      # every rank has mapped every buffer before anyone uses one
        ptr = self.lib.ixk_comm_buffer(self._comm)
        self._raw = _RawCudaMemory(ptr, buffer_bytes)
        self.bytes_view = torch.as_tensor(self._raw, device=self.device)   # uint8 [buffer_bytes], aliases the buffer
        self.base_ptr = ptr

    def view(self, offset_bytes: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor over [offset, offset + size) of this rank's exchange buffer: hand it to the
        producing kernel as its output, then call all_reduce with the same offset."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset_bytes % 16 or offset_bytes + nbytes > self.buffer_bytes:
            raise self.pkg.IxkError(self.pkg.IXK_INVALID_ARGUMENT, "view outside the exchange buffer or misaligned")
        return self.bytes_view[offset_bytes:offset_bytes + nbytes].view(dtype).view(*shape)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base_ptr
        if off < 0 or off + t.numel() * t.element_size() > self.buffer_bytes or not t.is_contiguous():
            raise self.pkg.IxkError(self.pkg.IXK_INVALID_ARGUMENT, "tensor is not a dense view of the exchange buffer")
        return off

    def all_reduce(self, contribution: torch.Tensor, out: Optional[torch.Tensor] = None, kind: str = "SUM",
                   stream=None) -> torch.Tensor:
        """Sum (or product / min / max) over ranks of `contribution`, a view of the exchange buffer at
        the same offset on every rank.  `out` defaults to the contribution itself (in place)."""
        out = contribution if out is None else out
        st = self.lib.ixk_all_reduce(self._comm, self.pkg._TORCH_TO_IXK[contribution.dtype], REDUCE_KINDS.index(kind),
                                     self.offset_of(contribution), out.data_ptr(), contribution.numel(),
                                     self.pkg._stream_ptr(stream))
        self.pkg._check(st)
        return out

    def all_reduce_residual(self, contribution: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """x + round(sum over ranks of contribution [+ bias]) in one launch."""
        out = torch.empty_like(x) if out is None else out
        cols = x.shape[-1]
        if contribution.numel() != x.numel() or not x.is_contiguous() or not out.is_contiguous():
            raise self.pkg.IxkError(self.pkg.IXK_INVALID_ARGUMENT, "x, out and the contribution must be dense and of one size")
        st = self.lib.ixk_all_reduce_residual(self._comm, self.pkg._TORCH_TO_IXK[x.dtype], self.offset_of(contribution),
                                              x.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                                              x.numel() // cols, cols, self.pkg._stream_ptr(stream))
        self.pkg._check(st)
        return out

    def reduce_scatter(self, contribution: torch.Tensor, out: torch.Tensor, kind: str = "SUM", stream=None) -> torch.Tensor:
        """`contribution`: a view of the exchange buffer holding world * out.numel() elements (the same
        offset on every rank); `out` (any dense local tensor) receives the combination of slice `rank`."""
        st = self.lib.ixk_reduce_scatter(self._comm, self.pkg._TORCH_TO_IXK[contribution.dtype], REDUCE_KINDS.index(kind),
                                         self.offset_of(contribution), out.data_ptr(), out.numel(),
                                         self.pkg._stream_ptr(stream))
        self.pkg._check(st)
        return out

    def all_gather(self, piece: torch.Tensor, gathered: torch.Tensor, stream=None) -> torch.Tensor:
        """`piece` (any dense local tensor) lands at slot `rank` of `gathered`, a view of the exchange
        buffer with world * piece.numel() elements, on every rank."""
        st = self.lib.ixk_all_gather(self._comm, self.pkg._TORCH_TO_IXK[piece.dtype], piece.data_ptr(),
                                     self.offset_of(gathered), piece.numel(), self.pkg._stream_ptr(stream))
        self.pkg._check(st)
        return gathered

    def gemm_scatter(self, lhs: torch.Tensor, rhs: torch.Tensor, slots_offset: int, *, c: Optional[torch.Tensor] = None,
                     beta: float = 0.0, bias: Optional[torch.Tensor] = None, epilogue: str = "DEFAULT", stream=None) -> None:
        """This rank's partial lhs @ rhs (+ beta * c) of a row-parallel projection, row block o stored
        straight into rank o's exchange buffer (slot `rank` of the slots at slots_offset) while the
        following tiles are computed.  all_reduce_scattered finishes the exchange."""
        m, n = lhs.shape[-2], rhs.shape[-1]
        shape_only = torch.empty((m, n), device="meta", dtype=lhs.dtype)   # carries the result's layout; no memory
        attrs = self.pkg.gemm_attrs_for(lhs, rhs, shape_only, beta)
        d = self.pkg.gemm_desc_from_attrs(attrs, epilogue)
        ptr = lambda t: None if t is None else t.data_ptr()
        st = self.lib.ixk_gemm_scatter(self._comm, ctypes.byref(d), ptr(lhs), ptr(rhs), ptr(c), ptr(bias), slots_offset,
                                       self.pkg._stream_ptr(stream))
        self.pkg._check(st)

    def all_reduce_scattered(self, slots_offset: int, out: torch.Tensor, x: Optional[torch.Tensor] = None,
                             bias: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """Adds up the slots gemm_scatter filled (the rows this rank owns), applies
        x + round(round(sum) + bias) and writes the rows into `out` — a [rows, cols] view of the
        exchange buffer at the same offset on every rank — of every rank."""
        rows, cols = out.numel() // out.shape[-1], out.shape[-1]
        if x is not None and (x.numel() != out.numel() or not x.is_contiguous()):
            raise self.pkg.IxkError(self.pkg.IXK_INVALID_ARGUMENT, "x must be dense and of the result's size")
        st = self.lib.ixk_all_reduce_scattered(self._comm, self.pkg._TORCH_TO_IXK[out.dtype], slots_offset,
                                               None if x is None else x.data_ptr(),
                                               None if bias is None else bias.data_ptr(), self.offset_of(out),
                                               rows, cols, self.pkg._stream_ptr(stream))
        self.pkg._check(st)
        return out

    def set_alternating(self, on: bool = True) -> None:
        """Promise that consecutive calls never use overlapping contribution ranges: the one-shot form
        then skips its second meeting with the peers (see ixk_comm_set_alternating)."""
        self.pkg._check(self.lib.ixk_comm_set_alternating(self._comm, 1 if on else 0))

    def set_wait_limit(self, cycles: int) -> None:
        self.pkg._check(self.lib.ixk_comm_set_wait_limit(self._comm, cycles))

    def close(self) -> None:
        """Collective: the ranks meet first, so that nobody still reads a buffer that goes away."""
        if self._comm is None:
            return
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
        self.bytes_view = None
        self.pkg._check(self.lib.ixk_comm_destroy(self._comm))
        self._comm = None
