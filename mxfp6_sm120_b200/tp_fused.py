"""Peer-memory all-reduce fused into the residual + RMSNorm + MXFP8 kernel (one node).

Set-up exchanges CUDA IPC handles of one symmetric block per rank over the process group's
host channel (``all_gather_object``); after that the data path is one kernel per
row-parallel projection: flags and partial rows travel as plain peer stores / loads over
NVLink.  See ``csrc/tp_fused.cu`` for the protocol.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ._loader import check, library, load_library
from .ops import MXFP8Tensor, _require_sm100, _stream, packed_scale_numel

HEADER_BYTES = 1024


class _DeviceBytes:
    """Minimal ``__cuda_array_interface__`` holder: lets torch view library-owned memory."""

    def __init__(self, pointer: int, size: int):
        self.__cuda_array_interface__ = {
            "shape": (size,), "typestr": "|u1", "data": (pointer, False), "version": 2,
        }


class SymmetricBlocks:
    """This rank's symmetric block plus mappings of every peer's block."""

    def __init__(self, max_rows: int, hidden: int, device: torch.device, group=None):
        _require_sm100(device)
        load_library()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("at most 8 ranks of one node")
        self.device = device
        self.partial_bytes = (max_rows * hidden * 2 + 255) // 256 * 256
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        failure = None
        try:
            with torch.cuda.device(device):
                check(library().mxfp6_tp_block_alloc(self.partial_bytes, ctypes.byref(own), handle))
        except Exception as error:  # reported to every rank below, so that none waits alone
            failure = f"rank {self.rank}: {error}"
        self._own = own.value or 0
        handles = [None] * self.world
        mine = bytes(handle) if failure is None else None
        if self.world > 1:
            dist.all_gather_object(handles, mine, group=group)
        else:
            handles[0] = mine
        self._opened: list[int] = []
        pointers = []
        try:
            if any(raw is None for raw in handles):
                raise RuntimeError(failure or "a peer could not allocate its block")
            for r, raw in enumerate(handles):
                if r == self.rank:
                    pointers.append(self._own)
                    continue
                peer = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(raw)
                with torch.cuda.device(device):
                    check(library().mxfp6_tp_block_open(buf, ctypes.byref(peer)))
                self._opened.append(peer.value)
                pointers.append(peer.value)
        except Exception as error:  # reported to every rank below, so that none waits alone
            failure = f"rank {self.rank}: {error}"
        if self.world > 1:
            failures = [None] * self.world
            dist.all_gather_object(failures, failure, group=group)  # also: every block is mapped
            failure = next((f for f in failures if f is not None), None)
        if failure is not None:
            raise RuntimeError(f"could not map the peers' symmetric blocks ({failure})")
        self._blocks = (ctypes.c_void_p * self.world)(*pointers)
        size = HEADER_BYTES + 2 * self.partial_bytes
        self._bytes = torch.as_tensor(_DeviceBytes(self._own, size), device=device)
        self._next = 0
        self._last: int | None = None

    def _take(self, buffer: int) -> int:
        """Books ``buffer`` for the next collective.

        Two collectives in a row on one buffer are refused: passing the handshake of a step
        proves that the peers have STARTED it, not that they have finished reading this
        rank's buffer.  (The kernels check the same on the device, status 302, which also
        covers a replayed CUDA graph that ends and starts on the same buffer.)"""
        if buffer not in (0, 1):
            raise ValueError("buffer must be 0 or 1")
        if self.world > 1 and buffer == self._last:
            raise ValueError(
                f"buffer {buffer} was used by the previous collective; consecutive collectives "
                "must alternate the two partial buffers")
        self._last = buffer
        self._next = buffer ^ 1
        return buffer

    def partial(self, buffer: int, rows: int, hidden: int) -> torch.Tensor:
        """BF16 ``[rows, hidden]`` view of this rank's partial buffer ``buffer`` (GEMM output)."""
        if rows * hidden * 2 > self.partial_bytes:
            raise ValueError("the symmetric block is too small for this activation")
        begin = HEADER_BYTES + buffer * self.partial_bytes
        return self._bytes[begin : begin + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden)

    def next_partial(self, rows: int, hidden: int) -> torch.Tensor:
        """Partial buffer the next fused call will reduce (buffers alternate per call)."""
        return self.partial(self._next, rows, hidden)

    def allreduce_rmsnorm_quantize(self, x: torch.Tensor, weight: torch.Tensor, eps: float,
                                   values: torch.Tensor, scales: torch.Tensor) -> MXFP8Tensor:
        """``x += sum over ranks of next_partial``; returns MXFP8(RMSNorm(x) * weight)."""
        rows, hidden = (int(v) for v in x.shape)
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x and weight must be contiguous BF16")
        if values.numel() < rows * hidden or scales.numel() < packed_scale_numel(rows, hidden):
            raise ValueError("values / scales are too small")
        buffer = self._take(self._next)
        with torch.cuda.device(self.device):
            check(
                library().mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8(
                    self._blocks, self.world, self.rank, buffer, self.partial_bytes, x.data_ptr(),
                    weight.data_ptr(), float(eps), rows, hidden, values.data_ptr(),
                    scales.data_ptr(), _stream(self.device),
                )
            )
        return MXFP8Tensor(values, scales, rows, hidden)

    def allreduce(self, out: torch.Tensor) -> torch.Tensor:
        """``out = sum over ranks of next_partial`` (BF16 ``[rows, hidden]``, rank order)."""
        rows, hidden = (int(v) for v in out.shape)
        if out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError("out must be contiguous BF16")
        buffer = self._take(self._next)
        with torch.cuda.device(self.device):
            check(
                library().mxfp6_tp_allreduce_bf16(
                    self._blocks, self.world, self.rank, buffer, self.partial_bytes,
                    out.data_ptr(), rows, hidden, _stream(self.device),
                )
            )
        return out

    # From this many bytes per rank on, the all-reduce runs in two phases (slices summed in
    # place, then gathered): every rank then moves 2 (G - 1) / G of the tensor instead of
    # reading all of it from every peer.
    TWO_PHASE_MIN_BYTES = 1 << 20

    def allreduce_any(self, out: torch.Tensor) -> torch.Tensor:
        """:meth:`allreduce` for small outputs, the two-phase form for large ones."""
        rows, hidden = (int(v) for v in out.shape)
        if rows * hidden * 2 < self.TWO_PHASE_MIN_BYTES or rows % self.world:
            return self.allreduce(out)
        if out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError("out must be contiguous BF16")
        buffer = self._take(self._next)
        with torch.cuda.device(self.device):
            check(
                library().mxfp6_tp_allreduce_two_phase_bf16(
                    self._blocks, self.world, self.rank, buffer, self.partial_bytes,
                    out.data_ptr(), rows, hidden, _stream(self.device),
                )
            )
        return out

    def allgather(self, buffer: int, segments) -> None:
        """``segments`` = up to four ``(offset_bytes, tensor)``: the ``tensor.nbytes / world``
        bytes at ``offset_bytes`` of every rank's partial buffer ``buffer`` are gathered into
        ``tensor`` in rank order.  One handshake for all segments."""
        count = len(segments)
        offsets = (ctypes.c_int64 * count)(*[int(o) for o, _ in segments])
        sizes = (ctypes.c_int64 * count)(
            *[t.numel() * t.element_size() // self.world for _, t in segments])
        dsts = (ctypes.c_void_p * count)(*[t.data_ptr() for _, t in segments])
        self._take(buffer)
        with torch.cuda.device(self.device):
            check(
                library().mxfp6_tp_allgather(
                    self._blocks, self.world, self.rank, buffer, self.partial_bytes, count, offsets,
                    sizes, dsts, _stream(self.device),
                )
            )

    def reduce_scatter(self, buffer: int, out: torch.Tensor) -> torch.Tensor:
        """``out [rows, hidden]`` = sum over ranks of rows ``[rank * rows, (rank + 1) * rows)``
        of every rank's BF16 ``[world * rows, hidden]`` partial in buffer ``buffer``."""
        rows, hidden = (int(v) for v in out.shape)
        if out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError("out must be contiguous BF16")
        self._take(buffer)
        with torch.cuda.device(self.device):
            check(
                library().mxfp6_tp_reduce_scatter_bf16(
                    self._blocks, self.world, self.rank, buffer, self.partial_bytes,
                    out.data_ptr(), rows, hidden, _stream(self.device),
                )
            )
        return out

    def view(self, buffer: int, offset: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Typed view of ``shape`` at ``offset`` bytes inside this rank's partial buffer."""
        elements = 1
        for d in shape:
            elements *= d
        size = elements * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + size > self.partial_bytes:
            raise ValueError("view must be 16-byte aligned and inside the partial buffer")
        begin = HEADER_BYTES + buffer * self.partial_bytes + offset
        return self._bytes[begin : begin + size].view(dtype).view(shape)

    def close(self) -> None:
        """Unmap the peers' blocks and free this rank's (call on every rank, between steps)."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)  # no kernel of any rank still uses a block
            for pointer in self._opened:
                check(library().mxfp6_tp_block_close(ctypes.c_void_p(pointer)))
            self._opened = []
            if self.world > 1:
                # An exported allocation may be freed only after every importer has closed
                # its mapping of it.
                dist.barrier(group=self.group)
            if self._own:
                self._bytes = None
                check(library().mxfp6_tp_block_free(ctypes.c_void_p(self._own)))
                self._own = 0
