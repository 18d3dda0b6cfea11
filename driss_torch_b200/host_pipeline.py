"""Quantizing matrices that live in HOST memory: the end-to-end path a caller with host
buffers takes.

A matrix is cut into row chunks.  Three streams overlap the host->device copy of chunk
c+1, the kernels of chunk c and the device->host copy of finished outputs:

  pass A (per chunk)  H2D -> MX cast that also delivers the chunk's amax -> D2H of MX payload/scales
  reduce              amax over the per-chunk values (and over ranks, if sharded)
  pass B (per chunk)  tensor-wise cast with the global amax -> D2H of the payload

The input stays resident on the device between the passes (pass B reads it from HBM, it is
not copied again).  PCIe is the bound: pass B's device->host copy cannot start before the
whole input has arrived (the global amax), so one matrix alone keeps the host->device
direction idle during pass B.  ``submit`` / ``wait`` therefore pipeline consecutive matrices
over ``depth`` sets of device buffers: matrix k+1's input copy runs while matrix k's payload
goes back.  ``run`` is ``wait(submit(...))``.

All buffers are allocated once in the constructor; ``submit`` allocates no device memory.
Kernels are called through the C ABI with preallocated outputs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi

E4M3 = torch.float8_e4m3fn


class _Slot:
    """One set of device buffers: a matrix in flight."""

    def __init__(self, rows, cols, nchunks, fp8_dtype, dev):
        self.x = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        self.payload = torch.empty(rows, cols, dtype=fp8_dtype, device=dev)
        self.mx_payload = torch.empty(rows, cols, dtype=E4M3, device=dev)
        self.mx_scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=dev)
        self.partials = torch.zeros(max(nchunks, 1), dtype=torch.float32, device=dev)
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.scale = torch.zeros(1, dtype=torch.float32, device=dev)
        self.done: Optional[torch.cuda.Event] = None  # the last device->host copy of the matrix using this slot


class Ticket:
    """A submitted matrix: ``amax`` / ``scale`` are device tensors valid after ``HostQuantizer.wait``."""

    def __init__(self, slot: _Slot, done: torch.cuda.Event, launches: int):
        self.amax, self.scale, self.done, self.launches = slot.amax, slot.scale, done, launches


class HostQuantizer:
    def __init__(self, rows: int, cols: int, device, chunk_rows: int = 8192, fp8_dtype: torch.dtype = E4M3,
                 group: Optional[dist.ProcessGroup] = None, depth: int = 1):
        """``depth`` = matrices that may be in flight at once (sets of device buffers: 4.03 bytes per element each)."""
        if cols % 32:
            raise ValueError("cols must be a multiple of 32 (MX block)")
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.rows, self.cols, self.chunk_rows = rows, cols, min(chunk_rows, max(rows, 1))
        self.device = torch.device(device)
        self.fp8_dtype = fp8_dtype
        self.group = group
        self.nchunks = -(-rows // self.chunk_rows)
        dev = self.device
        self.slots = [_Slot(rows, cols, self.nchunks, fp8_dtype, dev) for _ in range(depth)]
        self.s_in = torch.cuda.Stream(dev)
        self.s_compute = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        with torch.cuda.stream(self.s_compute):
            self.ws = _cabi.workspace(dev)
        # the buffers were allocated (and some zero-filled) on the constructor's current stream: their first use
        # on the three side streams must come after that
        for st in (self.s_in, self.s_compute, self.s_out):
            st.wait_stream(torch.cuda.current_stream(dev))
        self.submitted = 0
        self.launches = 0

    def close(self) -> None:
        """Waits for everything in flight and releases the device buffers.  The buffers are used on side
        streams the caching allocator does not know about, so they must not be freed while work is queued."""
        for st in (self.s_in, self.s_compute, self.s_out):
            st.synchronize()
        self.slots = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _span(self, c):
        r0 = c * self.chunk_rows
        return r0, min(self.rows, r0 + self.chunk_rows)

    def submit(self, x_host: torch.Tensor, payload_host: torch.Tensor, mx_payload_host: torch.Tensor,
               mx_scales_host: torch.Tensor, copies_only: bool = False) -> Ticket:
        """Enqueues one matrix and returns at once.  ``x_host`` bf16 [rows, cols] (pinned for asynchronous
        copies); the three outputs are host tensors of the matching fp8 / e8m0 shapes, which must not be
        touched before ``wait``.  If all ``depth`` slots are still in flight, the wait for a free one
        happens on the device streams, not on the host.

        ``copies_only`` issues the same copies on the same streams with the same dependencies but no kernel
        (the outputs are whatever the device buffers hold): the PCIe bound of this pipeline, for benchmarks."""
        assert x_host.shape == (self.rows, self.cols) and x_host.dtype == torch.bfloat16
        slot = self.slots[self.submitted % len(self.slots)]
        self.submitted += 1
        if slot.done is not None:  # the matrix that used this slot must have left the device
            self.s_in.wait_event(slot.done)
            self.s_compute.wait_event(slot.done)
        bpr = self.cols // 32
        launches = 0
        ready_in = []
        with torch.cuda.stream(self.s_in):
            for c in range(self.nchunks):
                r0, r1 = self._span(c)
                slot.x[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                ready_in.append(ev)
        for c in range(self.nchunks):
            r0, r1 = self._span(c)
            with torch.cuda.stream(self.s_compute):
                self.s_compute.wait_event(ready_in[c])
                if not copies_only:
                    _cabi.mx_fp8_quantize_amax(slot.x[r0:r1], payload=slot.mx_payload[r0:r1],
                                               scales=slot.mx_scales[r0 * bpr : r1 * bpr],
                                               amax_out=slot.partials[c : c + 1], ws=self.ws)
                    launches += 2
                ev = torch.cuda.Event()
                ev.record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev)
                mx_payload_host[r0:r1].copy_(slot.mx_payload[r0:r1], non_blocking=True)
                mx_scales_host[r0 * bpr : r1 * bpr].copy_(slot.mx_scales[r0 * bpr : r1 * bpr], non_blocking=True)
        with torch.cuda.stream(self.s_compute):
            # max over the per-chunk values (each >= 0)
            if not copies_only:
                _cabi.amax(slot.partials.view(1, -1), out=slot.amax, ws=self.ws)
                launches += 1
            if not copies_only and (self.group is not None or (dist.is_initialized() and dist.get_world_size() > 1)):
                slot.amax.clamp_min_(0.0)
                dist.all_reduce(slot.amax, op=dist.ReduceOp.MAX, group=self.group)
            for c in range(self.nchunks):
                r0, r1 = self._span(c)
                if not copies_only:
                    _cabi.cast_with_amax(slot.x[r0:r1], slot.amax, self.fp8_dtype, out=slot.payload[r0:r1],
                                         scale_out=slot.scale)
                    launches += 1
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev)
                    payload_host[r0:r1].copy_(slot.payload[r0:r1], non_blocking=True)
        with torch.cuda.stream(self.s_out):
            done = torch.cuda.Event()
            done.record()
        slot.done = done
        if not copies_only:
            self.launches = launches
        return Ticket(slot, done, launches)

    def wait(self, ticket: Ticket):
        """Blocks until the matrix's outputs are in the host tensors; returns (amax[1], scale[1]) device
        tensors (valid until the slot is reused, ``depth`` submissions later)."""
        ticket.done.synchronize()
        return ticket.amax, ticket.scale

    def run(self, x_host: torch.Tensor, payload_host: torch.Tensor, mx_payload_host: torch.Tensor,
            mx_scales_host: torch.Tensor):
        """One matrix, start to finish."""
        return self.wait(self.submit(x_host, payload_host, mx_payload_host, mx_scales_host))
