"""Quantizing a matrix that lives in HOST memory: the end-to-end path a caller with host
buffers takes.

The matrix is cut into row chunks.  Three streams overlap the host->device copy of chunk
c+1, the kernels of chunk c and the device->host copy of finished outputs:

  pass A (per chunk)  H2D -> local amax -> MX cast -> D2H of MX payload/scales
  reduce              amax over the per-chunk partials (and over ranks, if sharded)
  pass B (per chunk)  tensor-wise cast with the global amax -> D2H of the payload

The input stays resident on the device between the passes (it is read by pass B from HBM,
not copied again).  All buffers are allocated once in the constructor; ``run`` allocates
nothing and ends with one stream synchronisation.  Kernels are called through the C ABI
with preallocated outputs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi

E4M3 = torch.float8_e4m3fn


class HostQuantizer:
    def __init__(self, rows: int, cols: int, device, chunk_rows: int = 8192, fp8_dtype: torch.dtype = E4M3,
                 group: Optional[dist.ProcessGroup] = None):
        if cols % 32:
            raise ValueError("cols must be a multiple of 32 (MX block)")
        self.rows, self.cols, self.chunk_rows = rows, cols, min(chunk_rows, max(rows, 1))
        self.device = torch.device(device)
        self.fp8_dtype = fp8_dtype
        self.group = group
        self.nchunks = -(-rows // self.chunk_rows)
        dev = self.device
        self.x = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        self.payload = torch.empty(rows, cols, dtype=fp8_dtype, device=dev)
        self.mx_payload = torch.empty(rows, cols, dtype=E4M3, device=dev)
        self.mx_scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=dev)
        self.partials = torch.zeros(max(self.nchunks, 1), dtype=torch.float32, device=dev)
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.scale = torch.zeros(1, dtype=torch.float32, device=dev)
        self.s_in = torch.cuda.Stream(dev)
        self.s_compute = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        with torch.cuda.stream(self.s_compute):
            self.ws = _cabi.workspace(dev)
        self.launches = 0

    def _span(self, c):
        r0 = c * self.chunk_rows
        return r0, min(self.rows, r0 + self.chunk_rows)

    def run(self, x_host: torch.Tensor, payload_host: torch.Tensor, mx_payload_host: torch.Tensor,
            mx_scales_host: torch.Tensor):
        """``x_host`` bf16 [rows, cols] (pinned for asynchronous copies); the three outputs are host
        tensors of the matching fp8 / e8m0 shapes.  Returns (amax[1], scale[1]) device tensors."""
        assert x_host.shape == (self.rows, self.cols) and x_host.dtype == torch.bfloat16
        bpr = self.cols // 32
        launches = 0
        ready_in, done_a = [], []
        for c in range(self.nchunks):
            r0, r1 = self._span(c)
            with torch.cuda.stream(self.s_in):
                self.x[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                ready_in.append(ev)
        for c in range(self.nchunks):
            r0, r1 = self._span(c)
            with torch.cuda.stream(self.s_compute):
                self.s_compute.wait_event(ready_in[c])
                _cabi.amax(self.x[r0:r1], out=self.partials[c : c + 1], ws=self.ws)
                _cabi.mx_fp8_quantize(self.x[r0:r1], payload=self.mx_payload[r0:r1],
                                      scales=self.mx_scales[r0 * bpr : r1 * bpr])
                launches += 2
                ev = torch.cuda.Event()
                ev.record()
                done_a.append(ev)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done_a[c])
                mx_payload_host[r0:r1].copy_(self.mx_payload[r0:r1], non_blocking=True)
                mx_scales_host[r0 * bpr : r1 * bpr].copy_(self.mx_scales[r0 * bpr : r1 * bpr], non_blocking=True)
        with torch.cuda.stream(self.s_compute):
            # max over the per-chunk partials (each >= 0 or -inf for an empty chunk)
            _cabi.amax(self.partials.view(1, -1), out=self.amax, ws=self.ws)
            launches += 1
            if self.group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
                self.amax.clamp_min_(0.0)
                dist.all_reduce(self.amax, op=dist.ReduceOp.MAX, group=self.group)
            for c in range(self.nchunks):
                r0, r1 = self._span(c)
                _cabi.cast_with_amax(self.x[r0:r1], self.amax, self.fp8_dtype, out=self.payload[r0:r1],
                                     scale_out=self.scale)
                launches += 1
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev)
                    payload_host[r0:r1].copy_(self.payload[r0:r1], non_blocking=True)
        self.s_out.synchronize()
        self.s_compute.synchronize()
        self.launches = launches
        return self.amax, self.scale
