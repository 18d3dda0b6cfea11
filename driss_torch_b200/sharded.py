"""Row-sharded quantization of one large matrix over the GPUs of a node.

One process per GPU (``torch.distributed``, NCCL over NVLink/NVSwitch).  Every op on this
path is independent per element, per 32-element block or per row, so rank ``g`` simply
runs the single-GPU kernels on its rows; the one cross-rank dependency is the tensor-wise
amax, a single fp32 that is max-all-reduced between the amax kernel and the cast kernel.
``max`` of non-negative floats is exact and order independent, so the sharded payload is
bit-identical to the single-GPU payload of the concatenated matrix.

The reference has no multi-GPU path; the per-shard arithmetic is its kernels'
(src/amax.cu:50-80, src/dynamic_scaled_quant.cu:111-117, src/mx_cast.cu:44-86,:131-155).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_rows(rows: int, world_size: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Rows ``[start, stop)`` owned by ``rank``: contiguous, in rank order, sizes a multiple of
    ``multiple`` except possibly the last non-empty shard, and as even as that allows."""
    if rows < 0 or world_size <= 0 or not (0 <= rank < world_size) or multiple <= 0:
        raise ValueError("invalid sharding request")
    units = -(-rows // multiple)  # ceil
    base, extra = divmod(units, world_size)
    first_unit = rank * base + min(rank, extra)
    n_units = base + (1 if rank < extra else 0)
    start = min(rows, first_unit * multiple)
    stop = min(rows, (first_unit + n_units) * multiple)
    return start, stop


class ExchangeTimeout(RuntimeError):
    """A bounded device-side wait for a peer's value gave up."""


class _CudaKernels:
    """The product kernels; resolved lazily so that importing this module needs no GPU."""

    def __getattr__(self, name):
        import driss_torch_b200 as pkg

        return getattr(pkg, name)


class ShardedQuantizer:
    """Quantizes this rank's row shard of a matrix that is row-sharded over ``group``.

    ``kernels`` supplies ``amax``, ``cast_with_amax``, ``dynamic_scaled_quant_with_scale``,
    ``mx_fp8_quantize``, ``mx_fp8_quantize_with_amax`` and ``dynamic_scaled_quant_rowwise``; it defaults to this package's CUDA ops and exists so
    that the host logic can be exercised on CPU ranks with another implementation.
    """

    #: Polls a rank spends waiting for its peers' maxima before it gives up (each poll is a round trip to
    #: its own exchange buffer plus a short sleep: this default is on the order of half a minute, so that
    #: ordinary skew between processes -- a first-iteration compile, a data-loader stall -- never trips it).
    DEFAULT_SPIN_LIMIT = 1 << 24

    def __init__(self, group: Optional[dist.ProcessGroup] = None, kernels=None, fused_exchange: bool = False,
                 device=None, spin_limit: Optional[int] = None, exchange_buffers: Optional[Sequence[int]] = None,
                 rank: Optional[int] = None):
        """``fused_exchange=True`` (CUDA ranks of one node only): ``tensorwise`` becomes ONE kernel launch
        per GPU that exchanges the per-GPU maxima itself through NVLink peer memory instead of calling a
        collective between an amax launch and a cast launch.  It needs a small symmetric buffer, set up
        here once (a collective call: construct the quantizer on every rank).

        ``spin_limit``: how long a rank waits for its peers inside the kernel (see DEFAULT_SPIN_LIMIT).  A
        wait that runs out does not hang the GPU: the kernel returns, amax / scale come back as NaN, and
        the next call on this quantizer -- or ``check()`` -- raises ``ExchangeTimeout``.

        ``exchange_buffers`` / ``rank``: for a host that maps the peers' exchange buffers itself instead of
        going through ``torch.distributed`` symmetric memory: entry r is rank r's buffer
        (``dtq_p2p_exchange_bytes()`` zero-filled bytes) as addressable from this device."""
        self.group = group
        self.kernels = _CudaKernels() if kernels is None else kernels
        self.spin_limit = self.DEFAULT_SPIN_LIMIT if spin_limit is None else int(spin_limit)
        self._exchange = None
        self._rank = rank
        self._watched = {}  # workspace data_ptr -> (workspace, pinned mirror of its status word)
        if exchange_buffers is not None:
            if rank is None or not (0 <= rank < len(exchange_buffers)):
                raise ValueError("exchange_buffers needs this process's rank among them")
            self._exchange = dict(buffer=None, handle=None, ptrs=[int(p) for p in exchange_buffers], epoch=0)
        elif fused_exchange:
            self._setup_exchange(device)

    def _setup_exchange(self, device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi

        if not dist.is_initialized():
            raise RuntimeError("fused_exchange needs an initialised process group (one process per GPU)")
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        nwords = _cabi.load().dtq_p2p_exchange_bytes() // 8
        buf = symm_mem.empty(nwords, dtype=torch.int64, device=device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        handle = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's buffer is zero before anybody's first launch
        self._exchange = dict(buffer=buf, handle=handle, ptrs=[int(p) for p in handle.buffer_ptrs], epoch=0)

    @property
    def world_size(self) -> int:
        if self._exchange is not None and self._exchange["handle"] is None:
            return len(self._exchange["ptrs"])
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        if self._rank is not None:
            return self._rank
        return dist.get_rank(self.group) if dist.is_initialized() else 0

    # ---- a peer that never arrives ---------------------------------------------------------------------
    def _workspace(self, shard: torch.Tensor) -> torch.Tensor:
        """The workspace of the shard's device and current stream, watched from now on by ``check``."""
        from . import _cabi

        ws = _cabi.workspace(shard.device)
        if ws.data_ptr() not in self._watched:
            self._watched[ws.data_ptr()] = (ws, torch.zeros(1, dtype=torch.int32).pin_memory())
        return ws

    def _mirror_status(self, ws: torch.Tensor) -> None:
        from . import _cabi

        _cabi.workspace_status_async(ws, self._watched[ws.data_ptr()][1])

    def check(self, synchronize: bool = False) -> None:
        """Raises ``ExchangeTimeout`` if a bounded device-side wait of an earlier call on this quantizer gave
        up (a peer never made the matching call).  Without ``synchronize`` nothing blocks: the status words
        are read from pinned host mirrors that each exchanging call refreshes behind itself, so a timeout
        shows here once the stream has passed that call.  With ``synchronize`` the streams are drained first."""
        from . import _cabi

        for ws, mirror in self._watched.values():
            status = _cabi.workspace_status(ws) if synchronize else int(mirror.item())
            if status != 0:
                raise ExchangeTimeout(
                    f"rank {self.rank}: {_cabi.load().dtq_status_string(status).decode()} (status {status}): a peer did not "
                    "make the matching call in time; the amax / scale / payload of that call are not valid, and the "
                    "workspace must be re-initialised (dtq_workspace_init) before it is used again")

    def global_amax(self, shard: torch.Tensor) -> torch.Tensor:
        """max |x| over every rank's shard, as fp32 [1] on the shard's device (one collective)."""
        local = self.kernels.amax(shard)
        # an empty shard contributes -inf; clamp so that it cannot win the reduction
        local = torch.clamp_min(local, 0.0)
        if self.world_size > 1:
            dist.all_reduce(local, op=dist.ReduceOp.MAX, group=self.group)
        return local

    def tensorwise(self, shard: torch.Tensor, dtype: torch.dtype):
        """Tensor-wise dynamic quantisation of the whole sharded matrix.

        Returns ``(payload_shard, amax[1], scale[1])``; amax and scale are global.  A single rank
        needs no exchange and takes the fused single-launch op.
        """
        if self._exchange is not None:
            return self._tensorwise_fused_exchange(shard, dtype)
        if self.world_size == 1:
            return self.kernels.dynamic_scaled_quant_with_scale(shard, dtype)
        amax = self.global_amax(shard)
        payload, scale = self.kernels.cast_with_amax(shard, amax, dtype)
        return payload, amax, scale

    def _tensorwise_fused_exchange(self, shard: torch.Tensor, dtype: torch.dtype):
        from . import _cabi

        self.check()
        ex = self._exchange
        ex["epoch"] += 1  # the same sequence on every rank: all ranks make the same calls
        if not shard.is_contiguous():
            raise ValueError("the shard must be contiguous")
        amax = torch.empty(1, dtype=torch.float32, device=shard.device)
        scale = torch.empty(1, dtype=torch.float32, device=shard.device)
        ws = self._workspace(shard)
        payload = _cabi.dynamic_scaled_quant_p2p(shard, dtype, ex["ptrs"], self.rank, ex["epoch"], amax_out=amax,
                                                 scale_out=scale, ws=ws, spin_limit=self.spin_limit)
        self._mirror_status(ws)
        return payload, amax, scale

    def tensorwise_and_mx(self, shard: torch.Tensor, dtype: torch.dtype):
        """Both quantisations of the sharded matrix in two reads of the shard instead of three.

        The MX cast computes every chunk's largest magnitude anyway, so it also delivers the shard's amax;
        the maxima of the shards meet either in that call's own one-warp finishing launch (``fused_exchange``:
        it exchanges them through NVLink peer memory) or in one MAX all-reduce; the tensor-wise cast
        follows.  Returns ``(payload, amax[1], scale[1], mx_payload, mx_scales)``, bit-identical to
        ``tensorwise`` + ``mx``.
        """
        if not shard.is_contiguous():
            raise ValueError("the shard must be contiguous")
        if self._exchange is not None:
            from . import _cabi

            self.check()
            ex = self._exchange
            ex["epoch"] += 1
            ws = self._workspace(shard)
            mx_payload, mx_scales, amax = _cabi.mx_fp8_quantize_amax(shard, ws=ws, peer_ptrs=ex["ptrs"], rank=self.rank,
                                                                      epoch=ex["epoch"], spin_limit=self.spin_limit)
            payload, scale = self.kernels.cast_with_amax(shard, amax, dtype)
            self._mirror_status(ws)
            return payload, amax, scale, mx_payload, mx_scales
        else:
            mx_payload, mx_scales, amax = self.kernels.mx_fp8_quantize_with_amax(shard)
            if self.world_size > 1:
                dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        payload, scale = self.kernels.cast_with_amax(shard, amax, dtype)
        return payload, amax, scale, mx_payload, mx_scales

    def mx(self, shard: torch.Tensor):
        """MX block-32 cast of this rank's rows; no communication."""
        return self.kernels.mx_fp8_quantize(shard)

    def rowwise(self, shard: torch.Tensor, dtype: torch.dtype):
        """Row-wise dynamic quantisation of this rank's rows; no communication."""
        return self.kernels.dynamic_scaled_quant_rowwise(shard, dtype)
