"""The row-sharded path on CPU ranks (gloo, world_size 2 and 4): the host logic -- sharding,
the single max all-reduce, per-shard launches -- is the product's ``ShardedQuantizer``; the
per-shard arithmetic is injected from the CPU oracle, since the product kernels are CUDA only.
The sharded result must equal the single-process result on the concatenated matrix, byte for
byte."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from driss_torch_b200 import workloads
from driss_torch_b200.sharded import ShardedQuantizer, shard_rows
from oracle import quant_oracle as qo

E4M3 = torch.float8_e4m3fn


class OracleKernels:
    """Stands in for the CUDA ops on CPU ranks (test only)."""

    amax = staticmethod(qo.amax)
    mx_fp8_quantize = staticmethod(qo.mx_fp8_quantize)
    dynamic_scaled_quant_rowwise = staticmethod(qo.dynamic_scaled_quant_rowwise)
    dynamic_scaled_quant_with_scale = staticmethod(qo.dynamic_scaled_quant)

    @staticmethod
    def cast_with_amax(x, amax, dtype):
        return qo.cast_with_amax(x, amax.item(), dtype)

    @staticmethod
    def mx_fp8_quantize_with_amax(x):
        p, s = qo.mx_fp8_quantize(x)
        return p, s, torch.clamp_min(qo.amax(x), 0.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, outdir, rows, cols, empty_last):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = workloads.make_cfg5_shard(0, 1, chunk_rows=rows // 8, cols=cols)
        if empty_last:
            start, stop = shard_rows(rows, world - 1, rank, 128) if rank < world - 1 else (rows, rows)
        else:
            start, stop = shard_rows(rows, world, rank, 128)
        shard = full[start:stop].contiguous()
        q = ShardedQuantizer(kernels=OracleKernels())
        assert q.world_size == world and q.rank == rank
        payload, amax, scale = q.tensorwise(shard, E4M3)
        mx_payload, mx_scales = q.mx(shard)
        rw_payload, rw_amax, rw_scale = q.rowwise(shard, E4M3)
        both = q.tensorwise_and_mx(shard, E4M3)  # two reads of the shard instead of three: same bytes
        assert torch.equal(both[0].view(torch.uint8), payload.view(torch.uint8))
        assert both[1].item() == amax.item() and both[2].item() == scale.item()
        assert torch.equal(both[3].view(torch.uint8), mx_payload.view(torch.uint8))
        assert torch.equal(both[4].view(torch.uint8), mx_scales.view(torch.uint8))
        torch.save(
            dict(span=(start, stop), payload=payload.view(torch.uint8), amax=amax, scale=scale,
                 mx_payload=mx_payload.view(torch.uint8), mx_scales=mx_scales.view(torch.uint8),
                 rw_payload=rw_payload.view(torch.uint8), rw_amax=rw_amax, rw_scale=rw_scale),
            os.path.join(outdir, f"rank{rank}.pt"),
        )
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,empty_last", [(2, False), (4, False), (3, True)])
def test_sharded_equals_single_process(world, empty_last):
    rows, cols = 1024, 256
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_worker, args=(world, _free_port(), outdir, rows, cols, empty_last), nprocs=world, join=True)
        parts = [torch.load(os.path.join(outdir, f"rank{r}.pt")) for r in range(world)]
    full = workloads.make_cfg5_shard(0, 1, chunk_rows=rows // 8, cols=cols)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(full, E4M3)
    want_mx_p, want_mx_s = qo.mx_fp8_quantize(full)
    want_rw, want_rw_amax, want_rw_scale = qo.dynamic_scaled_quant_rowwise(full, E4M3)
    assert [p["span"][0] for p in parts] == sorted(p["span"][0] for p in parts)
    assert torch.equal(torch.cat([p["payload"] for p in parts]), want.view(torch.uint8))
    for p in parts:
        assert p["amax"].view(torch.int32).item() == want_amax.view(torch.int32).item()
        assert p["scale"].view(torch.int32).item() == want_scale.view(torch.int32).item()
    assert torch.equal(torch.cat([p["mx_payload"] for p in parts]), want_mx_p.view(torch.uint8))
    assert torch.equal(torch.cat([p["mx_scales"] for p in parts]), want_mx_s.view(torch.uint8))
    assert torch.equal(torch.cat([p["rw_payload"] for p in parts]), want_rw.view(torch.uint8))
    assert torch.equal(torch.cat([p["rw_amax"] for p in parts]), want_rw_amax)
    assert torch.equal(torch.cat([p["rw_scale"] for p in parts]), want_rw_scale)


def test_single_process_without_process_group():
    full = workloads.make_cfg5_shard(0, 1, chunk_rows=16, cols=64)
    q = ShardedQuantizer(kernels=OracleKernels())
    assert q.world_size == 1 and q.rank == 0
    payload, amax, scale = q.tensorwise(full, E4M3)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(full, E4M3)
    assert torch.equal(payload.view(torch.uint8), want.view(torch.uint8))
    assert amax.item() == want_amax.item() and scale.item() == want_scale.item()
