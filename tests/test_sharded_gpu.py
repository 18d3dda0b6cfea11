"""The row-sharded path with the CUDA kernels (GPU): one process per GPU over NCCL when the box
has several GPUs, and the single-process degenerate case always.  The sharded payload, amax,
scale and MX outputs must equal the CPU oracle's result on the concatenated matrix byte for
byte."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import as_bytes
from driss_torch_b200 import workloads
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn
ROWS, COLS = 2048, 1024


def _expected():
    full = workloads.make_cfg5_shard(0, 1, chunk_rows=ROWS // 8, cols=COLS)
    return full, qo.dynamic_scaled_quant(full, E4M3), qo.mx_fp8_quantize(full), qo.dynamic_scaled_quant_rowwise(full, E4M3)


def test_world_size_one_uses_the_cuda_ops():
    import driss_torch_b200 as dt

    full, (want, want_amax, want_scale), (want_mx_p, want_mx_s), (want_rw, want_rw_amax, want_rw_scale) = _expected()
    q = dt.ShardedQuantizer()
    payload, amax, scale = q.tensorwise(full.cuda(), E4M3)
    assert torch.equal(as_bytes(payload), as_bytes(want))
    assert amax.cpu().view(torch.int32).item() == want_amax.view(torch.int32).item()
    assert scale.cpu().view(torch.int32).item() == want_scale.view(torch.int32).item()
    p, s = q.mx(full.cuda())
    assert torch.equal(as_bytes(p), as_bytes(want_mx_p)) and torch.equal(as_bytes(s), as_bytes(want_mx_s))
    p, am, sc = q.rowwise(full.cuda(), E4M3)
    assert torch.equal(as_bytes(p), as_bytes(want_rw)) and torch.equal(am.cpu(), want_rw_amax) and torch.equal(sc.cpu(), want_rw_scale)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import driss_torch_b200 as dt
        from driss_torch_b200.sharded import shard_rows

        full = workloads.make_cfg5_shard(0, 1, chunk_rows=ROWS // 8, cols=COLS)
        start, stop = shard_rows(ROWS, world, rank, 128)
        shard = full[start:stop].contiguous().cuda()
        q = dt.ShardedQuantizer()
        payload, amax, scale = q.tensorwise(shard, E4M3)
        mx_p, mx_s = q.mx(shard)
        torch.cuda.synchronize()
        dt.check_device_status()
        torch.save(dict(payload=as_bytes(payload), amax=amax.cpu(), scale=scale.cpu(), mx_p=as_bytes(mx_p), mx_s=as_bytes(mx_s)),
                   os.path.join(outdir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ranks_over_nccl_equal_the_single_process_result():
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_worker, args=(world, _free_port(), outdir), nprocs=world, join=True)
        parts = [torch.load(os.path.join(outdir, f"rank{r}.pt")) for r in range(world)]
    full, (want, want_amax, want_scale), (want_mx_p, want_mx_s), _ = _expected()
    assert torch.equal(torch.cat([p["payload"] for p in parts]), as_bytes(want))
    assert torch.equal(torch.cat([p["mx_p"] for p in parts]), as_bytes(want_mx_p))
    assert torch.equal(torch.cat([p["mx_s"] for p in parts]), as_bytes(want_mx_s))
    for p in parts:
        assert p["amax"].view(torch.int32).item() == want_amax.view(torch.int32).item()
        assert p["scale"].view(torch.int32).item() == want_scale.view(torch.int32).item()
