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
    both = q.tensorwise_and_mx(full.cuda(), E4M3)
    assert torch.equal(as_bytes(both[0]), as_bytes(want)) and both[1].item() == want_amax.item()
    assert both[2].item() == want_scale.item()
    assert torch.equal(as_bytes(both[3]), as_bytes(want_mx_p)) and torch.equal(as_bytes(both[4]), as_bytes(want_mx_s))
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
        # the same through ONE launch per GPU that exchanges the maxima itself over peer memory;
        # several calls in a row (the exchange slots alternate with the call count), the last one on
        # different data so that a stale value from an earlier call would show
        qf = dt.ShardedQuantizer(fused_exchange=True)
        for _ in range(3):
            f_payload, f_amax, f_scale = qf.tensorwise(shard, E4M3)
        shard2 = (shard.float() * 0.5).to(torch.bfloat16)
        f2_payload, f2_amax, _ = qf.tensorwise(shard2, torch.float8_e5m2)
        # both quantisations in two reads: MX cast that also delivers the amax (exchanged inside that launch,
        # or by one all-reduce), then the cast; interleaved with the other fused call on the same exchange buffers
        b_f = qf.tensorwise_and_mx(shard, E4M3)
        b_f2 = qf.tensorwise_and_mx(shard2, torch.float8_e5m2)
        b_n = q.tensorwise_and_mx(shard, E4M3)
        torch.cuda.synchronize()
        for b in (b_f, b_n):
            assert torch.equal(as_bytes(b[0]), as_bytes(payload)) and b[1].item() == amax.item() and b[2].item() == scale.item()
            assert torch.equal(as_bytes(b[3]), as_bytes(mx_p)) and torch.equal(as_bytes(b[4]), as_bytes(mx_s))
        assert torch.equal(as_bytes(b_f2[0]), as_bytes(f2_payload)) and b_f2[1].item() == f2_amax.item()
        dt.check_device_status()
        torch.save(dict(payload=as_bytes(payload), amax=amax.cpu(), scale=scale.cpu(), mx_p=as_bytes(mx_p), mx_s=as_bytes(mx_s),
                        f_payload=as_bytes(f_payload), f_amax=f_amax.cpu(), f_scale=f_scale.cpu(),
                        f2_payload=as_bytes(f2_payload), f2_amax=f2_amax.cpu()),
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
        assert p["f_amax"].view(torch.int32).item() == want_amax.view(torch.int32).item()
        assert p["f_scale"].view(torch.int32).item() == want_scale.view(torch.int32).item()
    assert torch.equal(torch.cat([p["f_payload"] for p in parts]), as_bytes(want)), "fused exchange payload"
    half = (full.float() * 0.5).to(torch.bfloat16)
    want2, want2_amax, _ = qo.dynamic_scaled_quant(half, torch.float8_e5m2)
    assert torch.equal(torch.cat([p["f2_payload"] for p in parts]), as_bytes(want2)), "fused exchange, second tensor"
    assert all(p["f2_amax"].item() == want2_amax.item() for p in parts)


def test_fused_exchange_single_rank_and_missing_peer_timeout():
    # world 1: the exchange degenerates to a store and a load on the rank's own buffer.
    # world 2 with a peer that never writes: the bounded wait gives up, the launch returns, the
    # workspace reports DTQ_ERR_TIMEOUT (5) and the context stays usable.
    from driss_torch_b200 import _cabi

    lib = _cabi.load()
    x = workloads.make_cfg2(rows=512, cols=1024)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(x, E4M3)
    xd = x.cuda()
    mine = torch.zeros(lib.dtq_p2p_exchange_bytes() // 8, dtype=torch.int64, device="cuda")
    amax, scale = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    for epoch in (1, 2, 3):
        got = _cabi.dynamic_scaled_quant_p2p(xd, E4M3, [mine.data_ptr()], 0, epoch, amax_out=amax, scale_out=scale)
        assert torch.equal(as_bytes(got), as_bytes(want))
        assert amax.item() == want_amax.item() and scale.item() == want_scale.item()

    silent_peer = torch.zeros_like(mine)
    ws = torch.empty(lib.dtq_workspace_bytes(), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), stream), "init")
    out = torch.full(x.shape, 0x5A, dtype=torch.uint8, device="cuda")
    _cabi.dynamic_scaled_quant_p2p(xd, E4M3, [mine.data_ptr(), silent_peer.data_ptr()], 0, 4, out=out.view(E4M3), ws=ws,
                                   spin_limit=2000)
    torch.cuda.synchronize()  # returns: nothing hangs
    assert _cabi.workspace_status(ws) == 5
    assert (out == 0x5A).all()  # no payload is written without a global maximum
    # the rank's own value did reach the peer's buffer (what a live peer would have read)
    assert (silent_peer.cpu() != 0).sum().item() == 1
    # the MX cast with the amax exchange in its last block: world 1, then the same silent peer
    want_p, want_s = qo.mx_fp8_quantize(x)
    for epoch in (5, 6):
        p, s_, am = _cabi.mx_fp8_quantize_amax(xd, peer_ptrs=[mine.data_ptr()], rank=0, epoch=epoch)
        assert torch.equal(as_bytes(p), as_bytes(want_p)) and torch.equal(as_bytes(s_), as_bytes(want_s))
        assert am.item() == want_amax.item()
    _cabi.check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), stream), "init")
    p, s_, am = _cabi.mx_fp8_quantize_amax(xd, ws=ws, peer_ptrs=[mine.data_ptr(), silent_peer.data_ptr()], rank=0, epoch=7,
                                           spin_limit=2000)
    torch.cuda.synchronize()  # returns: nothing hangs
    assert _cabi.workspace_status(ws) == 5 and torch.isnan(am).all()  # NaN, never a value that could pass for a maximum
    assert torch.equal(as_bytes(p), as_bytes(want_p))  # the MX outputs do not depend on the peers
    # a fresh workspace and the ordinary op still work
    _cabi.check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), stream), "init")
    assert torch.equal(as_bytes(_cabi.dynamic_scaled_quant(xd, E4M3, ws=ws)), as_bytes(want))
    assert _cabi.workspace_status(ws) == 0


def test_sharded_quantizer_reports_a_peer_that_never_arrives():
    # Through the public class, one process: rank 0 of a world of two whose peer buffer nobody writes.  The
    # bounded wait runs out (a small spin_limit keeps that to milliseconds), the launches return, amax and scale
    # come back as NaN so that nothing can consume them unnoticed, and the quantizer raises -- from check(),
    # and by itself at the top of the next exchanging call -- without any GPU fault or hang.
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi
    from driss_torch_b200.sharded import ExchangeTimeout

    lib = _cabi.load()
    x = workloads.make_cfg2(rows=512, cols=1024).cuda()
    nwords = lib.dtq_p2p_exchange_bytes() // 8
    mine = torch.zeros(nwords, dtype=torch.int64, device="cuda")
    silent_peer = torch.zeros_like(mine)
    side = torch.cuda.Stream()  # its own stream, hence its own workspace: the default stream's stays clean
    with torch.cuda.stream(side):
        q = dt.ShardedQuantizer(exchange_buffers=[mine.data_ptr(), silent_peer.data_ptr()], rank=0, spin_limit=2000)
        assert q.world_size == 2 and q.rank == 0
        q.check()  # nothing has run yet
        payload, amax, scale, mx_p, mx_s = q.tensorwise_and_mx(x, E4M3)
        side.synchronize()
        assert torch.isnan(amax).all() and torch.isnan(scale).all()
        want_p, want_s = qo.mx_fp8_quantize(x.cpu())
        assert torch.equal(as_bytes(mx_p), as_bytes(want_p)) and torch.equal(as_bytes(mx_s), as_bytes(want_s))
        with pytest.raises(ExchangeTimeout):
            q.check()  # no synchronisation needed: the pinned mirror was refreshed behind the call
        with pytest.raises(ExchangeTimeout):
            q.tensorwise(x, E4M3)  # the next call refuses to build on a broken exchange
        # the single-launch form reports the same way
        ws = _cabi.workspace(x.device)
        _cabi.check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), side.cuda_stream), "init")
        q2 = dt.ShardedQuantizer(exchange_buffers=[mine.data_ptr(), silent_peer.data_ptr()], rank=0, spin_limit=2000)
        q2._exchange["epoch"] = 10
        _, amax2, scale2 = q2.tensorwise(x, E4M3)
        with pytest.raises(ExchangeTimeout):
            q2.check(synchronize=True)
        assert torch.isnan(amax2).all() and torch.isnan(scale2).all()
        _cabi.check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), side.cuda_stream), "init")
        side.synchronize()
    # the context is intact and the ordinary ops still work
    want, want_amax, _ = qo.dynamic_scaled_quant(x.cpu(), E4M3)
    got, am, _ = dt.dynamic_scaled_quant_with_scale(x, E4M3)
    assert torch.equal(as_bytes(got), as_bytes(want)) and am.item() == want_amax.item()
    dt.check_device_status()
