"""Full-size checks (GPU) at the benchmark configurations, where the CPU oracle would take too
long: the CUDA kernels against the tensor-level eager forms of the same arithmetic evaluated
with stock PyTorch ops on the GPU (an independent implementation), plus size-independent
properties: chunked == whole, a checksum of checksums, dequantisation error bounds."""
import pytest
import torch

from conftest import as_bytes
from driss_torch_b200 import workloads
from oracle import eager
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu
E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def _same(a, b, what):
    a8, b8 = a.view(torch.uint8), b.view(torch.uint8)
    if not torch.equal(a8, b8):
        raise AssertionError(f"{what}: {(a8 != b8).sum().item()} of {a8.numel()} bytes differ")


def test_cfg1_saturated_cast_full_size():
    import driss_torch_b200 as dt

    x = workloads.make_cfg1(device="cuda")
    scale = workloads.tensor_scale(x, E4M3)
    got = dt.saturated_cast(x, scale, E4M3)
    _same(got, eager.saturated_cast_kernel_faithful(x, scale, E4M3), "cfg1 vs eager (bf16 scale)")
    rows = slice(1000, 1064)
    _same(got[rows].cpu(), qo.saturated_cast(x[rows].cpu(), scale.item(), E4M3), "cfg1 rows vs oracle")


@pytest.mark.parametrize("fp8_dtype", [E4M3, E5M2])
def test_cfg2_amax_and_fused_full_size(fp8_dtype):
    import driss_torch_b200 as dt

    x = workloads.make_cfg2(device="cuda")
    amax = dt.amax(x)
    assert amax.item() == x.abs().max().float().item()
    p, am, sc = dt.dynamic_scaled_quant_with_scale(x, fp8_dtype)
    assert am.item() == amax.item()
    _same(p, eager.dynamic_scaled_quant_eager(x, fp8_dtype), "cfg2 fused vs eager (fp64)")
    _same(dt.dynamic_scaled_quant(x, fp8_dtype), p, "with and without extra outputs")
    p2, sc2 = dt.cast_with_amax(x, amax, fp8_dtype)
    _same(p2, p, "amax + cast vs fused")
    assert sc2.item() == sc.item()
    rows = slice(4000, 4032)
    want, _ = qo.cast_with_amax(x[rows].cpu(), amax.item(), fp8_dtype)
    _same(p[rows].cpu(), want, "cfg2 rows vs oracle")


def test_cfg3_mx_full_size():
    import driss_torch_b200 as dt

    x = workloads.make_cfg3(device="cuda")
    p, s = dt.mx_fp8_quantize(x)
    ep, es = eager.mx_fp8_quantize_eager(x)
    _same(p, ep, "cfg3 payload vs eager")
    _same(s, es, "cfg3 scales vs eager")
    assert not p.float().isnan().any()
    # dequantised value within half an e4m3 step of the scaled input
    scale = torch.ldexp(torch.ones((), device="cuda"), s.view(torch.uint8).to(torch.int32) - 127).view(x.shape[0], -1, 1)
    deq = p.float().view(x.shape[0], -1, 32) * scale
    err = (deq - x.float().view(x.shape[0], -1, 32)).abs()
    assert (err <= scale * 16.0 + 1e-30).all()  # largest e4m3 step below 256 is 32
    rows = slice(9000, 9016)
    wp, ws_ = qo.mx_fp8_quantize(x[rows].cpu())
    _same(p[rows].cpu(), wp, "cfg3 rows vs oracle")


def test_cfg4_rowwise_full_size():
    import driss_torch_b200 as dt

    x = workloads.make_cfg4(device="cuda")
    p, am, sc = dt.dynamic_scaled_quant_rowwise(x, E4M3)
    ep, eam, esc = eager.dynamic_scaled_quant_rowwise_eager(x, E4M3)
    _same(p, ep, "cfg4 payload vs eager (fp64)")
    assert torch.equal(am, eam) and torch.equal(sc, esc)
    # every row uses its full range: the row maximum maps to +-448
    assert (p.float().abs().amax(dim=1) == 448.0).all()


def test_large_input_split_path_and_chunk_invariance():
    # 384 MiB: above the size where the fused op issues amax + cast launches instead of its
    # single launch; the result must not depend on that, nor on how the rows are chunked.
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    x = torch.cat([workloads.make_cfg5_chunk(c, rows=3072, device="cuda") for c in range(8)])
    assert x.numel() * 2 > 320 << 20
    p, am, sc = dt.dynamic_scaled_quant_with_scale(x, E4M3)
    assert am.item() == x.abs().max().float().item()
    _same(p, eager.dynamic_scaled_quant_eager(x, E4M3), "split path vs eager (fp64)")
    parts = [dt.cast_with_amax(x[i * 3072:(i + 1) * 3072], am, E4M3)[0] for i in range(8)]
    _same(torch.cat(parts), p, "chunked vs whole")
    mx_p, mx_s = dt.mx_fp8_quantize(x)
    mx_parts = [dt.mx_fp8_quantize(x[i * 3072:(i + 1) * 3072]) for i in range(8)]
    _same(torch.cat([q[0] for q in mx_parts]), mx_p, "mx chunked vs whole")
    _same(torch.cat([q[1] for q in mx_parts]), mx_s, "mx scales chunked vs whole")
    # checksum of checksums
    total = sum(int(q.view(torch.uint8).sum(dtype=torch.int64)) for q in parts)
    assert total == int(p.view(torch.uint8).sum(dtype=torch.int64))
    assert _cabi.workspace_status(_cabi.workspace()) == 0
    dt.check_device_status()


def test_two_orientation_ops_full_size_are_the_base_ops_and_their_transposes():
    # size-independent properties at the benchmark shapes: the row-major outputs are the base ops' outputs,
    # the transposed outputs are the base ops on the transposed input (MX) or the transposed payload (elementwise casts)
    import driss_torch_b200 as dt

    x = workloads.make_cfg3(device="cuda")  # [16384, 8192]
    p, s = dt.mx_fp8_quantize(x)
    dp, ds, dpt, dst = dt.mx_fp8_quantize_dual(x)
    _same(dp, p, "dual payload")
    _same(ds, s, "dual scales")
    xt = x.t().contiguous()
    pt, st = dt.mx_fp8_quantize(xt)
    _same(dpt, pt, "dual transposed payload")
    _same(dst, st, "dual transposed scales")
    del xt, pt, st, dpt, dst
    mp, ms, am = dt.mx_fp8_quantize_with_amax(x)
    _same(mp, p, "payload of the MX cast that delivers the amax")
    _same(ms, s, "its scales")
    assert am.item() == dt.amax(x).item()
    x2 = workloads.make_cfg2(device="cuda")  # [8192, 8192]
    for fp8_dtype in (E4M3, E5M2):
        want = dt.dynamic_scaled_quant(x2, fp8_dtype)
        q, qt, amax, scale = dt.dynamic_scaled_quant_dual(x2, fp8_dtype)
        _same(q, want, "dynamic dual, row-major")
        _same(qt, want.view(torch.uint8).t().contiguous(), "dynamic dual, transposed")
        sc = workloads.tensor_scale(x2, fp8_dtype)
        y = dt.saturated_cast(x2, sc, fp8_dtype)
        y2, yt = dt.saturated_cast_dual(x2, sc, fp8_dtype)
        _same(y2, y, "saturated dual, row-major")
        _same(yt, y.view(torch.uint8).t().contiguous(), "saturated dual, transposed")
        _same(dt.saturated_cast_transposed(x2, sc, fp8_dtype), yt, "transposed only")


def test_other_mx_formats_full_size_properties():
    # e5m2 / e2m1 at the cfg3 shape: scale bytes are e4m3's shifted by the formats' exponent difference (no block
    # of this workload is near a clamp), chunked == whole, and dequantised values stay within half a step
    import driss_torch_b200 as dt

    x = workloads.make_cfg3(device="cuda")
    _, s8 = dt.mx_fp8_quantize(x)
    p5, s5 = dt.mx_fp8_quantize(x, ScalarType=E5M2)
    p4, s4 = dt.mx_fp4_quantize(x)
    e8, e5, e4 = (t.view(torch.uint8).int() for t in (s8, s5, s4))
    assert torch.equal(e5, e8 - 7) and torch.equal(e4, e8 + 6)
    half = x.shape[0] // 2
    q4, t4 = dt.mx_fp4_quantize(x[half:])
    _same(q4, p4[half:], "fp4 chunked == whole")
    _same(t4, s4[half * (x.shape[1] // 32):], "fp4 scales chunked == whole")
    rows = slice(5000, 5016)
    want_p, want_s = qo.mx_quantize(x[rows].cpu(), "e2m1")
    _same(p4[rows].cpu(), want_p, "fp4 rows vs oracle")
    want_p, want_s = qo.mx_quantize(x[rows].cpu(), E5M2)
    _same(p5[rows].cpu(), want_p, "e5m2 rows vs oracle")
    # dequantisation: |x - q * 2^(e-127)| <= half the largest step of the format at that block's scale
    scale = torch.exp2(e5.float() - 127).view(x.shape[0], -1, 1)
    err = (p5.float().view(x.shape[0], -1, 32) * scale - x.float().view(x.shape[0], -1, 32)).abs()
    assert bool((err <= scale * 2.0**13 * 0.5 + 1e-30).all())  # e5m2: two mantissa bits, largest binade 2^15


def test_cfg5_full_size_step_vs_oracle_chunk_by_chunk():
    # The benchmark's own workload at its own size: bf16 [262144, 8192] (4 GiB) as 8 seeded row chunks, run through
    # the step the benchmark times (MX cast that delivers the amax, then the tensor-wise cast) and compared with the
    # C oracle byte for byte, one chunk at a time -- the comparison of the reference's own small tests
    # (test/test_dynamic_quant.py:28-44, test/test_mx.py:70-94) at full size.  Host memory stays near 3 GB.
    from driss_torch_b200 import ShardedQuantizer

    chunks, chunk_rows, cols = 8, workloads.CFG5_CHUNK_ROWS, workloads.WORKLOADS["cfg5"].cols
    x = torch.empty(chunks * chunk_rows, cols, dtype=torch.bfloat16, device="cuda")
    oracle_amax = 0.0
    for c in range(chunks):
        part = workloads.make_cfg5_chunk(c)  # CPU generator: the one source of the values
        oracle_amax = max(oracle_amax, qo.amax(part).item())
        x[c * chunk_rows:(c + 1) * chunk_rows].copy_(part)
        del part
    payload, amax, scale, mx_payload, mx_scales = ShardedQuantizer().tensorwise_and_mx(x, E4M3)
    torch.cuda.synchronize()
    assert amax.item() == oracle_amax
    bpr = cols // 32
    sums = [0, 0, 0]
    for c in range(chunks):
        r0, r1 = c * chunk_rows, (c + 1) * chunk_rows
        part = x[r0:r1].cpu()
        want, want_scale = qo.cast_with_amax(part, oracle_amax, E4M3)
        _same(payload[r0:r1].cpu(), want, f"cfg5 tensor-wise payload, chunk {c}")
        assert want_scale.item() == scale.item()
        want_p, want_s = qo.mx_fp8_quantize(part)
        _same(mx_payload[r0:r1].cpu(), want_p, f"cfg5 MX payload, chunk {c}")
        _same(mx_scales[r0 * bpr:r1 * bpr].cpu(), want_s, f"cfg5 MX scales, chunk {c}")
        for i, t in enumerate((want, want_p, want_s)):
            sums[i] += int(t.view(torch.uint8).sum(dtype=torch.int64))
        del part, want, want_p, want_s
    # the byte sums the benchmark prints as output_checksums, from the oracle's outputs
    got = [int(t.view(torch.uint8).sum(dtype=torch.int64)) for t in (payload, mx_payload, mx_scales)]
    assert got == sums
