"""Fused tensor-wise dynamic quantisation parity (GPU): reference grid
(test/test_dynamic_quant.py:28-44, fp32) extended to bf16, extra outputs, the cast phase
alone, and the row-wise variant."""
import pytest
import torch

from conftest import FP8_DTYPES, IN_DTYPES, assert_fp8_equal
from driss_torch_b200 import workloads
from oracle import eager
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

ROWS = [3, 64, 512, 4096]
COLS = [7, 17, 127, 512, 3212, 4097]


def _bits(t):
    return t.detach().cpu().view(torch.int32).flatten().tolist()


@pytest.mark.parametrize("num_rows", ROWS)
@pytest.mark.parametrize("num_cols", COLS)
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_fused(num_rows, num_cols, in_dtype, fp8_dtype):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(num_rows * 7919 + num_cols)
    a = torch.rand(num_rows, num_cols, generator=g).to(in_dtype)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(a, fp8_dtype)
    ad = a.cuda()
    amax_out = torch.full((1,), -1.0, device="cuda")
    scale_out = torch.full((1,), -1.0, device="cuda")
    got = _cabi.dynamic_scaled_quant(ad, fp8_dtype, amax_out=amax_out, scale_out=scale_out)
    assert_fp8_equal(got, want, fp8_dtype, "fused")
    assert _bits(amax_out) == _bits(want_amax) and _bits(scale_out) == _bits(want_scale)
    # second call on the same workspace; nullable extras
    assert_fp8_equal(_cabi.dynamic_scaled_quant(ad, fp8_dtype), want, fp8_dtype, "fused again")


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_ops_and_signed_outlier_data(in_dtype, fp8_dtype):
    import driss_torch_b200 as dt

    a = workloads.make_cfg2(rows=2048, cols=2048).to(in_dtype)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(a, fp8_dtype)
    ad = a.cuda()
    out = dt.dynamic_scaled_quant(ad, fp8_dtype)
    assert out.dtype == fp8_dtype and out.shape == a.shape
    assert_fp8_equal(out, want, fp8_dtype, "op")
    p, am, sc = dt.dynamic_scaled_quant_with_scale(ad, fp8_dtype)
    assert_fp8_equal(p, want, fp8_dtype, "op with scale")
    assert _bits(am) == _bits(want_amax) and _bits(sc) == _bits(want_scale)
    # eager double-precision formula agrees with the oracle on this data
    assert_fp8_equal(eager.dynamic_scaled_quant_eager(a, fp8_dtype), want, fp8_dtype, "eager")
    # cast phase alone, from the amax op
    p2, sc2 = dt.cast_with_amax(ad, dt.amax(ad), fp8_dtype)
    assert_fp8_equal(p2, want, fp8_dtype, "amax + cast")
    assert _bits(sc2) == _bits(want_scale)


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_every_bf16_bit_pattern_through_the_cast_phase(fp8_dtype):
    from driss_torch_b200 import _cabi

    a = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256)
    for amax in (1.0, 3.3, 1e-30, 65000.0, 0.0):
        want, want_scale = qo.cast_with_amax(a, amax, fp8_dtype)
        scale_out = torch.zeros(1, device="cuda")
        got = _cabi.cast_with_amax(a.cuda(), torch.tensor([amax], device="cuda"), fp8_dtype, scale_out=scale_out)
        assert_fp8_equal(got, want, fp8_dtype, f"amax={amax}")
        assert _bits(scale_out) == _bits(want_scale)


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_every_bf16_pattern_against_every_amax_mantissa(fp8_dtype):
    # amax is itself a bf16 value, so fp8_max / amax is a ratio of small integers and many bf16
    # products land exactly on fp8 rounding ties (up to the 1e-12 in the scale): every mantissa
    # of amax gives a different tie lattice.  One launch per amax over all 65536 inputs.
    from driss_torch_b200 import _cabi

    a = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256)
    ad = a.cuda()
    amax_dev = torch.zeros(1, device="cuda")
    for exponent in (-3, -2, 0, 9, 40, 63, 64, 70):  # the compensated path covers [0.25, 2^64], the bracket path the rest
        for mant in range(128, 256):
            amax = mant / 128.0 * 2.0**exponent
            want, _ = qo.cast_with_amax(a, amax, fp8_dtype)
            got = _cabi.cast_with_amax(ad, amax_dev.fill_(amax), fp8_dtype)
            assert_fp8_equal(got, want, fp8_dtype, f"amax={amax}")


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_fp32_rounding_boundaries(in_dtype):
    # products that land on or next to fp8 midpoints: the double product and its single
    # narrowing to fp32 decide the byte
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(3)
    grid = torch.arange(0, 449, dtype=torch.float32) / 448.0  # amax 1 -> scale ~448: products near integers
    near = torch.cat([grid, torch.nextafter(grid, torch.tensor(2.0)), torch.nextafter(grid, torch.tensor(-1.0)),
                      torch.rand(100_000, generator=g), torch.tensor([1.0])])
    a = near[: near.numel() // 2 * 2].view(2, -1).to(in_dtype).contiguous()
    for fp8_dtype in FP8_DTYPES:
        want, _, _ = qo.dynamic_scaled_quant(a, fp8_dtype)
        assert_fp8_equal(_cabi.dynamic_scaled_quant(a.cuda(), fp8_dtype), want, fp8_dtype, "boundaries")


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_all_zero_and_tiny_inputs(in_dtype):
    from driss_torch_b200 import _cabi

    for a in (torch.zeros(8, 64), torch.full((8, 64), 1e-38), torch.full((3, 5), -2.0)):
        a = a.to(in_dtype)
        want, want_amax, want_scale = qo.dynamic_scaled_quant(a, torch.float8_e4m3fn)
        amax_out, scale_out = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
        got = _cabi.dynamic_scaled_quant(a.cuda(), torch.float8_e4m3fn, amax_out=amax_out, scale_out=scale_out)
        assert_fp8_equal(got, want, torch.float8_e4m3fn, "degenerate")
        assert _bits(amax_out) == _bits(want_amax) and _bits(scale_out) == _bits(want_scale)


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
@pytest.mark.parametrize("numel,offset", [(1, 0), (9, 0), (4099, 0), (100_003, 0), (10_000, 1), (10_000, 3)])
def test_ragged_and_misaligned(in_dtype, numel, offset):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(numel + offset)
    base = torch.randn(numel + 8, generator=g).to(in_dtype)
    a = base[offset : offset + numel].view(1, numel)
    want, _, _ = qo.dynamic_scaled_quant(a.contiguous(), torch.float8_e4m3fn)
    buf = torch.full((numel + 16,), 0x5A, dtype=torch.uint8, device="cuda")
    out = buf[offset : offset + numel].view(torch.float8_e4m3fn).view(1, numel)
    _cabi.dynamic_scaled_quant(base.cuda()[offset : offset + numel].view(1, numel), torch.float8_e4m3fn, out=out)
    assert_fp8_equal(out, want, torch.float8_e4m3fn, "ragged")
    assert (buf[:offset] == 0x5A).all() and (buf[offset + numel :] == 0x5A).all()


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_larger_than_one_wave(in_dtype):
    # more tiles than the blocks keep on chip: the rest are claimed dynamically in both phases (counters in the
    # workspace that alternate with the launch parity), so several launches in a row, the last on other data
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg2(rows=4096, cols=8192 if in_dtype == torch.bfloat16 else 6144).to(in_dtype)
    b = (a.float() * 0.37).to(in_dtype)
    amax_out = torch.zeros(1, device="cuda")
    for x in (a, a, a, b, a):
        want, want_amax, _ = qo.dynamic_scaled_quant(x, torch.float8_e4m3fn)
        got = _cabi.dynamic_scaled_quant(x.cuda(), torch.float8_e4m3fn, amax_out=amax_out)
        assert_fp8_equal(got, want, torch.float8_e4m3fn, "multi-wave")
        assert _bits(amax_out) == _bits(want_amax)
    assert _cabi.workspace_status(_cabi.workspace()) == 0


def test_errors_and_compile():
    import driss_torch_b200 as dt

    a = torch.rand(64, 64, device="cuda")
    with pytest.raises(RuntimeError):
        dt.dynamic_scaled_quant(a, torch.float16)
    with pytest.raises(RuntimeError):
        dt.dynamic_scaled_quant(a.t(), torch.float8_e4m3fn)  # must be contiguous, as in the reference
    with pytest.raises(RuntimeError):
        dt.dynamic_scaled_quant(a.view(-1), torch.float8_e4m3fn)
    for backend in ("aot_eager", "inductor"):  # the reference compiles with the default backend
        torch._dynamo.reset()
        fn = torch.compile(dt.dynamic_scaled_quant, fullgraph=True, backend=backend)
        assert_fp8_equal(fn(a, torch.float8_e4m3fn), dt.dynamic_scaled_quant(a, torch.float8_e4m3fn))
    dt.check_device_status()


# ---- row-wise ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 64), (33, 256), (64, 4096), (17, 4104), (9, 8192), (4, 32768),
                                       (3, 40000), (7, 127), (6, 3212), (2, 65536 + 24)])
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_rowwise(rows, cols, in_dtype, fp8_dtype):
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg4(rows=rows, cols=cols).to(in_dtype)
    want, want_amax, want_scale = qo.dynamic_scaled_quant_rowwise(a, fp8_dtype)
    amax_out = torch.full((rows, 1), -1.0, device="cuda")
    scale_out = torch.full((rows, 1), -1.0, device="cuda")
    got = _cabi.dynamic_scaled_quant_rowwise(a.cuda(), fp8_dtype, amax_out=amax_out, scale_out=scale_out)
    assert_fp8_equal(got, want, fp8_dtype, "rowwise")
    assert _bits(amax_out) == _bits(want_amax) and _bits(scale_out) == _bits(want_scale)


def test_rowwise_op_cfg4_slice_and_zero_rows():
    import driss_torch_b200 as dt

    a = workloads.make_cfg4(rows=2048, cols=4096)
    a[5] = 0
    a[77] = -0.0
    want, want_amax, want_scale = qo.dynamic_scaled_quant_rowwise(a, torch.float8_e4m3fn)
    p, am, sc = dt.dynamic_scaled_quant_rowwise(a.cuda(), torch.float8_e4m3fn)
    assert am.shape == (2048, 1) and sc.shape == (2048, 1)
    assert_fp8_equal(p, want, torch.float8_e4m3fn, "rowwise op")
    assert _bits(am) == _bits(want_amax) and _bits(sc) == _bits(want_scale)
    e_p, e_am, e_sc = eager.dynamic_scaled_quant_rowwise_eager(a, torch.float8_e4m3fn)
    assert_fp8_equal(e_p, want, torch.float8_e4m3fn, "rowwise eager")
    assert _bits(e_am) == _bits(want_amax) and _bits(e_sc) == _bits(want_scale)


def test_ops_capture_into_a_cuda_graph_and_replay():
    # The C ABI neither allocates nor synchronises, so a whole quantisation step can be captured
    # once and replayed on new data in the same buffers.
    from driss_torch_b200 import _cabi

    E4M3 = torch.float8_e4m3fn
    x = workloads.make_cfg2(rows=1024, cols=2048).cuda()
    x2 = workloads.make_cfg3(rows=1024, cols=2048)
    out = torch.empty(x.shape, dtype=E4M3, device="cuda")
    fused = torch.empty_like(out)
    mx_p = torch.empty_like(out)
    mx_s = torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, device="cuda")
    amax, scale = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ws = _cabi.workspace()  # created (and the kernels' one-time set-up done) before the capture
        for _ in range(2):
            _cabi.amax(x, out=amax, ws=ws)
            _cabi.cast_with_amax(x, amax, E4M3, out=out, scale_out=scale)
            _cabi.dynamic_scaled_quant(x, E4M3, out=fused, ws=ws)
            _cabi.mx_fp8_quantize(x, payload=mx_p, scales=mx_s)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        _cabi.amax(x, out=amax, ws=ws)
        _cabi.cast_with_amax(x, amax, E4M3, out=out, scale_out=scale)
        _cabi.dynamic_scaled_quant(x, E4M3, out=fused, ws=ws)
        _cabi.mx_fp8_quantize(x, payload=mx_p, scales=mx_s)
    x.copy_(x2)  # new data, same buffers
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    want, want_amax, want_scale = qo.dynamic_scaled_quant(x2, E4M3)
    assert_fp8_equal(out, want, E4M3, "graph: amax + cast")
    assert_fp8_equal(fused, want, E4M3, "graph: fused")
    assert _bits(amax) == _bits(want_amax) and _bits(scale) == _bits(want_scale)
    wp, ws_ = qo.mx_fp8_quantize(x2)
    assert_fp8_equal(mx_p, wp, E4M3, "graph: mx payload")
    assert torch.equal(mx_s.view(torch.uint8).cpu(), ws_.view(torch.uint8))
    assert _cabi.workspace_status(ws) == 0


def test_shared_read_step_and_two_orientation_casts_capture_into_a_cuda_graph():
    # The step's default composition (MX cast that delivers the amax, its one-warp finishing launch, the cast)
    # and the two-orientation casts, captured once and replayed on new data.
    from driss_torch_b200 import _cabi

    E4M3 = torch.float8_e4m3fn
    x = workloads.make_cfg2(rows=1024, cols=2048).cuda()
    x2 = workloads.make_cfg3(rows=1024, cols=2048)
    out = torch.empty(x.shape, dtype=E4M3, device="cuda")
    mx_p = torch.empty_like(out)
    mx_s = torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, device="cuda")
    amax, scale = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    dual = None
    sat = None
    stream = torch.cuda.Stream()

    def step():
        nonlocal dual, sat
        _cabi.mx_fp8_quantize_amax(x, payload=mx_p, scales=mx_s, amax_out=amax, ws=ws)
        _cabi.cast_with_amax(x, amax, E4M3, out=out, scale_out=scale)
        dual = _cabi.mx_fp8_quantize_dual(x, *(dual or ()))
        sat = _cabi.saturated_cast_transposed(x, scale, E4M3, *((sat[1], sat[0]) if sat else ()), both=True)

    with torch.cuda.stream(stream):
        ws = _cabi.workspace()
        for _ in range(2):
            step()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    x.copy_(x2)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    want, want_amax, want_scale = qo.dynamic_scaled_quant(x2, E4M3)
    assert_fp8_equal(out, want, E4M3, "graph: MX cast with amax + cast")
    assert _bits(amax) == _bits(want_amax) and _bits(scale) == _bits(want_scale)
    wp, ws_ = qo.mx_fp8_quantize(x2)
    wpt, wst = qo.mx_fp8_quantize(x2.t().contiguous())
    assert_fp8_equal(mx_p, wp, E4M3, "graph: mx payload")
    assert torch.equal(mx_s.view(torch.uint8).cpu(), ws_.view(torch.uint8))
    assert_fp8_equal(dual[0], wp, E4M3, "graph: dual payload")
    assert_fp8_equal(dual[2], wpt, E4M3, "graph: dual transposed payload")
    assert torch.equal(dual[3].view(torch.uint8).cpu(), wst.view(torch.uint8))
    # the transposed cast read the scale the graph itself produced
    want_sat = qo.saturated_cast(x2, want_scale.item(), E4M3)
    assert_fp8_equal(sat[0], want_sat, E4M3, "graph: saturated_cast")
    assert_fp8_equal(sat[1], want_sat.t().contiguous(), E4M3, "graph: saturated_cast transposed")
    assert _cabi.workspace_status(ws) == 0


# ---- both orientations of the dynamic cast ----------------------------------------------------------------

DUAL_SHAPES = [(128, 128), (16, 8), (48, 200), (144, 1032), (2048, 1024), (1040, 4104),  # tiled path
               (3, 7), (33, 512), (100, 36), (1, 1)]                                       # byte-tile path


@pytest.mark.parametrize("shape", DUAL_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_dynamic_quant_dual(shape, in_dtype, fp8_dtype):
    import driss_torch_b200 as dt

    a = workloads.make_cfg2(rows=shape[0], cols=shape[1]).to(in_dtype)
    want, want_amax, want_scale = qo.dynamic_scaled_quant(a, fp8_dtype)
    p, p_t, amax, scale = dt.dynamic_scaled_quant_dual(a.cuda(), fp8_dtype)
    assert p.shape == tuple(shape) and p_t.shape == (shape[1], shape[0]) and p_t.is_contiguous()
    assert_fp8_equal(p, want, fp8_dtype, "row-major")
    assert_fp8_equal(p_t, want.t().contiguous(), fp8_dtype, "transposed")
    assert _bits(amax) == _bits(want_amax) and _bits(scale) == _bits(want_scale)


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_cast_with_amax_dual_on_the_tie_lattice_and_with_foreign_amax(fp8_dtype):
    # every bf16 value against amax values that put many products exactly on fp8 rounding ties (compensated
    # path), an amax that is not a bf16 value (bracket path with the double-precision redo), and an amax
    # smaller than the data (saturation)
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256)
    bits = torch.where(bits.float().isnan(), torch.zeros((), dtype=torch.bfloat16), bits)
    xd = bits.cuda()
    for amax_value in (4.0, 5.3125, 448.0, 0.7431640625, 3.1415927, 1e-3):
        am = torch.tensor([amax_value], dtype=torch.float32)
        want, want_scale = qo.cast_with_amax(bits, am.item(), fp8_dtype)
        p, p_t, scale = dt.cast_with_amax_dual(xd, am.cuda(), fp8_dtype)
        assert_fp8_equal(p, want, fp8_dtype, f"row-major, amax {amax_value}")
        assert_fp8_equal(p_t, want.t().contiguous(), fp8_dtype, f"transposed, amax {amax_value}")
        assert _bits(scale) == _bits(want_scale)
        only_t = _cabi.cast_with_amax_transposed(xd, am.cuda(), fp8_dtype)
        assert_fp8_equal(only_t, want.t().contiguous(), fp8_dtype, "transposed only")
        f32 = bits.float()
        want32, _ = qo.cast_with_amax(f32, am.item(), fp8_dtype)
        p32, p32_t, _ = dt.cast_with_amax_dual(f32.cuda(), am.cuda(), fp8_dtype)
        assert_fp8_equal(p32, want32, fp8_dtype, "fp32 row-major")
        assert_fp8_equal(p32_t, want32.t().contiguous(), fp8_dtype, "fp32 transposed")
