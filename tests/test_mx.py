"""mx_fp8_quantize parity (GPU) on the reference test's sizes (test/test_mx.py:70-94) and on
the degenerate blocks the reference arithmetic defines (zero / tiny / non-finite)."""
import pytest
import torch

from conftest import as_bytes, assert_fp8_equal
from driss_torch_b200 import workloads
from oracle import eager
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

E4M3 = torch.float8_e4m3fn
SIZES = [(128, 32), (256, 32), (8192, 32), (128, 64), (128, 128), (128, 8192), (256, 64), (256, 128), (8192, 8192)]


def _check(a, what):
    from driss_torch_b200 import _cabi

    want_p, want_s = qo.mx_fp8_quantize(a)
    p, s = _cabi.mx_fp8_quantize(a.cuda())
    assert_fp8_equal(p, want_p, E4M3, what + " payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s)), what + " scales"
    return p, s


@pytest.mark.parametrize("size", SIZES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_mx_cast(size):
    import driss_torch_b200 as dt

    g = torch.Generator().manual_seed(size[0] + size[1])
    a = torch.rand(size, generator=g).to(torch.bfloat16)
    _check(a, "rand")
    data, scale = dt.mx_fp8_quantize(a.cuda())
    assert data.dtype == E4M3 and data.shape == a.shape
    assert scale.dtype == torch.float8_e8m0fnu and scale.shape == (size[0] * size[1] // 32,)
    want_p, want_s = qo.mx_fp8_quantize(a)
    assert_fp8_equal(data, want_p, E4M3, "op payload")
    assert torch.equal(as_bytes(scale), as_bytes(want_s))


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 96), (5, 4128), (130, 160), (1000, 32), (77, 2048)])
def test_rows_need_not_be_a_multiple_of_128(rows, cols):
    _check(workloads.make_cfg3(rows=rows, cols=cols), "ragged rows")


def test_wide_exponent_range_matches_eager_form_too():
    a = workloads.make_cfg3(rows=512, cols=8192)
    p, s = _check(a, "cfg3")
    e_p, e_s = eager.mx_fp8_quantize_eager(a)
    assert_fp8_equal(p, e_p, E4M3, "eager payload")
    assert torch.equal(as_bytes(s), as_bytes(e_s))
    assert not p.float().isnan().any()


def test_every_bf16_pattern_as_block_maximum():
    # block b = [pattern b, then 31 elements that are small relative to it or zero]
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    a = torch.zeros(65536, 32, dtype=torch.bfloat16)
    a[:, 0] = bits
    a[:, 5] = (bits.float() * 0.37).to(torch.bfloat16)
    a[:, 31] = (bits.float() * -0.011).to(torch.bfloat16)
    _check(a.view(8192, 256), "all patterns")


def test_every_bf16_pattern_everywhere_in_a_block():
    # all 65536 patterns laid out contiguously: blocks mix neighbours in value
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    _check(bits.view(64, 1024), "dense patterns")
    g = torch.Generator().manual_seed(1)
    perm = torch.randperm(65536, generator=g)
    _check(bits[perm].view(64, 1024), "shuffled patterns")


def test_degenerate_blocks():
    inf, nan = float("inf"), float("nan")
    rows = [
        [0.0] * 32,                                  # all zero -> scale byte 0, payload NaN bytes
        [-0.0] * 32,
        [2.0**-125] * 16 + [0.0] * 16,               # E <= -119 -> scale 0.0 -> +-448 and NaN
        [2.0**-119, -(2.0**-120)] * 16,
        [2.0**-118] * 32,                            # just inside the normal range
        [1e-40] * 31 + [0.0],                        # subnormals
        [inf] + [1.0] * 31,
        [-inf] * 32,
        [nan] + [1.0] * 31,
        [3.0e38] * 32,                               # largest exponents
        [1.0] * 32,                                  # power of two maximum -> code 0x78 region
        [1.5, -1.0] * 16,
    ]
    a = torch.tensor(rows, dtype=torch.float32).to(torch.bfloat16)
    _check(a, "degenerate")


def test_misaligned_pointers_take_the_scalar_path():
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg3(rows=64, cols=512)
    base = torch.zeros(64 * 512 + 8, dtype=torch.bfloat16, device="cuda")
    view = base[3 : 3 + 64 * 512].view(64, 512)
    view.copy_(a)
    pbuf = torch.zeros(64 * 512 + 8, dtype=torch.uint8, device="cuda")
    payload = pbuf[5 : 5 + 64 * 512].view(E4M3).view(64, 512)
    p, s = _cabi.mx_fp8_quantize(view, payload=payload)
    want_p, want_s = qo.mx_fp8_quantize(a)
    assert_fp8_equal(p, want_p, E4M3, "misaligned payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s))


def test_no_byte_outside_the_outputs_is_written():
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg3(rows=33, cols=96)
    n = a.numel()
    pbuf = torch.full((n + 256,), 0x5A, dtype=torch.uint8, device="cuda")
    sbuf = torch.full((n // 32 + 256,), 0x5A, dtype=torch.uint8, device="cuda")
    _cabi.mx_fp8_quantize(a.cuda(), payload=pbuf[:n].view(E4M3).view(33, 96), scales=sbuf[: n // 32].view(torch.float8_e8m0fnu))
    want_p, want_s = qo.mx_fp8_quantize(a)
    assert_fp8_equal(pbuf[:n].view(E4M3).view(33, 96), want_p, E4M3, "payload")
    assert torch.equal(sbuf[: n // 32].cpu(), as_bytes(want_s))
    assert (pbuf[n:] == 0x5A).all() and (sbuf[n // 32 :] == 0x5A).all()


def test_errors_and_compile():
    import driss_torch_b200 as dt

    a = torch.rand(128, 64, device="cuda").to(torch.bfloat16)
    for bad in (
        lambda: dt.mx_fp8_quantize(a.double()),
        lambda: dt.mx_fp8_quantize(a, block_size=16),
        lambda: dt.mx_fp8_quantize(a, axis=2),
        lambda: dt.mx_fp8_quantize(a[:48], transpose=True),  # rows not a multiple of 32
        lambda: dt.mx_fp8_quantize(a, axis=0, ScalarType=torch.float8_e5m2),
        lambda: dt.mx_fp8_quantize(a, ScalarType=torch.float16),
        lambda: dt.mx_fp4_quantize(a[:, :48]),
        lambda: dt.mx_fp4_quantize(a.double()),
        lambda: dt.mx_fp8_quantize(a[:, :48]),
        lambda: dt.mx_fp8_quantize(a.t()),
        lambda: dt.mx_fp8_quantize(a.view(-1)),
    ):
        with pytest.raises(RuntimeError):
            bad()
    assert dt.mx_cast is dt.mx_fp8_quantize
    torch._dynamo.reset()
    p0, s0 = dt.mx_fp8_quantize(a)
    for backend in ("aot_eager", "inductor"):  # the reference's tests compile with the default backend
        torch._dynamo.reset()
        fn = torch.compile(dt.mx_fp8_quantize, fullgraph=True, backend=backend)
        p, s = fn(a)
        assert torch.equal(as_bytes(p), as_bytes(p0)) and torch.equal(as_bytes(s), as_bytes(s0))


@pytest.mark.parametrize("rows,cols", [(32, 32), (128, 64), (96, 288), (1024, 512)])
def test_axis_and_transpose_arguments_of_the_schema(rows, cols):
    # the reference declares both and ignores them (src/mx_cast.cu:168-171); here: transpose=True is the op on
    # input.t(), axis=0 puts the blocks down the columns, both together cancel up to the payload's view
    import driss_torch_b200 as dt

    a = workloads.make_cfg3(rows=rows, cols=cols)
    ad = a.cuda()
    want_p, want_s = qo.mx_fp8_quantize(a)
    want_pt, want_st = qo.mx_fp8_quantize(a.t().contiguous())
    p, s = dt.mx_fp8_quantize(ad, transpose=True)
    assert p.shape == (cols, rows) and p.is_contiguous()
    assert_fp8_equal(p, want_pt, E4M3, "transpose=True payload")
    assert torch.equal(as_bytes(s), as_bytes(want_st))
    p, s = dt.mx_fp8_quantize(ad, axis=0)
    assert p.shape == (rows, cols)
    assert_fp8_equal(p.t(), want_pt, E4M3, "axis=0 payload")
    assert torch.equal(as_bytes(s), as_bytes(want_st))
    p, s = dt.mx_fp8_quantize(ad, axis=0, transpose=True)
    assert p.shape == (cols, rows)
    assert_fp8_equal(p.t(), want_p, E4M3, "axis=0, transpose=True payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s))
    torch._dynamo.reset()
    fn = torch.compile(lambda t: dt.mx_fp8_quantize(t, axis=0), fullgraph=True, backend="aot_eager")
    q, qs = fn(ad)
    assert q.shape == (rows, cols) and q.stride() == (1, rows)
    assert_fp8_equal(q.t(), want_pt, E4M3, "compiled axis=0 payload")


# ---- scales in the blocked layout of the MX GEMM ------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 256), (384, 4096), (129, 256), (133, 512), (64, 96),
                                       (1, 32), (1000, 2080), (8192, 8192)])
def test_blocked_scales_are_the_row_major_scales_rearranged(rows, cols):
    import driss_torch_b200 as dt

    a = workloads.make_cfg3(rows=rows, cols=cols)
    p, s = dt.mx_fp8_quantize_blocked(a.cuda())
    want_p, want_s = qo.mx_fp8_quantize(a)
    assert_fp8_equal(p, want_p, E4M3, "payload")
    want_blocked = qo.to_blocked(want_s, rows, cols // 32)
    assert s.dtype == torch.float8_e8m0fnu and s.numel() == want_blocked.numel()
    assert torch.equal(as_bytes(s), want_blocked)


def test_blocked_layout_matches_the_cutlass_layout_function():
    # the index map the kernel uses, against CUTLASS's own tile_atom_to_shape_SFA evaluated on the
    # host by oracle/cute_sf_layout.cpp (built on demand from the CUTLASS headers vendored in the image)
    import subprocess
    import sysconfig
    from pathlib import Path

    import numpy as np

    from driss_torch_b200 import _cabi

    root = Path(__file__).resolve().parents[1]
    cutlass = Path(sysconfig.get_paths()["purelib"]) / "flashinfer" / "data" / "cutlass" / "include"
    if not (cutlass / "cutlass" / "detail" / "sm100_blockscaled_layout.hpp").exists():
        pytest.skip("no CUTLASS headers in this image")
    exe = root / "oracle" / "_build" / "cute_sf_layout"
    src = root / "oracle" / "cute_sf_layout.cpp"
    if not exe.exists() or exe.stat().st_mtime < src.stat().st_mtime:
        exe.parent.mkdir(exist_ok=True)
        subprocess.check_call(["g++", "-std=c++17", "-O1", f"-I{cutlass}", "-I/usr/local/cuda/include", str(src), "-o", str(exe)])
    for rows, cols in ((128, 128), (256, 1024), (133, 512), (384, 4096)):
        lines = subprocess.check_output([str(exe), str(rows), str(cols)], text=True).split("\n")
        cosize = int(lines[0].split()[1])
        table = np.array([[int(v) for v in ln.split()] for ln in lines[1:] if ln], dtype=np.int64)
        mine = qo.blocked_scale_offsets(rows, cols // 32)
        assert np.array_equal(mine[table[:, 0], table[:, 1]], table[:, 2]), (rows, cols)
        assert cosize <= _cabi.load().dtq_mx_blocked_scale_bytes(rows, cols)
        # and the kernel itself: scale (r, c) is found at that offset
        a = workloads.make_cfg3(rows=rows, cols=cols)
        _, s = _cabi.mx_fp8_quantize_blocked(a.cuda())
        _, row_major = qo.mx_fp8_quantize(a)
        got = as_bytes(s).numpy()[table[:, 2]]
        assert np.array_equal(got, row_major.view(torch.uint8).numpy()[table[:, 0] * (cols // 32) + table[:, 1]])


# ---- the shared-memory-staged (TMA bulk copy) variant ---------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 96), (128, 128), (77, 2048), (1000, 2080), (4096, 8192), (5, 4128)])
def test_tma_staged_variant_gives_the_same_bytes(rows, cols):
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg3(rows=rows, cols=cols)
    want_p, want_s = qo.mx_fp8_quantize(a)
    n = a.numel()
    pbuf = torch.full((n + 256,), 0x5A, dtype=torch.uint8, device="cuda")
    sbuf = torch.full((n // 32 + 256,), 0x5A, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        _cabi.mx_fp8_quantize_tma(a.cuda(), payload=pbuf[:n].view(E4M3).view(rows, cols),
                                  scales=sbuf[: n // 32].view(torch.float8_e8m0fnu), status=status)
    assert status.item() == 0
    assert_fp8_equal(pbuf[:n].view(E4M3).view(rows, cols), want_p, E4M3, "tma payload")
    assert torch.equal(sbuf[: n // 32].cpu(), as_bytes(want_s))
    assert (pbuf[n:] == 0x5A).all() and (sbuf[n // 32 :] == 0x5A).all()


def test_tma_staged_variant_on_patterns_and_degenerate_blocks():
    from driss_torch_b200 import _cabi

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    zeros = torch.zeros(128, 64)
    zeros[:, 32:] = 2.0**-121
    for a in (bits.view(64, 1024), zeros.to(torch.bfloat16)):
        want_p, want_s = qo.mx_fp8_quantize(a)
        p, s, status = _cabi.mx_fp8_quantize_tma(a.cuda())
        assert status.item() == 0
        assert_fp8_equal(p, want_p, E4M3, "tma payload")
        assert torch.equal(as_bytes(s), as_bytes(want_s))


# ---- both orientations from one read --------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(32, 32), (64, 256), (96, 288), (32, 8224), (1024, 512), (4096, 4096), (160, 96), (1184, 448), (2048, 32), (32, 2048)])
def test_dual_equals_cast_of_the_matrix_and_of_its_transpose(rows, cols):
    import driss_torch_b200 as dt

    a = workloads.make_cfg3(rows=rows, cols=cols)
    ad = a.cuda()
    p, s, p_t, s_t = dt.mx_fp8_quantize_dual(ad)
    assert p.shape == (rows, cols) and p_t.shape == (cols, rows)
    assert s.shape == (rows * cols // 32,) and s_t.shape == (cols * rows // 32,)
    want_p, want_s = qo.mx_fp8_quantize(a)
    want_pt, want_st = qo.mx_fp8_quantize(a.t().contiguous())
    assert_fp8_equal(p, want_p, E4M3, "payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s))
    assert_fp8_equal(p_t, want_pt, E4M3, "transposed payload")
    assert torch.equal(as_bytes(s_t), as_bytes(want_st))
    # and against the single-orientation op on the GPU
    q, qs = dt.mx_fp8_quantize(ad.t().contiguous())
    assert torch.equal(as_bytes(p_t), as_bytes(q)) and torch.equal(as_bytes(s_t), as_bytes(qs))


def test_dual_on_every_bf16_pattern_and_degenerate_blocks_and_errors():
    import driss_torch_b200 as dt

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    zeros = torch.zeros(128, 64)
    zeros[:, 32:] = 2.0**-121
    zeros[64:, :] = 0.0
    for a in (bits.view(256, 256), bits[torch.randperm(65536, generator=g)].view(64, 1024), zeros.to(torch.bfloat16)):
        p, s, p_t, s_t = dt.mx_fp8_quantize_dual(a.cuda())
        want_p, want_s = qo.mx_fp8_quantize(a)
        want_pt, want_st = qo.mx_fp8_quantize(a.t().contiguous())
        assert_fp8_equal(p, want_p, E4M3, "payload")
        assert_fp8_equal(p_t, want_pt, E4M3, "transposed payload")
        assert torch.equal(as_bytes(s), as_bytes(want_s)) and torch.equal(as_bytes(s_t), as_bytes(want_st))
    a = torch.zeros(48, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        dt.mx_fp8_quantize_dual(a)  # rows not a multiple of 32
    with pytest.raises(RuntimeError):
        dt.mx_fp8_quantize_dual(torch.zeros(64, 64, device="cuda"))  # not bf16


# ---- the other element formats and input types ----------------------------------------------------------

FORMATS = [torch.float8_e4m3fn, torch.float8_e5m2, "e2m1"]
MX_INPUTS = [torch.bfloat16, torch.float16, torch.float32]


def _mx_input(rows, cols, in_dtype, seed):
    g = torch.Generator().manual_seed(seed)
    mag = torch.exp(3.0 * torch.randn(rows, cols, generator=g))
    sign = torch.where(torch.rand(rows, cols, generator=g) < 0.5, -1.0, 1.0)
    x = torch.where(torch.rand(rows, cols, generator=g) < 0.01, torch.zeros(()), mag * sign)
    return x.to(in_dtype)


def _assert_payload(got, want, elem, what):
    if elem == "e2m1":
        assert got.dtype == torch.uint8 and torch.equal(got.cpu(), want), what
    else:
        assert_fp8_equal(got, want, elem, what)


@pytest.mark.parametrize("elem", FORMATS, ids=str)
@pytest.mark.parametrize("in_dtype", MX_INPUTS, ids=str)
@pytest.mark.parametrize("shape", [(128, 32), (8, 64), (256, 8192), (33, 96), (2048, 2048)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_mx_formats_against_the_oracle(shape, in_dtype, elem):
    from driss_torch_b200 import _cabi

    a = _mx_input(shape[0], shape[1], in_dtype, seed=shape[0] + 7 * shape[1])
    want_p, want_s = qo.mx_quantize(a, elem)
    p, s = _cabi.mx_quantize(a.cuda(), elem)
    _assert_payload(p, want_p, elem, "payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s)), "scales"


@pytest.mark.parametrize("elem", FORMATS, ids=str)
def test_mx_formats_on_every_16_bit_pattern_and_degenerate_blocks(elem):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(11)
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    shuffled = bits[torch.randperm(65536, generator=g)]
    for in_dtype in (torch.bfloat16, torch.float16):
        for b in (bits, shuffled):
            a = b.view(in_dtype).view(64, 1024)  # sorted: blocks of near-equal magnitude; shuffled: mixed blocks
            want_p, want_s = qo.mx_quantize(a, elem)
            p, s = _cabi.mx_quantize(a.cuda(), elem)
            _assert_payload(p, want_p, elem, f"{in_dtype} payload")
            assert torch.equal(as_bytes(s), as_bytes(want_s))
    # fp32: every exponent with a few mantissas, plus zero / subnormal / tiny / huge blocks
    exps = torch.arange(256, dtype=torch.int32).repeat_interleave(32)
    mant = torch.tensor([0, 1, 0x400000, 0x7FFFFF], dtype=torch.int32).repeat(2048)
    sign = (torch.arange(8192, dtype=torch.int32) % 3 == 0).to(torch.int32) << 31
    a = ((exps << 23) | mant | sign).view(torch.float32).view(64, 128)
    a2 = a.clone().view(-1)[torch.randperm(8192, generator=g)].view(64, 128)
    z = torch.zeros(32, 64)
    z[8:16] = 1e-38
    z[16:24, ::7] = 3e38
    for x in (a, a2, z):
        want_p, want_s = qo.mx_quantize(x.contiguous(), elem)
        p, s = _cabi.mx_quantize(x.contiguous().cuda(), elem)
        _assert_payload(p, want_p, elem, "fp32 payload")
        assert torch.equal(as_bytes(s), as_bytes(want_s))


def test_mx_formats_bf16_e4m3_is_the_reference_kernel_and_ops():
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg3(rows=512, cols=1024).cuda()
    p0, s0 = _cabi.mx_fp8_quantize(a)
    p1, s1 = _cabi.mx_quantize(a, E4M3)
    assert torch.equal(as_bytes(p0), as_bytes(p1)) and torch.equal(as_bytes(s0), as_bytes(s1))
    # the ops: e5m2 payload, fp32 / fp16 input, fp4
    p, s = dt.mx_fp8_quantize(a, ScalarType=torch.float8_e5m2)
    want_p, want_s = qo.mx_quantize(a.cpu(), torch.float8_e5m2)
    assert p.dtype == torch.float8_e5m2 and p.shape == a.shape
    assert_fp8_equal(p, want_p, torch.float8_e5m2, "e5m2 op")
    assert torch.equal(as_bytes(s), as_bytes(want_s))
    for in_dtype in (torch.float32, torch.float16):
        x = a.to(in_dtype)
        p, s = dt.mx_fp8_quantize(x)
        want_p, want_s = qo.mx_quantize(x.cpu(), E4M3)
        assert_fp8_equal(p, want_p, E4M3, f"{in_dtype} op")
        assert torch.equal(as_bytes(s), as_bytes(want_s))
    p4, s4 = dt.mx_fp4_quantize(a)
    want_p, want_s = qo.mx_quantize(a.cpu(), "e2m1")
    assert p4.dtype == torch.uint8 and p4.shape == (512, 512) and torch.equal(p4.cpu(), want_p)
    assert torch.equal(as_bytes(s4), as_bytes(want_s))
    # dequantised fp4 is within half a step of the block scale: |x - q| <= 2^(E-2) * 1 (largest step is 2)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])
    q = torch.stack([lut[(p4.cpu() & 0xF).long()], lut[(p4.cpu() >> 4).long()]], dim=-1).view(512, 1024)
    scale = torch.exp2(as_bytes(s4).cpu().float() - 127).view(512, 32, 1)
    err = (q.view(512, 32, 32) * scale - a.cpu().float().view(512, 32, 32)).abs()
    assert (err <= scale * 1.0 + 1e-30).all()


# ---- MX cast with the tensor's amax as a by-product ---------------------------------------------------------

@pytest.mark.parametrize("shape", [(128, 32), (33, 96), (1024, 4096), (4096, 8192), (1, 32)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_mx_with_amax_equals_mx_and_amax(shape):
    import driss_torch_b200 as dt

    a = workloads.make_cfg3(rows=shape[0], cols=shape[1])
    for _ in range(2):  # twice: the workspace must be left clean
        p, s, amax = dt.mx_fp8_quantize_with_amax(a.cuda())
        want_p, want_s = qo.mx_fp8_quantize(a)
        assert_fp8_equal(p, want_p, E4M3, "payload")
        assert torch.equal(as_bytes(s), as_bytes(want_s))
        assert amax.shape == (1,) and amax.dtype == torch.float32
        assert amax.item() == qo.amax(a).item() == dt.amax(a.cuda()).item()
    assert dt.amax(a.cuda()).item() == qo.amax(a).item()  # the plain amax kernel still finds the workspace clean


def test_mx_with_amax_drops_nans_and_handles_empty_and_all_nan():
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(4)
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    a = bits[torch.randperm(65536, generator=g)].view(torch.bfloat16).view(64, 1024)  # NaNs and infs in most chunks
    p, s, amax = dt.mx_fp8_quantize_with_amax(a.cuda())
    want_p, want_s = qo.mx_fp8_quantize(a)
    assert_fp8_equal(p, want_p, E4M3, "payload")
    assert torch.equal(as_bytes(s), as_bytes(want_s))
    assert amax.item() == float("inf") == qo.amax(a).item()
    b = a.clone()
    b[b.float().isinf()] = 3.0
    b[5, 77] = -7e30  # the largest finite magnitude sits in a chunk that also holds NaNs
    b[5, 78] = float("nan")
    _, _, amax = dt.mx_fp8_quantize_with_amax(b.cuda())
    assert amax.item() == qo.amax(b).item() and amax.item() >= 7e30 * 0.99
    nan = torch.full((32, 64), float("nan"), dtype=torch.bfloat16)
    _, _, amax = dt.mx_fp8_quantize_with_amax(nan.cuda())
    assert amax.item() == 0.0  # no non-NaN element: the fused op's starting value
    empty = torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda")
    p, s, amax = dt.mx_fp8_quantize_with_amax(empty)
    assert p.shape == (0, 64) and s.numel() == 0 and amax.item() == 0.0
    # a misaligned payload is refused rather than sent down a different kernel
    buf = torch.empty(64 * 64 + 8, dtype=torch.uint8, device="cuda")
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        _cabi.mx_fp8_quantize_amax(x, payload=buf[4:4 + 64 * 64].view(E4M3).view(64, 64))


@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 512), (96, 288), (1184, 448), (4096, 4096)])
def test_dual_with_blocked_scales(rows, cols):
    import driss_torch_b200 as dt

    a = workloads.make_cfg3(rows=rows, cols=cols)
    p, s, p_t, s_t = dt.mx_fp8_quantize_dual(a.cuda(), blocked=True)
    want_p, want_s = qo.mx_fp8_quantize(a)
    want_pt, want_st = qo.mx_fp8_quantize(a.t().contiguous())
    assert_fp8_equal(p, want_p, E4M3, "payload")
    assert_fp8_equal(p_t, want_pt, E4M3, "transposed payload")
    assert torch.equal(as_bytes(s).cpu(), as_bytes(qo.to_blocked(want_s, rows, cols // 32)))
    assert torch.equal(as_bytes(s_t).cpu(), as_bytes(qo.to_blocked(want_st, cols, rows // 32)))
    # and equal to the single-orientation blocked op on both orientations
    q, qs = dt.mx_fp8_quantize_blocked(a.cuda())
    qt, qts = dt.mx_fp8_quantize_blocked(a.t().contiguous().cuda())
    assert torch.equal(as_bytes(s), as_bytes(qs)) and torch.equal(as_bytes(s_t), as_bytes(qts))
