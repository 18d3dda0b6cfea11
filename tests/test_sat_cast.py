"""saturated_cast parity (GPU): the CUDA kernel through the C ABI and through the
torch.ops.DrissTorch op against the CPU oracle, on the reference test's shape grid
(test/test_sat_cast.py:27-42), plus exhaustive and edge cases the oracle enumerates."""
import pytest
import torch

from conftest import FP8_DTYPES, IN_DTYPES, assert_fp8_equal
from driss_torch_b200 import workloads
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu

ROWS = [3, 64, 512, 4096]
COLS = [7, 17, 127, 512, 3212, 4097]


def _input(rows, cols, in_dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(rows, cols, generator=g, dtype=torch.float32).to(in_dtype)


@pytest.mark.parametrize("num_rows", ROWS)
@pytest.mark.parametrize("num_cols", COLS)
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_cast(num_rows, num_cols, in_dtype, fp8_dtype):
    from driss_torch_b200 import _cabi

    a = _input(num_rows, num_cols, in_dtype, seed=num_rows * 10007 + num_cols)
    scale = workloads.tensor_scale(a, fp8_dtype)
    want = qo.saturated_cast(a, scale.item(), fp8_dtype)
    got = _cabi.saturated_cast(a.cuda(), scale.cuda(), fp8_dtype)
    assert_fp8_equal(got, want, fp8_dtype, "C ABI")


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_op_matches_oracle_and_keeps_layout(in_dtype, fp8_dtype):
    import driss_torch_b200 as dt

    a = _input(512, 384, in_dtype, seed=5).cuda()
    scale = workloads.tensor_scale(a, fp8_dtype)
    out = dt.saturated_cast(a, scale, fp8_dtype)
    assert out.dtype == fp8_dtype and out.shape == a.shape and out.stride() == a.stride()
    assert_fp8_equal(out, qo.saturated_cast(a.cpu(), scale.item(), fp8_dtype), fp8_dtype, "op")
    # 0-dim scale, as a tensor_to_scale-style helper returns it
    out0 = dt.saturated_cast(a, scale.reshape(()), fp8_dtype)
    assert_fp8_equal(out0, out, fp8_dtype, "0-dim scale")
    # exactly transposed input: processed over storage, output keeps the transposed strides
    at = a.t()
    out_t = dt.saturated_cast(at, scale, fp8_dtype)
    assert out_t.shape == at.shape and out_t.stride() == at.stride()
    assert_fp8_equal(out_t.contiguous(), qo.saturated_cast(at.cpu().contiguous(), scale.item(), fp8_dtype), fp8_dtype,
                     "transposed")
    # a view at a storage offset is made contiguous first
    sl = a[3:, 8:]
    out_s = dt.saturated_cast(sl, scale, fp8_dtype)
    assert out_s.is_contiguous()
    assert_fp8_equal(out_s, qo.saturated_cast(sl.cpu().contiguous(), scale.item(), fp8_dtype), fp8_dtype, "slice")


def test_known_answer_vector():
    # test/test_sat_cast.py:65-83: the kernel's answer is 16384.0, not eager's 20480.0
    import driss_torch_b200 as dt

    a = torch.tensor([0.3223, 0.3223], dtype=torch.float32).to(device="cuda", dtype=torch.bfloat16).view(2, 1)
    scale = torch.tensor([57344.0], device="cuda")
    out = dt.saturated_cast(a, scale, torch.float8_e5m2)
    assert out.float().flatten().tolist() == [16384.0, 16384.0]


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("scale", [1.0, 0.3330078125, 448.0 / 5.21875, 57344.0, 3.0e-5, 2.0**-120, 2.0**120, 0.0,
                                   float("inf")])
def test_every_bf16_bit_pattern(fp8_dtype, scale):
    from driss_torch_b200 import _cabi

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    a = bits.view(torch.bfloat16).view(256, 256)
    s = torch.tensor([scale], dtype=torch.float32)
    want = qo.saturated_cast(a, s.item(), fp8_dtype)
    got = _cabi.saturated_cast(a.cuda(), s.cuda(), fp8_dtype)
    assert_fp8_equal(got, want, fp8_dtype, f"scale={scale}")


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_fp32_specials_midpoints_and_saturation(fp8_dtype):
    from driss_torch_b200 import _cabi

    fmax = torch.finfo(fp8_dtype).max
    g = torch.Generator().manual_seed(11)
    pieces = [
        torch.linspace(-1.25 * fmax, 1.25 * fmax, 200_001),
        torch.linspace(-0.05, 0.05, 100_001),
        torch.randint(-(2**31), 2**31 - 1, (300_000,), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32),
        torch.tensor([0.0, -0.0, float("inf"), -float("inf"), float("nan"), fmax, -fmax, 1e-45, -1e-45]),
    ]
    a = torch.cat(pieces)
    a = a[: a.numel() // 2 * 2].view(2, -1).contiguous()
    for scale in (1.0, 0.75):
        s = torch.tensor([scale])
        want = qo.saturated_cast(a, scale, fp8_dtype)
        got = _cabi.saturated_cast(a.cuda(), s.cuda(), fp8_dtype)
        assert_fp8_equal(got, want, fp8_dtype, f"fp32 scale={scale}")


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
@pytest.mark.parametrize("numel", [0, 1, 2, 7, 8, 9, 15, 31, 1023, 1025, 4099, 262147])
def test_ragged_sizes_and_unwritten_bytes(in_dtype, numel):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(numel + 1)
    a = torch.randn(1, numel, generator=g).to(in_dtype)
    s = torch.tensor([3.5])
    want = qo.saturated_cast(a, 3.5, torch.float8_e4m3fn)
    # poisoned, oversized output: every byte inside must be written, none outside
    buf = torch.full((numel + 64,), 0x5A, dtype=torch.uint8, device="cuda")
    out = buf[:numel].view(torch.float8_e4m3fn).view(1, numel)
    _cabi.saturated_cast(a.cuda(), s.cuda(), torch.float8_e4m3fn, out=out)
    assert_fp8_equal(out, want, torch.float8_e4m3fn, f"numel={numel}")
    assert (buf[numel:] == 0x5A).all()


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
@pytest.mark.parametrize("offset", [1, 3, 5])
def test_misaligned_pointers_take_the_scalar_path(in_dtype, offset):
    from driss_torch_b200 import _cabi

    n = 10_000
    g = torch.Generator().manual_seed(offset)
    base = torch.randn(n + 16, generator=g).to(in_dtype).cuda()
    a = base[offset : offset + n].view(1, n)  # element offset -> not 16-byte aligned
    s = torch.tensor([2.25], device="cuda")
    buf = torch.zeros(n + 16, dtype=torch.uint8, device="cuda")
    out = buf[offset : offset + n].view(torch.float8_e5m2).view(1, n)
    _cabi.saturated_cast(a, s, torch.float8_e5m2, out=out)
    assert_fp8_equal(out, qo.saturated_cast(a.cpu().contiguous(), 2.25, torch.float8_e5m2), torch.float8_e5m2, "misaligned")


def test_argument_errors():
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    a = torch.zeros(4, 4, dtype=torch.bfloat16, device="cuda")
    s = torch.ones(1, device="cuda")
    with pytest.raises(RuntimeError):
        dt.saturated_cast(a, s, torch.float16)
    with pytest.raises(RuntimeError):
        dt.saturated_cast(a.half(), s, torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):
        dt.saturated_cast(a, torch.ones(2, device="cuda"), torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):
        dt.saturated_cast(a, s.double(), torch.float8_e4m3fn)
    with pytest.raises(RuntimeError):
        dt.saturated_cast(a.view(16), s, torch.float8_e4m3fn)
    with pytest.raises(AssertionError):
        dt.saturated_cast(a, s, torch.float8_e4m3fn, transpose=True)
    with pytest.raises(NotImplementedError):
        dt.saturated_cast(a.cpu(), s.cpu(), torch.float8_e4m3fn)  # CUDA only: no CPU kernel
    L = _cabi.load()
    assert L.dtq_saturated_cast(None, None, None, 4, 0, 0, None) == 1
    assert L.dtq_saturated_cast(a.data_ptr(), a.data_ptr(), s.data_ptr(), 4, 7, 0, None) == 2


def test_compile_fullgraph_uses_fake_impl():
    # test/test_sat_cast.py:45-62: the op must trace under torch.compile(fullgraph=True)
    import driss_torch_b200 as dt

    torch._dynamo.reset()
    a = torch.rand(64, 127, device="cuda").to(torch.bfloat16)
    s = workloads.tensor_scale(a, torch.float8_e4m3fn)
    for backend in ("aot_eager", "inductor"):  # the reference compiles with the default backend
        torch._dynamo.reset()
        fn = torch.compile(dt.saturated_cast, fullgraph=True, backend=backend)
        assert_fp8_equal(fn(a, s, torch.float8_e4m3fn), dt.saturated_cast(a, s, torch.float8_e4m3fn))


def test_transpose_argument_of_the_operator():
    # the wrapper keeps the reference's assert (driss_torch/__init__.py:37); the operator's own flag, which the
    # reference only uses to choose a kernel (src/saturated_cast.cu:168-181), gives the cast of input.t()
    import driss_torch_b200 as dt

    a = workloads.make_cfg1(rows=160, cols=96)
    for fp8_dtype in FP8_DTYPES:
        s = workloads.tensor_scale(a, fp8_dtype)
        want = qo.saturated_cast(a, s.item(), fp8_dtype)
        got = torch.ops.DrissTorch.saturated_cast(a.cuda(), s.cuda(), fp8_dtype, True)
        assert got.shape == (96, 160) and got.is_contiguous()
        assert_fp8_equal(got, want.t().contiguous(), fp8_dtype, "transpose=True")


# ---- transposed output / both orientations from one read -----------------------------------------------

T_SHAPES = [(128, 128), (256, 64), (16, 8), (48, 200), (144, 1032), (4096, 512), (1040, 4104),  # tiled path
            (3, 7), (64, 17), (33, 512), (512, 4097), (1, 1), (100, 36)]                         # byte-tile path


@pytest.mark.parametrize("shape", T_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_transposed_and_dual_outputs(shape, in_dtype, fp8_dtype):
    import driss_torch_b200 as dt

    a = _input(shape[0], shape[1], in_dtype, seed=shape[0] * 31 + shape[1])
    scale = workloads.tensor_scale(a, fp8_dtype)
    a[0, 0] = float("inf")  # saturates
    a[-1, -1] = -1e30       # saturates
    a[shape[0] // 2, shape[1] // 2] = float("nan")
    want = qo.saturated_cast(a, scale.item(), fp8_dtype)
    ad, sd = a.cuda(), scale.cuda()
    out_t = dt.saturated_cast_transposed(ad, sd, fp8_dtype)
    assert out_t.shape == (shape[1], shape[0]) and out_t.is_contiguous() and out_t.dtype == fp8_dtype
    assert_fp8_equal(out_t, want.t().contiguous(), fp8_dtype, "transposed")
    out, out_t2 = dt.saturated_cast_dual(ad, sd, fp8_dtype)
    assert out.shape == tuple(shape) and out.is_contiguous()
    assert_fp8_equal(out, want, fp8_dtype, "dual: row-major")
    assert_fp8_equal(out_t2, want.t().contiguous(), fp8_dtype, "dual: transposed")
    # a non-contiguous input is made contiguous first
    out_v = dt.saturated_cast_transposed(ad.t(), sd, fp8_dtype)
    assert_fp8_equal(out_v, want, fp8_dtype, "transposed view in")


def test_transposed_on_every_bf16_pattern():
    import driss_torch_b200 as dt

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256)
    for fp8_dtype in FP8_DTYPES:
        for s in (1.0, 0.37, 448.0):
            scale = torch.tensor([s])
            want = qo.saturated_cast(bits, s, fp8_dtype)
            out, out_t = dt.saturated_cast_dual(bits.cuda(), scale.cuda(), fp8_dtype)
            assert_fp8_equal(out, want, fp8_dtype, "row-major")
            assert_fp8_equal(out_t, want.t().contiguous(), fp8_dtype, "transposed")
