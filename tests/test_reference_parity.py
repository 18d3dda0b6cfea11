"""Bit-exact parity (GPU) of the product kernels AND of the CPU oracle with the unmodified
reference CUDA kernels (oracle/_ref, torch.ops.DrissTorchRef) on the same seeded inputs, on
the domain the reference supports.  Skipped when oracle/_ref has not been built."""
import pytest
import torch

from conftest import FP8_DTYPES, IN_DTYPES, as_bytes, assert_fp8_equal
from driss_torch_b200 import workloads
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu


def _rand(rows, cols, dtype, seed, randn=False):
    g = torch.Generator().manual_seed(seed)
    f = torch.randn if randn else torch.rand
    return f(rows, cols, generator=g).to(dtype)


@pytest.mark.parametrize("num_rows", [3, 64, 512, 4096])
@pytest.mark.parametrize("num_cols", [7, 17, 127, 512, 3212, 4097])
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_saturated_cast(ref_ops, num_rows, num_cols, in_dtype, fp8_dtype):
    import driss_torch_b200 as dt

    a = _rand(num_rows, num_cols, in_dtype, num_rows + num_cols).cuda()
    scale = workloads.tensor_scale(a, fp8_dtype)
    want = ref_ops.saturated_cast(a, scale, fp8_dtype, False)
    assert torch.equal(as_bytes(dt.saturated_cast(a, scale, fp8_dtype)), as_bytes(want))
    assert_fp8_equal(qo.saturated_cast(a.cpu(), scale.item(), fp8_dtype), want, fp8_dtype, "oracle vs reference")


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_saturated_cast_cfg1_and_all_patterns(ref_ops, fp8_dtype):
    import driss_torch_b200 as dt

    a = workloads.make_cfg1().cuda()
    scale = workloads.tensor_scale(a, fp8_dtype)
    assert torch.equal(as_bytes(dt.saturated_cast(a, scale, fp8_dtype)), as_bytes(ref_ops.saturated_cast(a, scale, fp8_dtype, False)))
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256).cuda()
    for s in (1.0, 0.3330078125, 85.84, 57344.0, 2.0**-120, 2.0**120):
        st = torch.tensor([s], device="cuda")
        # byte-exact including NaN inputs: both sides use the same conversion instruction
        assert torch.equal(as_bytes(dt.saturated_cast(bits, st, fp8_dtype)), as_bytes(ref_ops.saturated_cast(bits, st, fp8_dtype, False))), s


@pytest.mark.parametrize("num_rows", [4, 64, 512, 4096])
@pytest.mark.parametrize("num_cols", [8, 18, 128, 512, 3212, 4098])
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_amax(ref_ops, num_rows, num_cols, in_dtype):
    import driss_torch_b200 as dt

    a = _rand(num_rows, num_cols, in_dtype, num_rows * num_cols, randn=True).cuda()
    want = ref_ops.amax(a)
    assert dt.amax(a).view(torch.int32).item() == want.view(torch.int32).item()
    assert qo.amax(a.cpu()).view(torch.int32).item() == want.cpu().view(torch.int32).item()


def test_amax_cfg2(ref_ops):
    import driss_torch_b200 as dt

    a = workloads.make_cfg2(device="cuda")
    assert dt.amax(a).view(torch.int32).item() == ref_ops.amax(a).view(torch.int32).item()


@pytest.mark.parametrize("num_rows", [3, 64, 512, 4096])
@pytest.mark.parametrize("num_cols", [7, 17, 127, 512, 3212, 4097])
@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_dynamic_scaled_quant_fp32(ref_ops, num_rows, num_cols, fp8_dtype):
    import driss_torch_b200 as dt

    a = _rand(num_rows, num_cols, torch.float32, num_rows * 3 + num_cols).cuda()
    want = ref_ops.dynamic_scaled_quant(a, fp8_dtype)
    assert torch.equal(as_bytes(dt.dynamic_scaled_quant(a, fp8_dtype)), as_bytes(want))
    got, _, _ = qo.dynamic_scaled_quant(a.cpu(), fp8_dtype)
    assert_fp8_equal(got, want, fp8_dtype, "oracle vs reference")


@pytest.mark.parametrize("fp8_dtype", FP8_DTYPES)
def test_dynamic_scaled_quant_bf16_is_reference_on_float(ref_ops, fp8_dtype):
    # the reference instantiates fp32 only; bf16 input is defined as the same arithmetic on float(x)
    import driss_torch_b200 as dt

    a = workloads.make_cfg2(rows=4096, cols=8192, device="cuda")
    want = ref_ops.dynamic_scaled_quant(a.float(), fp8_dtype)
    assert torch.equal(as_bytes(dt.dynamic_scaled_quant(a, fp8_dtype)), as_bytes(want))
    p, am, sc = dt.dynamic_scaled_quant_with_scale(a, fp8_dtype)
    assert torch.equal(as_bytes(p), as_bytes(want))
    assert am.view(torch.int32).item() == ref_ops.amax(a).view(torch.int32).item()


@pytest.mark.parametrize("size", [(128, 32), (256, 32), (8192, 32), (128, 64), (128, 128), (128, 8192), (256, 64),
                                  (256, 128), (8192, 8192)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_mx(ref_ops, size):
    import driss_torch_b200 as dt

    a = _rand(size[0], size[1], torch.bfloat16, size[0] ^ size[1]).cuda()
    rp, rs = ref_ops.mx_fp8_quantize(a, 32, 1, False, torch.float8_e4m3fn)
    p, s = dt.mx_fp8_quantize(a)
    assert torch.equal(as_bytes(p), as_bytes(rp)) and torch.equal(as_bytes(s), as_bytes(rs))
    op, os_ = qo.mx_fp8_quantize(a.cpu())
    assert_fp8_equal(op, rp, torch.float8_e4m3fn, "oracle payload vs reference")
    assert torch.equal(as_bytes(os_), as_bytes(rs))


def test_mx_wide_range_patterns_and_degenerate_blocks(ref_ops):
    import driss_torch_b200 as dt

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    g = torch.Generator().manual_seed(9)
    zeros = torch.zeros(128, 64)
    zeros[:, 32:] = 2.0**-121
    for a in (workloads.make_cfg3(rows=2048, cols=8192), bits.view(128, 512), bits[torch.randperm(65536, generator=g)].view(128, 512),
              zeros.to(torch.bfloat16)):
        a = a.cuda()
        rp, rs = ref_ops.mx_fp8_quantize(a, 32, 1, False, torch.float8_e4m3fn)
        p, s = dt.mx_fp8_quantize(a)
        assert torch.equal(as_bytes(p), as_bytes(rp)) and torch.equal(as_bytes(s), as_bytes(rs))


# test/test_mx.py:41-57 (M, K, N), and the benchmark's shapes
GEMM_SIZES = [(128, 128, 128), (256, 256, 256), (384, 384, 384), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024),
              (128, 256, 384), (256, 384, 512), (129, 256, 384), (133, 512, 528), (4096, 4096, 4096), (2048, 1024, 8192)]


@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow", "auto"])
@pytest.mark.parametrize("size", GEMM_SIZES, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_mx_fp8_bf16_equals_the_reference_kernel_bit_for_bit(ref_gemm_ops, size, kernel):
    # Same operands through the reference's CUTLASS kernel and through each of ours: fp32 accumulation over K in the
    # same order (128 at a time, 32 per instruction), one rounding to bf16 -- the results are the same bits, on
    # random data, not only on exactly summable inputs.
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    m, k, n = size
    g = torch.Generator(device="cuda").manual_seed(m * 7 + k * 3 + n)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", generator=g) * 0.25).to(torch.bfloat16)
    pa, sa = dt.mx_fp8_quantize_blocked(a)
    pb, sb = dt.mx_fp8_quantize_blocked(b)
    want = ref_gemm_ops.mx_fp8_bf16(pa, pb.t(), sa, sb)
    got = _cabi.mx_fp8_bf16(pa, pb, sa, sb, kernel=kernel)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
        f"{(got.view(torch.int16) != want.view(torch.int16)).sum().item()} of {got.numel()} outputs differ"


@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow"])
@pytest.mark.parametrize("size", [(128, 128, 128), (512, 512, 512), (129, 256, 384), (133, 512, 528), (2048, 2048, 2048)],
                         ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_mx_fp4_bf16_equals_the_reference_kernel_bit_for_bit(ref_gemm_ops, size, kernel):
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    m, k, n = size
    g = torch.Generator(device="cuda").manual_seed(m + k + n)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda", generator=g).to(torch.bfloat16)
    pa, sa = dt.mx_fp4_quantize(a, blocked=True)
    pb, sb = dt.mx_fp4_quantize(b, blocked=True)
    want = ref_gemm_ops.mx_fp4_bf16(pa, pb.t(), sa, sb)
    got = _cabi.mx_fp8_bf16(pa, pb, sa, sb, kernel=kernel, fp4=True)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow"])
def test_mx_fp8_bf16_special_values_equal_the_reference_kernel(ref_gemm_ops, kernel):
    # Every e4m3 byte pattern as an operand (the two NaN encodings included) and every E8M0 scale byte (0 = 2^-127 and
    # 255 = NaN included), at random positions: the same tensor-core instructions see the same inputs in both kernels,
    # so the outputs -- infinities, NaNs and their bf16 encodings included -- are the same bits.
    from driss_torch_b200 import _cabi

    m, n, k = 256, 512, 512
    g = torch.Generator().manual_seed(99)
    a = torch.randint(0, 256, (m, k), generator=g, dtype=torch.int32).to(torch.uint8)
    b = torch.randint(0, 256, (n, k), generator=g, dtype=torch.int32).to(torch.uint8)
    # keep most rows free of NaN operands so that finite results are compared too
    a[16:] = torch.where((a[16:] & 0x7F) == 0x7F, torch.zeros_like(a[16:]), a[16:])
    b[16:] = torch.where((b[16:] & 0x7F) == 0x7F, torch.zeros_like(b[16:]), b[16:])
    sa = torch.randint(110, 140, (m, k // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    sb = torch.randint(110, 140, (n, k // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    sa[3, 2], sa[40, 0], sb[5, 1], sb[77, 3] = 255, 0, 255, 0
    sab = qo.to_blocked(sa, m, k // 32).cuda().view(torch.float8_e8m0fnu)
    sbb = qo.to_blocked(sb, n, k // 32).cuda().view(torch.float8_e8m0fnu)
    ad, bd = a.cuda().view(torch.float8_e4m3fn), b.cuda().view(torch.float8_e4m3fn)
    want = ref_gemm_ops.mx_fp8_bf16(ad, bd.t(), sab, sbb)
    got = _cabi.mx_fp8_bf16(ad, bd, sab, sbb, kernel=kernel)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
        f"{(got.view(torch.int16) != want.view(torch.int16)).sum().item()} of {got.numel()} outputs differ"
    assert got.float().isnan().any() and got.float().isfinite().any()
