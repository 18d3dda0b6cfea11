"""mx_fp8_bf16: the MX block-scaled GEMM that consumes the MX casts.

CPU part: the oracle's restatement (oracle_mx_gemm_bf16) against an independent evaluation with
PyTorch CPU ops, its e4m3 / e8m0 decoders against PyTorch's casts, its blocked-scale indexing.
GPU part, modelled on the reference's test (test/test_mx.py:9-67): operands from the MX casts,
result against a bf16 matmul of the dequantised operands with the reference's own bar (SQNR above
80 dB) on the reference's size grid; and, because a tensor-core accumulation order cannot be
restated on a CPU, byte-exact equality with the oracle on inputs whose partial sums are all exactly
representable (small integers times powers of two), including shapes that are not multiples of the
tile and of the scale atoms.
"""
import pytest
import torch

from conftest import as_bytes
from oracle import quant_oracle as qo

E4M3 = torch.float8_e4m3fn
E8M0 = torch.float8_e8m0fnu

# test/test_mx.py:41-57 (M, K, N)
REFERENCE_SIZES = [(128, 128, 128), (256, 256, 256), (384, 384, 384), (512, 512, 512), (768, 768, 768),
                   (1024, 1024, 1024), (8192, 8192, 8192), (128, 256, 384), (256, 384, 512), (129, 256, 384),
                   (133, 512, 528)]


def _dequant(payload, scales_row_major, rows, k):
    s = torch.exp2(scales_row_major.view(torch.uint8).float() - 127.0).view(rows, k // 32, 1)
    return (payload.float().view(rows, k // 32, 32) * s).view(rows, k)


def _sqnr(want, got):
    # torchao.float8.float8_utils.compute_error as the reference's test uses it: 20 log10(|x| / |x - y|)
    err = (want.float() - got.float()).norm()
    return float("inf") if err == 0 else float(20 * torch.log10(want.float().norm() / err))


def _small_int_operands(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-3, 4, (m, k), generator=g).float().to(E4M3)
    b = torch.randint(-3, 4, (n, k), generator=g).float().to(E4M3)
    sa = torch.randint(125, 130, (m, k // 32), generator=g).to(torch.uint8)
    sb = torch.randint(125, 130, (n, k // 32), generator=g).to(torch.uint8)
    return a, b, sa, sb


_ORACLE_CACHE = {}


def _oracle_cached(a, b, sab, sbb, key):
    if key not in _ORACLE_CACHE:
        _ORACLE_CACHE[key] = qo.mx_gemm_bf16(a, b, sab, sbb)
    return _ORACLE_CACHE[key]


# ---- CPU: the oracle itself ----------------------------------------------------------------------------

def test_oracle_decoders_match_pytorch_casts():
    every = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    every[0x7F] = 0  # the two NaN encodings would poison every sum (NaN x 0); checked on their own below
    every[0xFF] = 0
    a = every.view(E4M3).view(1, 256).repeat(8, 1)  # [8, 256]: every finite e4m3 byte as an A row
    ident = torch.zeros(256, 256)
    ident.fill_diagonal_(1.0)
    one_scales = torch.full((256 * 8,), 127, dtype=torch.uint8)
    sa = qo.to_blocked(one_scales[: 8 * 8], 8, 8)
    sb = qo.to_blocked(one_scales, 256, 8)
    out = qo.mx_gemm_bf16(a, ident.to(E4M3), sa, sb)  # picks out each element: bf16(e4m3 value), exact
    assert torch.equal(out[0].float(), every.view(E4M3).float())
    nan_row = torch.zeros(1, 32, dtype=torch.uint8)
    nan_row[0, 5] = 0x7F
    s1 = qo.to_blocked(torch.full((1,), 127, dtype=torch.uint8), 1, 1)
    assert qo.mx_gemm_bf16(nan_row.view(E4M3), torch.ones(1, 32).to(E4M3), s1, s1).float().isnan().all()
    # e8m0: 2^(b - 127); a single 1.0 x 1.0 product per output scaled by sa only
    for byte in (0, 1, 100, 127, 128, 200, 254):
        s = torch.full((4,), byte, dtype=torch.uint8)
        x = torch.zeros(1, 128)
        x[0, 0] = 1.0
        o = qo.mx_gemm_bf16(x.to(E4M3), x.to(E4M3), qo.to_blocked(s, 1, 4), qo.to_blocked(torch.full((4,), 127, dtype=torch.uint8), 1, 4))
        assert o.float().item() == 2.0 ** (byte - 127) or (byte < 127 - 126 - 7 and o.float().item() == 0.0)


@pytest.mark.parametrize("m,n,k", [(8, 16, 32), (33, 40, 96), (130, 136, 160), (64, 48, 512)])
def test_oracle_against_an_independent_evaluation(m, n, k):
    g = torch.Generator().manual_seed(m * 1000 + n)
    a = (torch.randn(m, k, generator=g) * 3).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16)
    pa, sa = qo.mx_fp8_quantize(a)
    pb, sb = qo.mx_fp8_quantize(b)
    out = qo.mx_gemm_bf16(pa, pb, qo.to_blocked(sa, m, k // 32), qo.to_blocked(sb, n, k // 32))
    want = (_dequant(pa, sa, m, k).double() @ _dequant(pb, sb, n, k).double().t()).to(torch.bfloat16)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


# ---- GPU ----------------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("size", REFERENCE_SIZES, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_reference_size_grid_sqnr(size):
    import driss_torch_b200 as dt

    m, k, n = size
    a = torch.rand(m, k, device="cuda").to(torch.bfloat16)
    b = torch.rand(n, k, device="cuda").to(torch.bfloat16)
    a_data, a_scale = dt.mx_fp8_quantize_blocked(a)
    b_data, b_scale = dt.mx_fp8_quantize_blocked(b)
    out = dt.mx_fp8_bf16(a_data, b_data.t(), a_scale, b_scale)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    pa, sa = dt.mx_fp8_quantize(a)
    pb, sb = dt.mx_fp8_quantize(b)
    out_hp = _dequant(pa, sa, m, k).to(torch.bfloat16) @ _dequant(pb, sb, n, k).to(torch.bfloat16).t()
    assert _sqnr(out_hp, out) > 80, f"SQNR {_sqnr(out_hp, out)} dB"
    dt.check_device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 128, 128), (256, 512, 512), (129, 256, 384), (133, 528, 512),
                                   (384, 384, 384), (64, 8, 32), (300, 520, 96), (1, 8, 64), (1024, 1024, 1024),
                                   (2560, 4096, 256),    # several rounds of tiles per SM: accumulator and stage reuse
                                   (18944, 504, 128),    # many tile rows, a ragged last tile column
                                   (9472, 376, 160)])    # a last tile column whose second scale atom does not exist
def test_exact_against_the_oracle_on_exactly_summable_inputs(m, n, k, kernel):
    # every kernel (an SM pair per 256 x 256 tile; one CTA per 128 x 256 or per 128 x 128 tile) on every size
    from driss_torch_b200 import _cabi

    a, b, sa, sb = _small_int_operands(m, n, k, seed=m + n + k)
    sab, sbb = qo.to_blocked(sa, m, k // 32), qo.to_blocked(sb, n, k // 32)
    want = _oracle_cached(a, b, sab, sbb, (m, n, k))
    out = _cabi.mx_fp8_bf16(a.cuda(), b.cuda(), sab.cuda(), sbb.cuda(), kernel=kernel)
    got = out.cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
        f"{(got.view(torch.int16) != want.view(torch.int16)).sum().item()} of {got.numel()} outputs differ"
    assert _cabi.workspace_status(_cabi.workspace(torch.device("cuda", torch.cuda.current_device()))) == 0


@pytest.mark.gpu
def test_every_scale_position_is_used_where_it_belongs():
    # all data 1.0: out[m, n] = 32 * sum_kb 2^(sa[m,kb] + sb[n,kb] - 254); one k-block at a time carries a
    # row-dependent exponent, so a scale read from the wrong row, quadrant or k-block changes the result
    from driss_torch_b200 import _cabi

    m, n, k = 256, 512, 256
    ones_a = torch.ones(m, k).to(E4M3)
    ones_b = torch.ones(n, k).to(E4M3)
    for kb in range(k // 32):
        sa = torch.full((m, k // 32), 97, dtype=torch.uint8)
        sb = torch.full((n, k // 32), 97, dtype=torch.uint8)
        sa[:, kb] = (120 + torch.arange(m) % 13).to(torch.uint8)
        sb[:, kb] = (122 + torch.arange(n) % 11).to(torch.uint8)
        sab, sbb = qo.to_blocked(sa, m, k // 32), qo.to_blocked(sb, n, k // 32)
        want = qo.mx_gemm_bf16(ones_a, ones_b, sab, sbb)
        for kernel in ("pair", "wide", "narrow"):
            out = _cabi.mx_fp8_bf16(ones_a.cuda(), ones_b.cuda(), sab.cuda(), sbb.cuda(), kernel=kernel).cpu()
            assert torch.equal(out.view(torch.int16), want.view(torch.int16)), f"k-block {kb}, {kernel} kernel"


@pytest.mark.gpu
def test_operator_checks_fake_and_repeatability():
    import driss_torch_b200 as dt

    a = torch.rand(256, 512, device="cuda").to(torch.bfloat16)
    b = torch.rand(384, 512, device="cuda").to(torch.bfloat16)
    pa, sa = dt.mx_fp8_quantize_blocked(a)
    pb, sb = dt.mx_fp8_quantize_blocked(b)
    out = dt.mx_fp8_bf16(pa, pb.t(), sa, sb)
    for _ in range(3):  # the accumulation order is fixed: bit-identical from run to run
        assert torch.equal(as_bytes(dt.mx_fp8_bf16(pa, pb.t(), sa, sb).view(torch.int16)), as_bytes(out.view(torch.int16)))
    for bad in (
        lambda: dt.mx_fp8_bf16(pa, pb, sa, sb),                      # b must be the column-major [K, N] view
        lambda: dt.mx_fp8_bf16(pa, pb.t(), sa[:-1], sb),             # scale sizes as the reference's validate()
        lambda: dt.mx_fp8_bf16(pa, pb.t(), sa, sb[:-512]),
        lambda: dt.mx_fp8_bf16(pa.view(torch.uint8), pb.t(), sa, sb),
        lambda: dt.mx_fp8_bf16(pa[:, :96], pb.t(), sa, sb),
        lambda: dt.mx_fp8_bf16(pa, pb[:380].t(), sa, sb),            # N % 8
    ):
        with pytest.raises(RuntimeError):
            bad()
    with pytest.raises(NotImplementedError):
        dt.mx_fp8_bf16(pa.cpu(), pb.cpu().t(), sa.cpu(), sb.cpu())  # CUDA only
    torch._dynamo.reset()
    fn = torch.compile(dt.mx_fp8_bf16, fullgraph=True, backend="aot_eager")
    assert torch.equal(as_bytes(fn(pa, pb.t(), sa, sb).view(torch.int16)), as_bytes(out.view(torch.int16)))
    import driss_torch

    assert driss_torch.mx_fp8_bf16 is dt.mx_fp8_bf16
    dt.check_device_status()


# ---- MXFP4 (e2m1 packed two per byte): mx_fp4_bf16 -----------------------------------------------------------------

def test_oracle_fp4_against_an_independent_evaluation():
    g = torch.Generator().manual_seed(44)
    m, n, k = 40, 24, 192
    a = torch.randint(0, 256, (m, k // 2), generator=g).to(torch.uint8)
    b = torch.randint(0, 256, (n, k // 2), generator=g).to(torch.uint8)
    sa = torch.randint(120, 134, (m, k // 32), generator=g).to(torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), generator=g).to(torch.uint8)
    out = qo.mx_gemm_bf16(a, b, qo.to_blocked(sa, m, k // 32), qo.to_blocked(sb, n, k // 32), fp4=True)
    table = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=torch.float64)

    def unpack(p, s, rows):
        lo, hi = table[(p & 0xF).long()], table[(p >> 4).long()]
        vals = torch.stack([lo, hi], dim=-1).view(rows, k)  # the lower index in the low nibble
        return (vals.view(rows, k // 32, 32) * torch.exp2(s.double() - 127).view(rows, k // 32, 1)).view(rows, k)

    want = (unpack(a, sa, m) @ unpack(b, sb, n).t()).to(torch.bfloat16)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 128, 128), (256, 512, 1024), (129, 256, 384), (133, 528, 512),
                                   (64, 8, 32), (300, 520, 96), (1024, 1024, 1024), (2560, 2048, 512), (9472, 376, 320)])
def test_fp4_exact_against_the_oracle(m, n, k, kernel):
    # every product of two e2m1 values is a multiple of 1/4 below 64 and the scales span a few binades, so all
    # partial sums are exact in fp32 and the device must agree with the oracle bit for bit; K = 128, 384, 96, 320
    # leave the second scale atom of a 256-element stage partly or wholly outside the matrix
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randint(0, 256, (m, k // 2), generator=g).to(torch.uint8)
    b = torch.randint(0, 256, (n, k // 2), generator=g).to(torch.uint8)
    sa = torch.randint(125, 130, (m, k // 32), generator=g).to(torch.uint8)
    sb = torch.randint(125, 130, (n, k // 32), generator=g).to(torch.uint8)
    sab, sbb = qo.to_blocked(sa, m, k // 32), qo.to_blocked(sb, n, k // 32)
    key = ("fp4", m, n, k)
    if key not in _ORACLE_CACHE:
        _ORACLE_CACHE[key] = qo.mx_gemm_bf16(a, b, sab, sbb, fp4=True)
    want = _ORACLE_CACHE[key]
    got = _cabi.mx_fp4_bf16(a.cuda(), b.cuda(), sab.cuda(), sbb.cuda(), kernel=kernel).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
        f"{(got.view(torch.int16) != want.view(torch.int16)).sum().item()} of {got.numel()} outputs differ"
    assert _cabi.workspace_status(_cabi.workspace(torch.device("cuda", torch.cuda.current_device()))) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("size", REFERENCE_SIZES, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_fp4_reference_size_grid_sqnr(size):
    # test/test_mx.py:36-67 with format "fp4": operands from the MXFP4 cast (scales straight in the blocked layout),
    # result against a bf16 matmul of the dequantised operands, SQNR above 80 dB
    import driss_torch_b200 as dt

    m, k, n = size
    a = torch.rand(m, k, device="cuda").to(torch.bfloat16)
    b = torch.rand(n, k, device="cuda").to(torch.bfloat16)
    a_data, a_scale = dt.mx_fp4_quantize(a, blocked=True)
    b_data, b_scale = dt.mx_fp4_quantize(b, blocked=True)
    out = dt.mx_fp4_bf16(a_data, b_data.t(), a_scale, b_scale)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    table = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], device="cuda")

    def dequant(x, rows):
        p, s = dt.mx_fp4_quantize(x)
        vals = torch.stack([table[(p & 0xF).long()], table[(p >> 4).long()]], dim=-1).view(rows, k)
        return (vals.view(rows, k // 32, 32) * torch.exp2(s.view(torch.uint8).float() - 127).view(rows, k // 32, 1)).view(rows, k)

    out_hp = dequant(a, m).to(torch.bfloat16) @ dequant(b, n).to(torch.bfloat16).t()
    assert _sqnr(out_hp, out) > 80, f"SQNR {_sqnr(out_hp, out)} dB"
    # the blocked scales are the row-major ones rearranged
    _, s_rm = dt.mx_fp4_quantize(a)
    assert torch.equal(as_bytes(a_scale), qo.to_blocked(s_rm.cpu(), m, k // 32))
    dt.check_device_status()
