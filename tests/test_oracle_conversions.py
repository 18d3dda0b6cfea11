"""Pins the plain-C oracle's number-format conversions (CPU only).

* the one known-answer vector of the reference's tests (test/test_sat_cast.py:65-83);
* every bf16 bit pattern and a wide fp32 sweep against the CUDA toolkit's host-callable
  conversion helpers -- the functions the reference kernels call on the device;
* PyTorch's CPU fp8 casts as a third opinion.
"""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo

KINDS = [(qo.E4M3, torch.float8_e4m3fn, 448.0), (qo.E5M2, torch.float8_e5m2, 57344.0)]


def all_bf16_bits():
    return np.arange(65536, dtype=np.uint32).astype(np.uint16)


def bf16_bits_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def fp32_sweep():
    """All bf16 values, fp8 midpoints and their fp32 neighbours, plus random bit patterns."""
    rng = np.random.default_rng(7)
    base = bf16_bits_to_f32(all_bf16_bits())
    rand = rng.integers(0, 2**32, size=2_000_000, dtype=np.uint32).view(np.float32)
    fine = np.concatenate([np.linspace(-500, 500, 400_001), np.linspace(-60000, 60000, 400_001),
                           np.linspace(-0.05, 0.05, 400_001)]).astype(np.float32)
    near = np.concatenate([np.nextafter(fine, np.float32(np.inf)), np.nextafter(fine, np.float32(-np.inf))])
    return np.concatenate([base, rand, fine, near]).astype(np.float32)


def test_known_answer_from_reference_tests():
    # bf16(0.3223) * 57344 -> e5m2: the kernel yields 16384.0 (0x74) because the product is
    # rounded to bf16 first; an fp32 product would give 20480.0 (0x75).
    a = torch.tensor([0.3223, 0.3223], dtype=torch.float32).to(torch.bfloat16).view(2, 1)
    out = qo.saturated_cast(a, 57344.0, torch.float8_e5m2)
    assert out.view(torch.uint8).flatten().tolist() == [0x74, 0x74]
    assert out.float().flatten().tolist() == [16384.0, 16384.0]
    fp32_product = (a.float() * 57344.0).clamp(-57344, 57344).to(torch.float8_e5m2)
    assert fp32_product.float().flatten().tolist() == [20480.0, 20480.0]


@pytest.mark.parametrize("kind,dtype,vmax", KINDS)
def test_f32_to_fp8_matches_toolkit_header(kind, dtype, vmax):
    vals = fp32_sweep()
    mine = qo.f32_to_fp8_array(vals, kind)
    hdr = qo.f32_to_fp8_array(vals, kind, header=True)
    nan = np.isnan(vals)
    assert np.array_equal(mine[~nan], hdr[~nan])
    # NaN: both must produce a NaN encoding (the sign bit is not pinned)
    nan_code = {qo.E4M3: lambda b: (b & 0x7F) == 0x7F, qo.E5M2: lambda b: (b & 0x7F) > 0x7C}[kind]
    assert nan_code(mine[nan]).all() and nan_code(hdr[nan]).all()


@pytest.mark.parametrize("kind,dtype,vmax", KINDS)
def test_f32_to_fp8_matches_torch_cpu_after_clamp(kind, dtype, vmax):
    vals = fp32_sweep()
    vals = vals[~np.isnan(vals)]
    mine = qo.f32_to_fp8_array(vals, kind)
    t = torch.from_numpy(vals).clamp(-vmax, vmax).to(dtype).view(torch.uint8).numpy()
    assert np.array_equal(mine, t)


@pytest.mark.parametrize("kind,dtype,vmax", KINDS)
def test_saturation_and_specials(kind, dtype, vmax):
    cmax = 0x7E if kind == qo.E4M3 else 0x7B
    vals = np.array([vmax, np.nextafter(np.float32(vmax), np.float32(np.inf)), 1e30, np.inf, -np.inf, -1e30, 0.0, -0.0],
                    dtype=np.float32)
    got = qo.f32_to_fp8_array(vals, kind).tolist()
    assert got == [cmax, cmax, cmax, cmax, 0x80 | cmax, 0x80 | cmax, 0x00, 0x80]


def test_f32_to_bf16_matches_toolkit_header():
    vals = fp32_sweep()
    mine = qo.f32_to_bf16_array(vals)
    hdr = qo.f32_to_bf16_array(vals, header=True)
    nan = np.isnan(vals)
    assert np.array_equal(mine[~nan], hdr[~nan])
    assert ((mine[nan] & 0x7FFF) > 0x7F80).all()
    t = torch.from_numpy(vals[~nan]).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(mine[~nan], t)


@pytest.mark.parametrize("scale", [1.0, 0.5, 3.140625, 57344.0, 448.0 / 5.21875, 1e-3, 2.0**-100, 2.0**100])
def test_bf16_multiply_matches_toolkit_header(scale):
    # The header's host path rounds the fp32 product (its device path is one bf16 multiply);
    # the two agree whenever that fp32 product is exact, i.e. not subnormal in fp32.
    a = all_bf16_bits()
    s_bits = int(qo.f32_to_bf16_array(np.array([scale], dtype=np.float32))[0])
    mine = qo.bf16_mul_array(a, s_bits)
    hdr = qo.bf16_mul_array(a, s_bits, header=True)
    af = bf16_bits_to_f32(a).astype(np.float64)
    sf = float(bf16_bits_to_f32(np.array([s_bits], dtype=np.uint16))[0])
    exact = af * sf
    ok = ~np.isnan(exact) & ((np.abs(exact) >= 2.0**-126) | (exact == 0))
    assert np.array_equal(mine[ok], hdr[ok])
    # single rounding of the exact product: compare with numpy float64 -> bf16 by hand where normal
    nan = np.isnan(exact)
    assert ((mine[nan] & 0x7FFF) > 0x7F80).all()


def test_e8m0_matches_toolkit_header():
    H = qo.header_lib()
    for biased in range(0, 255):
        scale = np.array([biased << 23], dtype=np.uint32).view(np.float32)[0]
        assert H.hdr_f32_to_e8m0(float(scale)) == biased
    assert H.hdr_f32_to_e8m0(float("inf")) == 0xFE


def test_bf16_to_fp8_header_path_equals_via_fp32():
    H = qo.header_lib()
    bits = all_bf16_bits()
    vals = bf16_bits_to_f32(bits)
    for kind in (qo.E4M3, qo.E5M2):
        mine = qo.f32_to_fp8_array(vals, kind)
        for b in range(0, 65536, 7):  # a stride keeps this loop short; the fp32 sweep covers all values
            if np.isnan(vals[b]):
                continue
            assert H.hdr_bf16_to_fp8(int(bits[b]), kind) == mine[b]


def test_e2m1_conversion_matches_the_toolkit_header():
    """The plain-C e2m1 rounding against __nv_cvt_float_to_fp4 (host path of cuda_fp4.hpp), on every
    bf16-valued float, on a fine sweep around the representable values, and the packing order."""
    L, H = qo.lib(), qo.header_lib()
    vals = [float(v) for v in torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()]
    vals += [k / 64.0 for k in range(-512, 513)] + [float("inf"), float("-inf"), 1e-45, -1e-45, 6.0000005, 5.9999995]
    for v in vals:
        if v != v:
            continue  # NaN: compared below
        assert L.oracle_f32_to_e2m1(v) == H.hdr_f32_to_fp4(v), v
    assert L.oracle_f32_to_e2m1(float("nan")) == H.hdr_f32_to_fp4(float("nan")) == 0x7
    assert H.hdr_f32x2_to_fp4x2(1.0, -6.0) == 0xF2  # first element in the low nibble


def test_f16_widening_and_mx_formats_reduce_to_the_reference_case():
    L = qo.lib()
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    want = bits.view(torch.float16).float()
    got = torch.tensor([L.oracle_f16_to_f32(int(b) & 0xFFFF) for b in bits.tolist()])
    assert torch.equal(got.view(torch.int32)[~want.isnan()], want.view(torch.int32)[~want.isnan()])
    assert got[want.isnan()].isnan().all()
    # bf16 input, e4m3 payload: the generalised function is the reference restatement
    g = torch.Generator().manual_seed(3)
    a = bits[torch.randperm(65536, generator=g)].view(torch.bfloat16).view(64, 1024)
    p0, s0 = qo.mx_fp8_quantize(a)
    p1, s1 = qo.mx_quantize(a, torch.float8_e4m3fn)
    assert torch.equal(p0.view(torch.uint8), p1.view(torch.uint8)) and torch.equal(s0.view(torch.uint8), s1.view(torch.uint8))
    # fp32 input that is bf16-valued gives the same bytes as the bf16 input; e5m2 / e2m1 scale bytes differ
    # from e4m3's by the difference of the formats' largest exponents wherever no clamp acts
    p2, s2 = qo.mx_quantize(a.float(), torch.float8_e4m3fn)
    assert torch.equal(p1.view(torch.uint8), p2.view(torch.uint8)) and torch.equal(s1.view(torch.uint8), s2.view(torch.uint8))
    _, s5 = qo.mx_quantize(a, torch.float8_e5m2)
    _, s4 = qo.mx_quantize(a, "e2m1")
    e4, e5, e2 = (t.view(torch.uint8).int() for t in (s1, s5, s4))
    ok = (e4 > 7) & (e4 < 249)
    assert torch.equal(e5[ok], e4[ok] - 7) and torch.equal(e2[ok], e4[ok] + 6)
