"""sweep_mm: the row-wise scaled fp8 GEMM (the consumer of the row-wise quantisation scales).

The reference's kernels are CUTLASS Sm90 (Hopper wgmma) instantiations that cannot be built for a B200, so there
is no reference kernel to compare with here; its test (test/test_sweep_mm.py:17-54) compares with torchao's
`addmm_float8_unwrapped_inference`, which is not installed.  What pins this op: the oracle's restatement of the
reference's epilogue tree (src/scaled_mm_kernels/f8f8bf16_rowwise_kernel.h:151-175) checked against an independent
PyTorch evaluation on CPU, the device against the oracle bit for bit on exactly summable inputs (every kernel,
ragged shapes, e5m2 A operand, bias in fp32 and bf16), and the end-to-end property the op exists for: quantise
rows dynamically, multiply, and land close to the bf16 product.
"""
import pytest
import torch

from conftest import as_bytes
from oracle import quant_oracle as qo

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def _operands(m, n, k, a_dtype, seed, with_bias):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-3, 4, (m, k), generator=g).float().to(a_dtype)
    b = torch.randint(-3, 4, (n, k), generator=g).float().to(E4M3)
    xs = torch.exp2(torch.randint(-3, 3, (m,), generator=g).float()) * 1.25
    ws = torch.exp2(torch.randint(-3, 3, (n,), generator=g).float()) * 0.75
    bias = torch.randint(-8, 9, (n,), generator=g).float() * 0.5 if with_bias else None
    return a, b, xs, ws, bias


def test_oracle_against_an_independent_evaluation():
    g = torch.Generator().manual_seed(5)
    for a_dtype in (E4M3, E5M2):
        a = torch.randn(33, 96, generator=g).to(a_dtype)
        b = torch.randn(24, 96, generator=g).to(E4M3)
        xs, ws, bias = torch.rand(33, generator=g) + 0.5, torch.rand(24, generator=g) + 0.5, torch.randn(24, generator=g)
        got = qo.rowwise_gemm_bf16(a, b, xs, ws, bias)
        want = ((a.double() @ b.double().t()).float() * xs[:, None] * ws[None, :] + bias[None, :]).to(torch.bfloat16)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        got = qo.rowwise_gemm_bf16(a, b, xs, ws)
        want = ((a.double() @ b.double().t()).float() * xs[:, None] * ws[None, :]).to(torch.bfloat16)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["pair", "wide", "narrow"])
@pytest.mark.parametrize("m,n,k,a_dtype,bias", [(128, 256, 128, E4M3, None), (256, 512, 512, E4M3, "f32"), (129, 264, 400, E5M2, "bf16"),
                                                (1, 8, 16, E4M3, None), (300, 520, 96, E5M2, "f32"), (1024, 1024, 1024, E4M3, "bf16"),
                                                (2560, 2048, 256, E4M3, None)])
def test_exact_against_the_oracle(m, n, k, a_dtype, bias, kernel):
    from driss_torch_b200 import _cabi

    a, b, xs, ws, bias_f = _operands(m, n, k, a_dtype, seed=m + n + k, with_bias=bias is not None)
    want = qo.rowwise_gemm_bf16(a, b, xs, ws, bias_f)  # the bias values are bf16-exact, so fp32 and bf16 agree
    bias_d = None if bias is None else bias_f.to(torch.float32 if bias == "f32" else torch.bfloat16).cuda()
    got = _cabi.rowwise_fp8_bf16(a.cuda(), b.cuda(), xs.cuda(), ws.cuda(), bias=bias_d, kernel=kernel).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
        f"{(got.view(torch.int16) != want.view(torch.int16)).sum().item()} of {got.numel()} outputs differ"
    assert _cabi.workspace_status(_cabi.workspace(torch.device("cuda", torch.cuda.current_device()))) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1024, 4096, 2048), (333, 1000, 528), (4096, 4096, 4096)])
def test_rowwise_quantise_then_multiply_tracks_the_bf16_product(shape):
    # the pipeline the op exists for (test/test_sweep_mm.py:17-54 compares the op with another fp8 GEMM on the same
    # operands; here against the product of the dequantised operands, the same arithmetic in bf16/fp32)
    import driss_torch_b200 as dt

    m, k, n = shape
    n = (n + 7) // 8 * 8
    k = (k + 15) // 16 * 16
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    xq, _, x_scale = dt.dynamic_scaled_quant_rowwise(x, E4M3)
    wq, _, w_scale = dt.dynamic_scaled_quant_rowwise(w, E4M3)
    out = dt.sweep_mm(xq, wq.t(), 1.0 / x_scale, (1.0 / w_scale).t(), None, torch.bfloat16, True, 1, 2, 1, True, 8)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    ref = (xq.float() / x_scale) @ (wq.float() / w_scale).t()
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 4e-3, float(err)  # bf16 output rounding
    full = x.float() @ w.float().t()
    assert (out.float() - full).norm() / full.norm() < 0.06  # two e4m3 quantisations
    with pytest.raises(RuntimeError):
        dt.sweep_mm(xq, wq, 1.0 / x_scale, (1.0 / w_scale).t(), None, torch.bfloat16, True, 1, 2, 1, True, 8)  # w must be column-major
    with pytest.raises(RuntimeError):
        dt.sweep_mm(xq, wq.t(), 1.0 / x_scale, (1.0 / w_scale).t(), None, torch.float16, True, 1, 2, 1, True, 8)
    torch._dynamo.reset()
    fn = torch.compile(dt.sweep_mm, fullgraph=True, backend="aot_eager")
    again = fn(xq, wq.t(), 1.0 / x_scale, (1.0 / w_scale).t(), None, torch.bfloat16, True, 1, 2, 1, True, 8)
    assert torch.equal(as_bytes(again.view(torch.int16)), as_bytes(out.view(torch.int16)))
    dt.check_device_status()
