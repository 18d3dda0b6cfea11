"""TEST INFRASTRUCTURE ONLY: the PyTorch-eager computations the reference's tests
compare its kernels against, for CPU tensors.

These are what the benchmark times as the reference's CPU path.  They are NOT
bit-identical to the kernels in general (see ``saturated_cast_eager`` below);
the bit-exact checker is ``quant_oracle``.
"""
from __future__ import annotations

import torch


def fp8_max(dtype: torch.dtype) -> float:
    return float(torch.finfo(dtype).max)


def amax_to_scale(amax: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """fp32 tensor-wise scale ``fp8_max / max(amax, 1e-12)``, formed in float64 (0-dim)."""
    a = amax.to(torch.float64).reshape(()).clamp_min(1e-12)
    return (fp8_max(fp8_dtype) / a).to(torch.float32)


def amax_eager(a: torch.Tensor) -> torch.Tensor:
    """The amax test's expectation (test/test_amax.py:6-7): max |a| as an fp32 [1] tensor."""
    return a.abs().max().to(torch.float32).reshape(1)


def saturated_cast_eager(a: torch.Tensor, scale: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """The cast tests' expectation (test/test_sat_cast.py:7-24, test/test_dynamic_quant.py:9-26):
    multiply, clamp to the finite fp8 range, convert.

    With a bf16 ``a`` and a 1-element fp32 ``scale`` of shape [1] the product is formed in fp32,
    which is NOT what the bf16 kernel does (it rounds the scale and the product to bf16); the
    reference keeps a strict-xfail test for exactly that difference (test/test_sat_cast.py:65-83).
    Pass ``scale.to(a.dtype)`` for the kernel-faithful product.
    """
    m = fp8_max(fp8_dtype)
    return (a * scale).clamp(min=-m, max=m).to(fp8_dtype)


def saturated_cast_kernel_faithful(a: torch.Tensor, scale: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """Eager form of the kernel arithmetic: for bf16 input the scale is rounded to bf16 first."""
    return saturated_cast_eager(a, scale.to(a.dtype), fp8_dtype)


def dynamic_scaled_quant_eager(a: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """Eager form of src/dynamic_scaled_quant.cu:111-116: double scale and product, fp32, fp8."""
    amax = a.abs().max().to(torch.float64)
    sd = fp8_max(fp8_dtype) / (amax + 1e-12)
    p = (sd * a.to(torch.float64)).to(torch.float32)
    m = fp8_max(fp8_dtype)
    return p.clamp(min=-m, max=m).to(fp8_dtype)


def dynamic_scaled_quant_rowwise_eager(a: torch.Tensor, fp8_dtype: torch.dtype):
    amax = a.abs().amax(dim=1, keepdim=True).to(torch.float32)
    sd = fp8_max(fp8_dtype) / (amax.to(torch.float64) + 1e-12)
    p = (sd * a.to(torch.float64)).to(torch.float32)
    m = fp8_max(fp8_dtype)
    return p.clamp(min=-m, max=m).to(fp8_dtype), amax, sd.to(torch.float32)


def mx_fp8_quantize_eager(a: torch.Tensor):
    """Tensor-level form of src/mx_cast.cu:44-86,146-153 for bf16 [M, N], N % 32 == 0.

    Valid for blocks whose scale exponent stays in the normal range (the timed workloads);
    the degenerate all-zero / tiny / non-finite blocks are covered by ``quant_oracle`` only.
    """
    M, N = a.shape
    x = a.to(torch.float32).reshape(M, N // 32, 32)
    bits = x.abs().view(torch.int32)
    be = bits >> 23
    e = be - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    e = torch.where(be == 0, torch.where(bits == 0, -128, -126), e)
    E = e.amax(dim=2, keepdim=True)
    biased = (E - 8 + 127).clamp(0, 255)
    inv = torch.ldexp(torch.ones(biased.shape, dtype=torch.float32, device=biased.device), 127 - biased)
    p = (x * inv).clamp(min=-448.0, max=448.0).to(torch.float8_e4m3fn).reshape(M, N)
    scales = biased.clamp(max=254).to(torch.uint8).reshape(-1).view(torch.float8_e8m0fnu)
    return p, scales
