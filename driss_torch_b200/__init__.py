"""B200-native FP8 / MX quantization ops behind the ``torch.ops.DrissTorch`` API.

Drop-in for the quantization part of ``driss_torch`` (driss_torch/__init__.py:20-47,
:114-122): same function names, positional order, defaults and return types;
``import driss_torch_b200 as driss_torch`` is the whole migration for that path.

Importing loads ``lib/libdriss_torch.so`` (the ``TORCH_LIBRARY(DrissTorch)``
registration, which pulls in the CUDA kernels in ``lib/libdtq_b200.so``) and the
fake-tensor implementations.  There is no CPU implementation and no fallback: if the
libraries have not been built (``python driss_torch_b200/build.py``) the import fails.
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

_LIB_DIR = Path(__file__).resolve().parent / "lib"
lib_path = _LIB_DIR / "libdriss_torch.so"
kernels_lib_path = _LIB_DIR / "libdtq_b200.so"

if not lib_path.exists() or not kernels_lib_path.exists():
    raise ImportError(
        f"{lib_path.name} / {kernels_lib_path.name} not found in {_LIB_DIR}: build them with "
        "`python driss_torch_b200/build.py` (needs nvcc with sm_100a support); there is no fallback path"
    )

torch.ops.load_library(str(lib_path))
torch.ops.import_module("driss_torch_b200.abstract_impls")

ops = torch.ops.DrissTorch
Tensor = torch.Tensor


def saturated_cast(
    x: Tensor,
    scale: Tensor,
    out_dtype: torch.dtype,
    transpose: bool = False,
) -> Tensor:
    """``fp8(x * scale)`` with saturation to the largest finite fp8 value.

    Args:
        x: 2-D bf16 or fp32 CUDA tensor.
        scale: a one-element fp32 tensor on the same device (it is read on the device).
        out_dtype: ``torch.float8_e4m3fn`` or ``torch.float8_e5m2``.
        transpose: must be False.
    For bf16 input the scale is rounded to bf16 and the product is a bf16 multiply, as in the
    reference kernel (src/saturated_cast.cu:66,81).
    """
    assert not transpose, "Transpose is not supported yet"
    return ops.saturated_cast(x, scale, out_dtype, transpose)


def saturated_cast_transposed(x: Tensor, scale: Tensor, out_dtype: torch.dtype) -> Tensor:
    """``saturated_cast(x.t().contiguous(), scale, out_dtype)`` without the separate transpose:
    a contiguous ``[cols, rows]`` tensor.  (The reference declares ``transpose`` on
    ``saturated_cast`` but asserts it off, driss_torch/__init__.py:24-38.)"""
    return ops.saturated_cast_transposed(x, scale, out_dtype)


def saturated_cast_dual(x: Tensor, scale: Tensor, out_dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    """``(saturated_cast(x), saturated_cast(x.t().contiguous()))`` from a single read of ``x``."""
    return ops.saturated_cast_dual(x, scale, out_dtype)


def amax(x: Tensor) -> Tensor:
    """``max(abs(x))`` as an fp32 tensor of shape [1]."""
    return ops.amax(x)


def dynamic_scaled_quant(inpt: Tensor, dtype: torch.dtype) -> Tensor:
    """Tensor-wise amax -> scale -> fp8 cast in one launch; returns the fp8 tensor."""
    return ops.dynamic_scaled_quant(inpt, dtype)


def mx_fp8_quantize(
    input: Tensor,
    block_size: int = 32,
    axis: int = 1,
    transpose: bool = False,
    ScalarType: torch.dtype = torch.float8_e4m3fn,
) -> tuple[Tensor, Tensor]:
    """[M, N] -> (fp8 payload [M, N], E8M0 scales [M * N / 32]), blocks of 32 along N.

    bf16 input with e4m3 payload is the reference's kernel, bit for bit.  fp16 / fp32 inputs and
    ``ScalarType=torch.float8_e5m2`` (which the reference accepts but computes as bf16 -> e4m3) use
    the same scale rule with the format's own largest exponent (15 for e5m2).

    ``axis`` / ``transpose`` (declared and ignored by the reference, src/mx_cast.cu:168-171; bf16 -> e4m3,
    both dimensions multiples of 32): ``transpose=True`` returns ``mx_fp8_quantize(input.t().contiguous())``
    -- payload [N, M], one scale per 32 rows of a column of ``input`` -- from one read of ``input``;
    ``axis=0`` returns the same bytes with the payload viewed as [M, N]; both together give the ordinary
    blocks with the payload viewed as [N, M]."""
    return ops.mx_fp8_quantize(input, block_size, axis, transpose, ScalarType)


def mx_fp8_bf16(a: Tensor, b: Tensor, a_scale: Tensor, b_scale: Tensor) -> Tensor:
    """Matrix multiplication of two MX-quantised e4m3 operands with E8M0 scales of 32 elements along K
    (driss_torch/__init__.py:80-95): ``a`` [M, K] row-major, ``b`` [K, N] column-major (``w.t()`` of a
    row-major [N, K] payload), ``a_scale`` / ``b_scale`` in the blocked layout ``mx_fp8_quantize_blocked``
    writes; returns bf16 [M, N]."""
    return ops.mx_fp8_bf16(a, b, a_scale, b_scale)


def sweep_mm(
    x: Tensor,
    w: Tensor,
    x_scale: Tensor,
    w_scale: Tensor,
    bias: Optional[Tensor],
    out_dtype: torch.dtype,
    use_fast_accum: bool,
    cluster_shape_x: int,
    cluster_shape_y: int,
    cluster_shape_z: int,
    transposed: bool,
    swizzle: int,
) -> Tensor:
    """Row-wise scaled fp8 matrix multiplication (driss_torch/__init__.py:50-77): ``x`` [M, K] e4m3 / e5m2
    row-major, ``w`` [K, N] e4m3 column-major, ``x_scale`` [M, 1] and ``w_scale`` [1, N] fp32 dequantisation scales
    (the reciprocals of ``dynamic_scaled_quant_rowwise``'s), optional ``bias`` [N]; returns
    ``bf16((acc * x_scale) * w_scale + bias)``.  The arguments after ``out_dtype`` tune the reference's Hopper
    kernels and have no effect here."""
    return ops.sweep_mm(x, w, x_scale, w_scale, bias, out_dtype, use_fast_accum, cluster_shape_x, cluster_shape_y,
                        cluster_shape_z, transposed, swizzle)


def mx_fp4_bf16(a: Tensor, b: Tensor, a_scale: Tensor, b_scale: Tensor) -> Tensor:
    """Matrix multiplication of two MXFP4 operands (e2m1 values packed two per byte, the lower index in the low
    nibble; E8M0 scales of 32 elements along K, blocked layout) (driss_torch/__init__.py:98-111): ``a`` [M, K/2]
    bytes row-major, ``b`` [K/2, N] column-major (``w.t()`` of a row-major [N, K/2] payload); returns bf16 [M, N].
    ``mx_fp4_quantize(x, blocked=True)`` produces the payloads and the scales in that layout."""
    return ops.mx_fp4_bf16(a, b, a_scale, b_scale)


# The north-star text calls the MX op "mx_cast"; the reference symbol is mx_fp8_quantize.
mx_cast = mx_fp8_quantize


# ---- additions (no counterpart in the reference) ------------------------------------------------

def dynamic_scaled_quant_with_scale(inpt: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor, Tensor]:
    """As ``dynamic_scaled_quant`` but also returns ``amax`` [1] and the fp32 ``scale`` [1].

    The payload is computed from the double-precision scale, not from the returned fp32 one.
    """
    return ops.dynamic_scaled_quant_with_scale(inpt, dtype)


def dynamic_scaled_quant_rowwise(inpt: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor, Tensor]:
    """Per-row amax -> scale -> fp8 cast; returns (payload, amax [M,1], scale [M,1])."""
    return ops.dynamic_scaled_quant_rowwise(inpt, dtype)


def cast_with_amax(inpt: Tensor, amax_value: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    """The cast phase of ``dynamic_scaled_quant`` for a given device-resident amax; returns (payload, scale)."""
    return ops.cast_with_amax(inpt, amax_value, dtype)


def cast_with_amax_dual(inpt: Tensor, amax_value: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor, Tensor]:
    """``(payload, payload_t, scale)``: ``cast_with_amax`` of ``x`` and of ``x.t().contiguous()`` from one read."""
    return ops.cast_with_amax_dual(inpt, amax_value, dtype)


def dynamic_scaled_quant_dual(inpt: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """``(payload, payload_t, amax, scale)`` with ``payload == dynamic_scaled_quant(x)`` and
    ``payload_t == dynamic_scaled_quant(x.t().contiguous())``: the two fp8 operands tensor-wise scaled
    training needs, in two reads of ``x`` (amax, then both casts at once)."""
    return ops.dynamic_scaled_quant_dual(inpt, dtype)


def mx_fp8_quantize_with_amax(input: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """``mx_fp8_quantize(x)`` plus ``max(0, amax(x))`` (fp32 [1]) from the same read of ``x``: with
    ``cast_with_amax`` behind it, a tensor is quantised both tensor-wise and MX in two reads instead of three."""
    return ops.mx_fp8_quantize_with_amax(input)


def mx_fp4_quantize(input: Tensor, blocked: bool = False) -> tuple[Tensor, Tensor]:
    """MXFP4: ``(uint8 [M, N/2], E8M0 scales [M * N / 32])``; e2m1 values packed two per byte, the
    lower index in the low nibble -- the operands of the reference's ``mx_fp4_bf16``, which has no
    producer kernel there.  Same scale rule as ``mx_fp8_quantize`` with e2m1's largest exponent 2.
    ``blocked``: the scales in the blocked layout ``mx_fp4_bf16`` takes (as ``mx_fp8_quantize_blocked``)."""
    return ops.mx_fp4_quantize(input, blocked)


def mx_fp8_quantize_dual(input: Tensor, blocked: bool = False) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """``(p, s, p_t, s_t)`` with ``(p, s) == mx_fp8_quantize(x)`` and
    ``(p_t, s_t) == mx_fp8_quantize(x.t().contiguous())``, from a single read of ``x``
    (both dimensions multiples of 32).  ``blocked=True``: both scale tensors as
    ``mx_fp8_quantize_blocked`` lays them out, ready for the MX GEMM."""
    return ops.mx_fp8_quantize_dual(input, blocked)


def mx_fp8_quantize_blocked(input: Tensor) -> tuple[Tensor, Tensor]:
    """``mx_fp8_quantize`` with the E8M0 scales already in the blocked (128x4-atom) layout that the MX
    GEMM ``mx_fp8_bf16`` expects, i.e. without the separate ``to_blocked`` pass; zero in the padding."""
    return ops.mx_fp8_quantize_blocked(input)


def check_device_status() -> None:
    """Synchronises and raises if a kernel's bounded device-side wait ever gave up."""
    ops.check_device_status()


from .sharded import ShardedQuantizer  # noqa: E402

__all__ = [
    "saturated_cast",
    "amax",
    "dynamic_scaled_quant",
    "mx_fp8_quantize",
    "mx_cast",
    "mx_fp8_bf16",
    "mx_fp4_bf16",
    "sweep_mm",
    "dynamic_scaled_quant_with_scale",
    "dynamic_scaled_quant_rowwise",
    "cast_with_amax",
    "saturated_cast_transposed",
    "saturated_cast_dual",
    "cast_with_amax_dual",
    "dynamic_scaled_quant_dual",
    "mx_fp8_quantize_with_amax",
    "mx_fp4_quantize",
    "mx_fp8_quantize_dual",
    "mx_fp8_quantize_blocked",
    "check_device_status",
    "ShardedQuantizer",
]
