"""Fake-tensor (meta) implementations for ``torch.ops.DrissTorch``.

The first two repeat the reference's registrations (driss_torch/abstract_impls.py:5-19);
the reference registers none for ``dynamic_scaled_quant`` and ``mx_fp8_quantize``, which
makes them untraceable under ``torch.compile``; they are added here together with the
fakes of the new ops.
"""
import torch
from torch.library import register_fake


@register_fake("DrissTorch::saturated_cast")
def saturated_cast_meta(x: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype, transpose: bool = False):
    if transpose:
        return torch.empty((x.shape[1], x.shape[0]), dtype=out_dtype, device=x.device)
    return torch.empty_like(x, dtype=out_dtype)


@register_fake("DrissTorch::amax")
def amax_meta(x: torch.Tensor):
    return torch.empty(1, dtype=torch.float32, device=x.device)


@register_fake("DrissTorch::dynamic_scaled_quant")
def dynamic_scaled_quant_meta(x: torch.Tensor, dtype: torch.dtype):
    return torch.empty_like(x, dtype=dtype)


@register_fake("DrissTorch::mx_fp8_quantize")
def mx_fp8_quantize_meta(x: torch.Tensor, block_size: int, axis: int, transpose: bool, fp8_type: torch.dtype):
    m, n = x.shape
    along_rows = axis in (0, -2)
    if along_rows != transpose:  # blocks down the columns: the transposing kernel's outputs
        payload_t = torch.empty((n, m), dtype=fp8_type, device=x.device)
        scales_t = torch.empty(n * (m // 32), dtype=torch.float8_e8m0fnu, device=x.device)
        return (payload_t if transpose else payload_t.t()), scales_t
    payload = torch.empty_like(x, dtype=fp8_type)
    scales = torch.empty(m * ((n + 31) // 32), dtype=torch.float8_e8m0fnu, device=x.device)
    return (payload.t() if transpose else payload), scales


@register_fake("DrissTorch::mx_fp8_bf16")
def mx_fp8_bf16_meta(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor):
    return torch.empty((a.shape[0], b.shape[1]), dtype=torch.bfloat16, device=a.device)


@register_fake("DrissTorch::sweep_mm")
def sweep_mm_meta(x, w, x_scale, w_scale, bias, out_dtype, use_fast_accum, cluster_shape_x, cluster_shape_y, cluster_shape_z,
                  transposed, swizzle):
    return torch.empty((x.shape[0], w.shape[1]), dtype=out_dtype, device=x.device)


@register_fake("DrissTorch::mx_fp4_bf16")
def mx_fp4_bf16_meta(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor):
    return torch.empty((a.shape[0], b.shape[1]), dtype=torch.bfloat16, device=a.device)


@register_fake("DrissTorch::dynamic_scaled_quant_with_scale")
def dynamic_scaled_quant_with_scale_meta(x: torch.Tensor, dtype: torch.dtype):
    one = lambda: torch.empty(1, dtype=torch.float32, device=x.device)  # noqa: E731
    return torch.empty_like(x, dtype=dtype), one(), one()


@register_fake("DrissTorch::dynamic_scaled_quant_rowwise")
def dynamic_scaled_quant_rowwise_meta(x: torch.Tensor, dtype: torch.dtype):
    col = lambda: torch.empty(x.shape[0], 1, dtype=torch.float32, device=x.device)  # noqa: E731
    return torch.empty_like(x, dtype=dtype), col(), col()


@register_fake("DrissTorch::cast_with_amax")
def cast_with_amax_meta(x: torch.Tensor, amax: torch.Tensor, dtype: torch.dtype):
    return torch.empty_like(x, dtype=dtype), torch.empty(1, dtype=torch.float32, device=x.device)


@register_fake("DrissTorch::mx_fp8_quantize_blocked")
def mx_fp8_quantize_blocked_meta(x: torch.Tensor):
    m, n = x.shape
    nbytes = ((m + 127) // 128) * ((n // 32 + 3) // 4) * 512
    return torch.empty_like(x, dtype=torch.float8_e4m3fn), torch.empty(nbytes, dtype=torch.float8_e8m0fnu, device=x.device)


@register_fake("DrissTorch::mx_fp8_quantize_dual")
def mx_fp8_quantize_dual_meta(x: torch.Tensor, blocked: bool = False):
    m, n = x.shape
    e4m3, e8m0 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    if blocked:
        def nbytes(r, c):
            return ((r + 127) // 128) * ((c // 32 + 3) // 4) * 512
        return (torch.empty((m, n), dtype=e4m3, device=x.device), torch.empty(nbytes(m, n), dtype=e8m0, device=x.device),
                torch.empty((n, m), dtype=e4m3, device=x.device), torch.empty(nbytes(n, m), dtype=e8m0, device=x.device))
    return (torch.empty((m, n), dtype=e4m3, device=x.device), torch.empty(m * (n // 32), dtype=e8m0, device=x.device),
            torch.empty((n, m), dtype=e4m3, device=x.device), torch.empty(n * (m // 32), dtype=e8m0, device=x.device))


@register_fake("DrissTorch::saturated_cast_transposed")
def saturated_cast_transposed_meta(x: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype):
    return torch.empty((x.shape[1], x.shape[0]), dtype=dtype, device=x.device)


@register_fake("DrissTorch::saturated_cast_dual")
def saturated_cast_dual_meta(x: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype):
    return (torch.empty(tuple(x.shape), dtype=dtype, device=x.device),
            torch.empty((x.shape[1], x.shape[0]), dtype=dtype, device=x.device))


@register_fake("DrissTorch::mx_fp4_quantize")
def mx_fp4_quantize_meta(x: torch.Tensor, blocked: bool = False):
    m, n = x.shape
    nscales = ((m + 127) // 128) * ((n // 32 + 3) // 4) * 512 if blocked else m * (n // 32)
    return (torch.empty((m, n // 2), dtype=torch.uint8, device=x.device),
            torch.empty(nscales, dtype=torch.float8_e8m0fnu, device=x.device))


@register_fake("DrissTorch::mx_fp8_quantize_with_amax")
def mx_fp8_quantize_with_amax_meta(x: torch.Tensor):
    m, n = x.shape
    return (torch.empty_like(x, dtype=torch.float8_e4m3fn),
            torch.empty(m * (n // 32), dtype=torch.float8_e8m0fnu, device=x.device),
            torch.empty(1, dtype=torch.float32, device=x.device))


@register_fake("DrissTorch::cast_with_amax_dual")
def cast_with_amax_dual_meta(x: torch.Tensor, amax: torch.Tensor, dtype: torch.dtype):
    return (torch.empty(tuple(x.shape), dtype=dtype, device=x.device),
            torch.empty((x.shape[1], x.shape[0]), dtype=dtype, device=x.device),
            torch.empty(1, dtype=torch.float32, device=x.device))


@register_fake("DrissTorch::dynamic_scaled_quant_dual")
def dynamic_scaled_quant_dual_meta(x: torch.Tensor, dtype: torch.dtype):
    return (torch.empty(tuple(x.shape), dtype=dtype, device=x.device),
            torch.empty((x.shape[1], x.shape[0]), dtype=dtype, device=x.device),
            torch.empty(1, dtype=torch.float32, device=x.device), torch.empty(1, dtype=torch.float32, device=x.device))
