"""TEST INFRASTRUCTURE ONLY: ctypes front end of ``quant_oracle.c``.

Takes and returns CPU ``torch`` tensors so that tests read like the reference's
own tests; the arithmetic is all in the C file, which cites the reference lines
it restates.  Also loads ``header_check.cpp`` (shims over the CUDA toolkit's
host-callable conversion helpers) for the exhaustive conversion pins.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_BUILD = _HERE / "_build"

BF16, F32 = 0, 1
E4M3, E5M2 = 0, 1

_IN = {torch.bfloat16: BF16, torch.float32: F32}
_OUT = {torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}


def _stale(target: Path, src: Path) -> bool:
    return (not target.exists()) or target.stat().st_mtime < src.stat().st_mtime


def build(force: bool = False) -> None:
    """Compile the C oracle and the header shims into ``oracle/_build``."""
    _BUILD.mkdir(exist_ok=True)
    so = _BUILD / "libquant_oracle.so"
    src = _HERE / "quant_oracle.c"
    if force or _stale(so, src):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", str(src), "-o", str(so), "-lm"]
        )
    so = _BUILD / "libheader_check.so"
    src = _HERE / "header_check.cpp"
    cuda_inc = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
    if (force or _stale(so, src)) and Path(cuda_inc, "cuda_fp8.h").exists():
        subprocess.check_call(["g++", "-O2", "-shared", "-fPIC", "-I" + cuda_inc, str(src), "-o", str(so)])


_lib = None
_hdr = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_BUILD / "libquant_oracle.so"))
        vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
        L.oracle_saturated_cast.argtypes = [vp, i32, f32, vp, i64, i32]
        L.oracle_saturated_cast.restype = None
        L.oracle_amax.argtypes = [vp, i32, i64]
        L.oracle_amax.restype = f32
        L.oracle_cast_with_amax.argtypes = [vp, i32, f32, vp, i64, i32, vp]
        L.oracle_cast_with_amax.restype = None
        L.oracle_dynamic_scaled_quant.argtypes = [vp, i32, vp, i64, i32, vp, vp]
        L.oracle_dynamic_scaled_quant.restype = None
        L.oracle_dynamic_scaled_quant_rowwise.argtypes = [vp, i32, vp, i64, i64, i32, vp, vp]
        L.oracle_dynamic_scaled_quant_rowwise.restype = None
        L.oracle_mx_fp8_quantize.argtypes = [vp, vp, vp, i64]
        L.oracle_mx_fp8_quantize.restype = None
        L.oracle_mx_quantize.argtypes = [vp, i32, vp, vp, i64, i32]
        L.oracle_mx_quantize.restype = None
        L.oracle_mx_gemm_bf16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32]
        L.oracle_mx_gemm_bf16.restype = None
        L.oracle_rowwise_gemm_bf16.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32]
        L.oracle_rowwise_gemm_bf16.restype = None
        L.oracle_f32_to_e2m1.argtypes = [f32]
        L.oracle_f32_to_e2m1.restype = C.c_uint8
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f16_to_f32.restype = f32
        L.oracle_f32_to_fp8_array.argtypes = [vp, vp, i64, i32]
        L.oracle_bf16_mul_array.argtypes = [vp, C.c_uint16, vp, i64]
        L.oracle_f32_to_bf16_array.argtypes = [vp, vp, i64]
        L.oracle_num_threads.restype = i32
        L.oracle_set_num_threads.argtypes = [i32]
        _lib = L
    return _lib


def header_lib() -> C.CDLL:
    global _hdr
    if _hdr is None:
        build()
        H = C.CDLL(str(_BUILD / "libheader_check.so"))
        vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
        H.hdr_f32_to_fp8_array.argtypes = [vp, vp, i64, i32]
        H.hdr_bf16_mul_array.argtypes = [vp, C.c_uint16, vp, i64]
        H.hdr_f32_to_bf16_array.argtypes = [vp, vp, i64]
        H.hdr_f32_to_fp4.argtypes = [C.c_float]
        H.hdr_f32_to_fp4.restype = C.c_uint8
        H.hdr_f32x2_to_fp4x2.argtypes = [C.c_float, C.c_float]
        H.hdr_f32x2_to_fp4x2.restype = C.c_uint8
        H.hdr_f32_to_e8m0.argtypes = [C.c_float]
        H.hdr_f32_to_e8m0.restype = C.c_uint8
        H.hdr_bf16_to_fp8.argtypes = [C.c_uint16, i32]
        H.hdr_bf16_to_fp8.restype = C.c_uint8
        _hdr = H
    return _hdr


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def _chk(x: torch.Tensor) -> torch.Tensor:
    assert x.device.type == "cpu", "the oracle is a CPU checker"
    assert x.dtype in _IN, f"unsupported input dtype {x.dtype}"
    return x.contiguous()


def saturated_cast(x: torch.Tensor, scale, out_dtype: torch.dtype) -> torch.Tensor:
    x = _chk(x)
    out = torch.empty(x.shape, dtype=torch.uint8)
    lib().oracle_saturated_cast(x.data_ptr(), _IN[x.dtype], float(scale), out.data_ptr(), x.numel(), _OUT[out_dtype])
    return out.view(out_dtype)


def amax(x: torch.Tensor) -> torch.Tensor:
    x = _chk(x)
    v = lib().oracle_amax(x.data_ptr(), _IN[x.dtype], x.numel())
    return torch.tensor([v], dtype=torch.float32)


def cast_with_amax(x: torch.Tensor, amax_value: float, out_dtype: torch.dtype, out: torch.Tensor | None = None):
    """Cast phase of the fused op for a given (e.g. all-reduced) amax; ``out``: a uint8 buffer to reuse."""
    x = _chk(x)
    out = torch.empty(x.shape, dtype=torch.uint8) if out is None else out
    assert out.dtype == torch.uint8 and out.is_contiguous() and out.numel() == x.numel()
    scale = torch.empty(1, dtype=torch.float32)
    lib().oracle_cast_with_amax(
        x.data_ptr(), _IN[x.dtype], float(amax_value), out.data_ptr(), x.numel(), _OUT[out_dtype], scale.data_ptr()
    )
    return out.view(out_dtype), scale


def dynamic_scaled_quant(x: torch.Tensor, out_dtype: torch.dtype):
    """Returns (payload, amax[1], scale[1])."""
    x = _chk(x)
    out = torch.empty(x.shape, dtype=torch.uint8)
    am = torch.empty(1, dtype=torch.float32)
    sc = torch.empty(1, dtype=torch.float32)
    lib().oracle_dynamic_scaled_quant(
        x.data_ptr(), _IN[x.dtype], out.data_ptr(), x.numel(), _OUT[out_dtype], am.data_ptr(), sc.data_ptr()
    )
    return out.view(out_dtype), am, sc


def dynamic_scaled_quant_rowwise(x: torch.Tensor, out_dtype: torch.dtype):
    """Returns (payload, amax[M,1], scale[M,1])."""
    x = _chk(x)
    assert x.dim() == 2
    rows, cols = x.shape
    out = torch.empty(x.shape, dtype=torch.uint8)
    am = torch.empty(rows, 1, dtype=torch.float32)
    sc = torch.empty(rows, 1, dtype=torch.float32)
    lib().oracle_dynamic_scaled_quant_rowwise(
        x.data_ptr(), _IN[x.dtype], out.data_ptr(), rows, cols, _OUT[out_dtype], am.data_ptr(), sc.data_ptr()
    )
    return out.view(out_dtype), am, sc


def mx_fp8_quantize(x: torch.Tensor, payload: torch.Tensor | None = None, scales: torch.Tensor | None = None):
    """bf16 [M, N] with N % 32 == 0 -> (e4m3 payload [M, N], e8m0 scales [M * N / 32]); ``payload`` /
    ``scales``: uint8 buffers to reuse."""
    x = _chk(x)
    assert x.dtype == torch.bfloat16 and x.numel() % 32 == 0
    payload = torch.empty(x.shape, dtype=torch.uint8) if payload is None else payload
    scales = torch.empty(x.numel() // 32, dtype=torch.uint8) if scales is None else scales
    assert payload.dtype == torch.uint8 and payload.is_contiguous() and payload.numel() == x.numel()
    assert scales.dtype == torch.uint8 and scales.is_contiguous() and scales.numel() == x.numel() // 32
    lib().oracle_mx_fp8_quantize(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), x.numel() // 32)
    return payload.view(torch.float8_e4m3fn), scales.view(torch.float8_e8m0fnu)


MX_IN = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}
MX_FMT = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1, "e2m1": 2, torch.float4_e2m1fn_x2: 2}


def mx_quantize(x: torch.Tensor, elem):
    """[M, N] bf16 / fp16 / fp32 with N % 32 == 0 -> (payload, e8m0 scales [M * N / 32]); ``elem`` an fp8
    dtype (payload [M, N]) or "e2m1" (payload uint8 [M, N / 2], lower index in the low nibble)."""
    assert x.device.type == "cpu" and x.is_contiguous() and x.dtype in MX_IN and x.numel() % 32 == 0
    fmt = MX_FMT[elem]
    rows, cols = x.shape
    payload = torch.zeros((rows, cols // 2) if fmt == 2 else (rows, cols), dtype=torch.uint8)
    scales = torch.empty(x.numel() // 32, dtype=torch.uint8)
    lib().oracle_mx_quantize(x.data_ptr(), MX_IN[x.dtype], payload.data_ptr(), scales.data_ptr(), x.numel() // 32, fmt)
    return (payload if fmt == 2 else payload.view(elem)), scales.view(torch.float8_e8m0fnu)


def mx_gemm_bf16(a: torch.Tensor, b_nk: torch.Tensor, a_scale_blocked: torch.Tensor, b_scale_blocked: torch.Tensor,
                 fp4: bool = False) -> torch.Tensor:
    """The MX block-scaled GEMM: ``a`` [M, K] e4m3 (or uint8 [M, K/2] packed e2m1 with ``fp4``), ``b_nk`` [N, K]
    (the reference's operand ``b`` is its transpose view), scales as blocked e8m0 bytes; returns bf16 [M, N]."""
    a8 = a.contiguous().view(torch.uint8)
    b8 = b_nk.contiguous().view(torch.uint8)
    m, n = a8.shape[0], b8.shape[0]
    k = a8.shape[1] * (2 if fp4 else 1)
    assert b8.shape[1] == a8.shape[1]
    sa = a_scale_blocked.contiguous().view(torch.uint8)
    sb = b_scale_blocked.contiguous().view(torch.uint8)
    katoms = ((k + 31) // 32 + 3) // 4
    assert sa.numel() == ((m + 127) // 128) * katoms * 512 and sb.numel() == ((n + 127) // 128) * katoms * 512
    out = torch.empty(m, n, dtype=torch.int16)
    lib().oracle_mx_gemm_bf16(a8.data_ptr(), b8.data_ptr(), sa.data_ptr(), sb.data_ptr(), out.data_ptr(), m, n, k,
                              2 if fp4 else 0)
    return out.view(torch.bfloat16)


def rowwise_gemm_bf16(a: torch.Tensor, b_nk: torch.Tensor, a_row_scale: torch.Tensor, b_row_scale: torch.Tensor,
                      bias: torch.Tensor | None = None) -> torch.Tensor:
    """The row-wise scaled fp8 GEMM: ``a`` [M, K] e4m3 / e5m2, ``b_nk`` [N, K] e4m3, fp32 scales [M] and [N], optional
    bias [N] (given in fp32); returns bf16 [M, N]."""
    a8, b8 = a.contiguous().view(torch.uint8), b_nk.contiguous().view(torch.uint8)
    m, k = a8.shape
    n = b8.shape[0]
    xs = a_row_scale.contiguous().float().view(-1)
    ws = b_row_scale.contiguous().float().view(-1)
    assert xs.numel() == m and ws.numel() == n and b8.shape[1] == k
    bf = None if bias is None else bias.contiguous().float()
    out = torch.empty(m, n, dtype=torch.int16)
    lib().oracle_rowwise_gemm_bf16(a8.data_ptr(), b8.data_ptr(), xs.data_ptr(), ws.data_ptr(),
                                   None if bf is None else bf.data_ptr(), out.data_ptr(), m, n, k, _OUT[a.dtype])
    return out.view(torch.bfloat16)


# ---- conversion tables for the exhaustive pins -------------------------------------------------

def f32_to_fp8_array(vals: np.ndarray, kind: int, header: bool = False) -> np.ndarray:
    vals = np.ascontiguousarray(vals, dtype=np.float32)
    out = np.empty(vals.shape, dtype=np.uint8)
    fn = header_lib().hdr_f32_to_fp8_array if header else lib().oracle_f32_to_fp8_array
    fn(vals.ctypes.data, out.ctypes.data, vals.size, kind)
    return out


def bf16_mul_array(a_bits: np.ndarray, b_bits: int, header: bool = False) -> np.ndarray:
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    out = np.empty(a_bits.shape, dtype=np.uint16)
    fn = header_lib().hdr_bf16_mul_array if header else lib().oracle_bf16_mul_array
    fn(a_bits.ctypes.data, int(b_bits), out.ctypes.data, a_bits.size)
    return out


def f32_to_bf16_array(vals: np.ndarray, header: bool = False) -> np.ndarray:
    vals = np.ascontiguousarray(vals, dtype=np.float32)
    out = np.empty(vals.shape, dtype=np.uint16)
    fn = header_lib().hdr_f32_to_bf16_array if header else lib().oracle_f32_to_bf16_array
    fn(vals.ctypes.data, out.ctypes.data, vals.size)
    return out


def blocked_scale_offsets(rows: int, kblocks: int) -> np.ndarray:
    """Offset of scale (r, c) in the blocked layout of the reference's MX GEMM
    (src/mx_fp8_bf16.cu:97-110; CUTLASS Sm1xxBlockScaledConfig): 128 x 4 atoms of 512 bytes, k-major
    atom order, (r % 32) * 16 + (r % 128 // 32) * 4 + c % 4 inside an atom.  Shape [rows, kblocks]."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(kblocks, dtype=np.int64)[None, :]
    katoms = (kblocks + 3) // 4
    return ((r // 128) * katoms + c // 4) * 512 + (r % 32) * 16 + (r % 128 // 32) * 4 + c % 4


def to_blocked(scales_row_major: torch.Tensor, rows: int, kblocks: int) -> torch.Tensor:
    """Row-major [rows * kblocks] scale bytes -> blocked layout (uint8, zero padding)."""
    off = blocked_scale_offsets(rows, kblocks)
    out = np.zeros(((rows + 127) // 128) * ((kblocks + 3) // 4) * 512, dtype=np.uint8)
    out[off.ravel()] = scales_row_major.view(torch.uint8).numpy().ravel()
    return torch.from_numpy(out)
