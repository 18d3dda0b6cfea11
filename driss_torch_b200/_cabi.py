"""ctypes view of ``lib/libdtq_b200.so`` -- the C ABI declared in ``include/dtq_b200.h``.

This is how a host that is not PyTorch binds the kernels (raw device pointers, sizes and a
stream).  The GPU parity tests and the benchmark call the kernels through it; the wrappers
below only unwrap ``data_ptr()`` of CUDA tensors and raise on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import functools
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libdtq_b200.so"

BF16, F32 = 0, 1
E4M3, E5M2 = 0, 1
IN_CODE = {torch.bfloat16: BF16, torch.float32: F32}
OUT_CODE = {torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}

_vp, _i64, _i32, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t

SIGNATURES = {
    "dtq_status_string": ([_i32], C.c_char_p),
    "dtq_version": ([], C.c_char_p),
    "dtq_workspace_bytes": ([], _sz),
    "dtq_workspace_init": ([_vp, _sz, _vp], _i32),
    "dtq_workspace_status": ([_vp, _vp, _vp], _i32),
    "dtq_workspace_status_async": ([_vp, _vp, _vp], _i32),
    "dtq_dynamic_scaled_quant_dual": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp, _sz, _vp], _i32),
    "dtq_saturated_cast": ([_vp, _vp, _vp, _i64, _i32, _i32, _vp], _i32),
    "dtq_cast_with_amax_transposed": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp], _i32),
    "dtq_saturated_cast_transposed": ([_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp], _i32),
    "dtq_amax": ([_vp, _vp, _i64, _i32, _vp, _sz, _vp], _i32),
    "dtq_amax_static_scratch": ([_vp, _vp, _i64, _i32, _vp], _i32),
    "dtq_dynamic_scaled_quant": ([_vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp, _sz, _vp], _i32),
    "dtq_p2p_exchange_bytes": ([], _sz),
    "dtq_dynamic_scaled_quant_p2p": ([_vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp, _sz, _vp, _i32, _i32, C.c_uint32,
                                      C.c_uint32, _vp], _i32),
    "dtq_cast_with_amax": ([_vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp], _i32),
    "dtq_dynamic_scaled_quant_rowwise": ([_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp], _i32),
    "dtq_mx_fp8_quantize": ([_vp, _vp, _vp, _i64, _i64, _vp], _i32),
    "dtq_mx_fp8_quantize_amax": ([_vp, _vp, _vp, _vp, _i64, _i64, _vp, _sz, _vp], _i32),
    "dtq_mx_fp8_quantize_amax_p2p": ([_vp, _vp, _vp, _vp, _i64, _i64, _vp, _sz, _vp, _i32, _i32, C.c_uint32, C.c_uint32, _vp], _i32),
    "dtq_mx_quantize": ([_vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp], _i32),
    "dtq_mx_quantize_blocked": ([_vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp], _i32),
    "dtq_mx_fp8_quantize_dual": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp], _i32),
    "dtq_mx_fp8_quantize_dual_blocked": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp], _i32),
    "dtq_mx_fp8_quantize_tma": ([_vp, _vp, _vp, _i64, _i64, _vp, _vp], _i32),
    "dtq_mx_blocked_scale_bytes": ([_i64, _i64], _sz),
    "dtq_mx_gemm_scale_bytes": ([_i64, _i64], _sz),
    "dtq_mx_fp8_bf16": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp], _i32),
    "dtq_mx_fp4_bf16": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp], _i32),
    "dtq_rowwise_fp8_bf16": ([_vp, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _i64, _i64, _i32, _i32, _vp, _sz, _vp], _i32),
    "dtq_mx_gemm_bf16": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp, _sz, _vp], _i32),
    "dtq_mx_fp8_quantize_blocked": ([_vp, _vp, _vp, _i64, _i64, _vp], _i32),
}

_lib = None


def load() -> C.CDLL:
    """Loads the kernel library (no GPU needed to load it) and declares every prototype."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} not built: run `python driss_torch_b200/build.py`")
        lib = C.CDLL(str(LIB_PATH))
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


class DtqError(RuntimeError):
    def __init__(self, what: str, status: int):
        self.status = status
        super().__init__(f"{what} failed: {load().dtq_status_string(status).decode()} (status {status})")


def check(status: int, what: str) -> None:
    if status != 0:
        raise DtqError(what, status)


def _stream(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _on_device_of_first_tensor(fn):
    """The C ABI launches on the CURRENT device: make the first argument's device current for the call, so
    that its current stream and the workspace cached for that stream are the ones used."""

    @functools.wraps(fn)
    def wrapper(x, *args, **kwargs):
        with torch.cuda.device(x.device):
            return fn(x, *args, **kwargs)

    return wrapper


def _ptr(t):
    return None if t is None else t.data_ptr()


_workspaces: dict = {}


def workspace(device=None) -> torch.Tensor:
    """A zero-initialised workspace for the current stream of ``device`` (cached)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device.index, _stream(device))
    ws = _workspaces.get(key)
    if ws is None:
        lib = load()
        with torch.cuda.device(device):
            ws = torch.empty(lib.dtq_workspace_bytes(), dtype=torch.uint8, device=device)
            check(lib.dtq_workspace_init(ws.data_ptr(), ws.numel(), _stream(device)), "dtq_workspace_init")
        _workspaces[key] = ws
    return ws


@_on_device_of_first_tensor
def workspace_status(ws: torch.Tensor) -> int:
    """The workspace's sticky status word (0 = no bounded wait ever gave up); synchronises the stream."""
    out = C.c_int(0)
    check(load().dtq_workspace_status(ws.data_ptr(), C.addressof(out), _stream()), "dtq_workspace_status")
    return out.value


@_on_device_of_first_tensor
def workspace_status_async(ws: torch.Tensor, status_host: torch.Tensor) -> None:
    """Enqueues the copy of the status word into ``status_host`` (a pinned int32 tensor); no synchronisation."""
    check(load().dtq_workspace_status_async(ws.data_ptr(), status_host.data_ptr(), _stream()), "dtq_workspace_status_async")


@_on_device_of_first_tensor
def saturated_cast(x: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None = None):
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out is None else out
    check(
        load().dtq_saturated_cast(x.data_ptr(), out.data_ptr(), scale.data_ptr(), x.numel(), IN_CODE[x.dtype],
                                  OUT_CODE[out_dtype], _stream()),
        "dtq_saturated_cast",
    )
    return out


@_on_device_of_first_tensor
def amax(x: torch.Tensor, out: torch.Tensor | None = None, ws: torch.Tensor | None = None):
    out = torch.empty(1, dtype=torch.float32, device=x.device) if out is None else out
    ws = workspace(x.device) if ws is None else ws
    check(
        load().dtq_amax(x.data_ptr(), out.data_ptr(), x.numel(), IN_CODE[x.dtype], ws.data_ptr(), ws.numel(), _stream()),
        "dtq_amax",
    )
    return out


@_on_device_of_first_tensor
def amax_static_scratch(x: torch.Tensor, out: torch.Tensor | None = None):
    """amax through the entry point that allocates nothing (scratch inside the library image)."""
    out = torch.empty(1, dtype=torch.float32, device=x.device) if out is None else out
    check(load().dtq_amax_static_scratch(x.data_ptr(), out.data_ptr(), x.numel(), IN_CODE[x.dtype], _stream()),
          "dtq_amax_static_scratch")
    return out


@_on_device_of_first_tensor
def dynamic_scaled_quant(x, out_dtype, out=None, amax_out=None, scale_out=None, ws=None):
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out is None else out
    ws = workspace(x.device) if ws is None else ws
    check(
        load().dtq_dynamic_scaled_quant(x.data_ptr(), out.data_ptr(), _ptr(amax_out), _ptr(scale_out), x.numel(),
                                        IN_CODE[x.dtype], OUT_CODE[out_dtype], ws.data_ptr(), ws.numel(), _stream()),
        "dtq_dynamic_scaled_quant",
    )
    return out


@_on_device_of_first_tensor
def dynamic_scaled_quant_p2p(x, out_dtype, peer_ptrs, rank, epoch, out=None, amax_out=None, scale_out=None, ws=None,
                             spin_limit=0):
    """One launch per GPU of a row-sharded tensor; ``peer_ptrs[r]`` addresses rank r's exchange buffer."""
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out is None else out
    ws = workspace(x.device) if ws is None else ws
    world = len(peer_ptrs)
    ptrs = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
    check(
        load().dtq_dynamic_scaled_quant_p2p(x.data_ptr(), out.data_ptr(), _ptr(amax_out), _ptr(scale_out), x.numel(),
                                            IN_CODE[x.dtype], OUT_CODE[out_dtype], ws.data_ptr(), ws.numel(), ptrs,
                                            rank, world, epoch, spin_limit, _stream()),
        "dtq_dynamic_scaled_quant_p2p",
    )
    return out


@_on_device_of_first_tensor
def cast_with_amax(x, amax_value, out_dtype, out=None, scale_out=None):
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out is None else out
    check(
        load().dtq_cast_with_amax(x.data_ptr(), out.data_ptr(), amax_value.data_ptr(), _ptr(scale_out), x.numel(),
                                  IN_CODE[x.dtype], OUT_CODE[out_dtype], _stream()),
        "dtq_cast_with_amax",
    )
    return out


@_on_device_of_first_tensor
def dynamic_scaled_quant_rowwise(x, out_dtype, out=None, amax_out=None, scale_out=None):
    rows, cols = x.shape
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out is None else out
    check(
        load().dtq_dynamic_scaled_quant_rowwise(x.data_ptr(), out.data_ptr(), _ptr(amax_out), _ptr(scale_out), rows,
                                                cols, IN_CODE[x.dtype], OUT_CODE[out_dtype], _stream()),
        "dtq_dynamic_scaled_quant_rowwise",
    )
    return out


@_on_device_of_first_tensor
def mx_fp8_quantize(x, payload=None, scales=None):
    rows, cols = x.shape
    payload = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device) if payload is None else payload
    scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=x.device) if scales is None else scales
    check(load().dtq_mx_fp8_quantize(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, _stream()),
          "dtq_mx_fp8_quantize")
    return payload, scales


@_on_device_of_first_tensor
def mx_fp8_quantize_blocked(x, payload=None, scales=None):
    """MX cast with the scales in the blocked layout of the consumer GEMM (zero-filled padding)."""
    rows, cols = x.shape
    payload = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device) if payload is None else payload
    if scales is None:
        nbytes = load().dtq_mx_blocked_scale_bytes(rows, cols)
        scales = torch.zeros(nbytes, dtype=torch.uint8, device=x.device).view(torch.float8_e8m0fnu)
    check(load().dtq_mx_fp8_quantize_blocked(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, _stream()),
          "dtq_mx_fp8_quantize_blocked")
    return payload, scales


@_on_device_of_first_tensor
def mx_fp8_quantize_tma(x, payload=None, scales=None, status=None):
    """The shared-memory-staged (TMA bulk copy) variant of the MX cast; same outputs."""
    rows, cols = x.shape
    payload = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device) if payload is None else payload
    scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=x.device) if scales is None else scales
    status = torch.zeros(1, dtype=torch.int32, device=x.device) if status is None else status
    check(load().dtq_mx_fp8_quantize_tma(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols,
                                         status.data_ptr(), _stream()), "dtq_mx_fp8_quantize_tma")
    return payload, scales, status


@_on_device_of_first_tensor
def mx_fp8_quantize_dual(x, payload=None, scales=None, payload_t=None, scales_t=None, blocked=False):
    """MX cast of x and of its transpose from one read of x; ``blocked``: scales in the MX GEMM's layout."""
    rows, cols = x.shape
    e4m3, e8m0 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    payload = torch.empty(rows, cols, dtype=e4m3, device=x.device) if payload is None else payload
    payload_t = torch.empty(cols, rows, dtype=e4m3, device=x.device) if payload_t is None else payload_t
    if blocked:
        L = load()
        if scales is None:
            scales = torch.zeros(L.dtq_mx_blocked_scale_bytes(rows, cols), dtype=torch.uint8, device=x.device).view(e8m0)
        if scales_t is None:
            scales_t = torch.zeros(L.dtq_mx_blocked_scale_bytes(cols, rows), dtype=torch.uint8, device=x.device).view(e8m0)
        check(L.dtq_mx_fp8_quantize_dual_blocked(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), payload_t.data_ptr(),
                                                 scales_t.data_ptr(), rows, cols, _stream()), "dtq_mx_fp8_quantize_dual_blocked")
        return payload, scales, payload_t, scales_t
    scales = torch.empty(rows * (cols // 32), dtype=e8m0, device=x.device) if scales is None else scales
    scales_t = torch.empty(cols * (rows // 32), dtype=e8m0, device=x.device) if scales_t is None else scales_t
    check(load().dtq_mx_fp8_quantize_dual(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), payload_t.data_ptr(),
                                          scales_t.data_ptr(), rows, cols, _stream()), "dtq_mx_fp8_quantize_dual")
    return payload, scales, payload_t, scales_t


@_on_device_of_first_tensor
def saturated_cast_transposed(x, scale, out_dtype, out_t=None, out=None, both=False):
    """The cast of x transposed ([cols, rows]); with ``both`` (or ``out``) also the cast of x itself."""
    rows, cols = x.shape
    out_t = torch.empty(cols, rows, dtype=out_dtype, device=x.device) if out_t is None else out_t
    if both and out is None:
        out = torch.empty(rows, cols, dtype=out_dtype, device=x.device)
    check(load().dtq_saturated_cast_transposed(x.data_ptr(), out.data_ptr() if out is not None else None, out_t.data_ptr(),
                                               scale.data_ptr(), rows, cols, IN_CODE[x.dtype], OUT_CODE[out_dtype],
                                               _stream()), "dtq_saturated_cast_transposed")
    return (out, out_t) if out is not None else out_t


MX_IN_CODE = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}
MX_FMT_CODE = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1, torch.float4_e2m1fn_x2: 2, "e2m1": 2}


@_on_device_of_first_tensor
def mx_quantize(x, elem, payload=None, scales=None, blocked=False):
    """MX block-32 cast of bf16 / fp16 / fp32 to e4m3 / e5m2 (payload [M, N]) or e2m1 (uint8 [M, N/2]);
    ``blocked``: the scales in the MX GEMM's blocked layout (zero-filled padding)."""
    rows, cols = x.shape
    fmt = MX_FMT_CODE[elem]
    if payload is None:
        payload = (torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device) if fmt == 2
                   else torch.empty(rows, cols, dtype=elem, device=x.device))
    if blocked:
        if scales is None:
            nbytes = load().dtq_mx_blocked_scale_bytes(rows, cols)
            scales = torch.zeros(nbytes, dtype=torch.uint8, device=x.device).view(torch.float8_e8m0fnu)
        check(load().dtq_mx_quantize_blocked(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols,
                                             MX_IN_CODE[x.dtype], fmt, _stream()), "dtq_mx_quantize_blocked")
        return payload, scales
    scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=x.device) if scales is None else scales
    check(load().dtq_mx_quantize(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, MX_IN_CODE[x.dtype], fmt,
                                 _stream()), "dtq_mx_quantize")
    return payload, scales


@_on_device_of_first_tensor
def mx_fp8_quantize_amax(x, payload=None, scales=None, amax_out=None, ws=None, peer_ptrs=None, rank=0, epoch=0,
                         spin_limit=0):
    """MX cast + the tensor's amax (>= 0) from one read; with ``peer_ptrs`` the amax is exchanged with the
    other ranks of a row-sharded tensor inside the launch."""
    rows, cols = x.shape
    payload = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device) if payload is None else payload
    scales = torch.empty(rows * (cols // 32), dtype=torch.float8_e8m0fnu, device=x.device) if scales is None else scales
    amax_out = torch.empty(1, dtype=torch.float32, device=x.device) if amax_out is None else amax_out
    ws = workspace(x.device) if ws is None else ws
    if peer_ptrs is None:
        check(load().dtq_mx_fp8_quantize_amax(x.data_ptr(), payload.data_ptr(), scales.data_ptr(), amax_out.data_ptr(),
                                              rows, cols, ws.data_ptr(), ws.numel(), _stream()), "dtq_mx_fp8_quantize_amax")
    else:
        world = len(peer_ptrs)
        ptrs = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
        check(load().dtq_mx_fp8_quantize_amax_p2p(x.data_ptr(), payload.data_ptr(), scales.data_ptr(),
                                                  amax_out.data_ptr(), rows, cols, ws.data_ptr(), ws.numel(), ptrs, rank,
                                                  world, epoch, spin_limit, _stream()), "dtq_mx_fp8_quantize_amax_p2p")
    return payload, scales, amax_out


@_on_device_of_first_tensor
def cast_with_amax_transposed(x, amax_value, out_dtype, out_t=None, out=None, both=False, scale_out=None):
    """The dynamic cast of x transposed ([cols, rows]) for a device-resident amax; with ``both`` (or ``out``)
    also the cast of x itself."""
    rows, cols = x.shape
    out_t = torch.empty(cols, rows, dtype=out_dtype, device=x.device) if out_t is None else out_t
    if both and out is None:
        out = torch.empty(rows, cols, dtype=out_dtype, device=x.device)
    check(load().dtq_cast_with_amax_transposed(x.data_ptr(), out.data_ptr() if out is not None else None, out_t.data_ptr(),
                                               amax_value.data_ptr(), _ptr(scale_out), rows, cols, IN_CODE[x.dtype],
                                               OUT_CODE[out_dtype], _stream()), "dtq_cast_with_amax_transposed")
    return (out, out_t) if out is not None else out_t


@_on_device_of_first_tensor
def dynamic_scaled_quant_dual(x, out_dtype, out=None, out_t=None, amax_out=None, scale_out=None, ws=None):
    """Tensor-wise dynamic quantisation of x into both orientations: (payload [rows, cols], payload_t [cols, rows])."""
    rows, cols = x.shape
    out = torch.empty(rows, cols, dtype=out_dtype, device=x.device) if out is None else out
    out_t = torch.empty(cols, rows, dtype=out_dtype, device=x.device) if out_t is None else out_t
    ws = workspace(x.device) if ws is None else ws
    check(load().dtq_dynamic_scaled_quant_dual(x.data_ptr(), out.data_ptr(), out_t.data_ptr(), _ptr(amax_out), _ptr(scale_out),
                                               rows, cols, IN_CODE[x.dtype], OUT_CODE[out_dtype], ws.data_ptr(), ws.numel(),
                                               _stream()), "dtq_dynamic_scaled_quant_dual")
    return out, out_t


GEMM_KERNELS = {"auto": 0, "pair": 1, "wide": 2, "narrow": 3}


@_on_device_of_first_tensor
def mx_fp8_bf16(a, b_nk, a_scale_blocked, b_scale_blocked, out=None, ws=None, kernel="auto", fp4=False):
    """MX block-scaled GEMM: ``a`` [M, K] e4m3, ``b_nk`` [N, K] e4m3 (the memory of the reference's column-major
    [K, N] operand), blocked E8M0 scales -> bf16 [M, N].  ``fp4``: the operands are packed e2m1 bytes, [M, K/2] and
    [N, K/2].  ``kernel``: "auto", or one of "pair", "wide", "narrow"."""
    m = a.shape[0]
    k = a.shape[1] * (2 if fp4 else 1)
    n = b_nk.shape[0]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device) if out is None else out
    ws = workspace(a.device) if ws is None else ws
    check(load().dtq_mx_gemm_bf16(a.data_ptr(), b_nk.data_ptr(), a_scale_blocked.data_ptr(), b_scale_blocked.data_ptr(),
                                  out.data_ptr(), m, n, k, 2 if fp4 else 0, GEMM_KERNELS[kernel], ws.data_ptr(), ws.numel(),
                                  _stream()), "dtq_mx_gemm_bf16")
    return out


def mx_fp4_bf16(a, b_nk, a_scale_blocked, b_scale_blocked, out=None, ws=None, kernel="auto"):
    """The MXFP4 GEMM: packed e2m1 operands ``a`` [M, K/2], ``b_nk`` [N, K/2] (uint8), blocked E8M0 scales -> bf16."""
    return mx_fp8_bf16(a, b_nk, a_scale_blocked, b_scale_blocked, out=out, ws=ws, kernel=kernel, fp4=True)


@_on_device_of_first_tensor
def rowwise_fp8_bf16(a, b_nk, a_row_scale, b_row_scale, bias=None, out=None, ws=None, kernel="auto"):
    """Row-wise scaled fp8 GEMM: ``a`` [M, K] e4m3 / e5m2, ``b_nk`` [N, K] e4m3, fp32 dequantisation scales [M] and
    [N], optional bias [N] (fp32 or bf16) -> bf16 [M, N]."""
    m, k = a.shape
    n = b_nk.shape[0]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device) if out is None else out
    ws = workspace(a.device) if ws is None else ws
    bias_code = 0 if bias is None or bias.dtype == torch.bfloat16 else 1
    check(load().dtq_rowwise_fp8_bf16(a.data_ptr(), b_nk.data_ptr(), a_row_scale.data_ptr(), b_row_scale.data_ptr(), _ptr(bias),
                                      bias_code, out.data_ptr(), m, n, k, OUT_CODE[a.dtype], GEMM_KERNELS[kernel], ws.data_ptr(),
                                      ws.numel(), _stream()), "dtq_rowwise_fp8_bf16")
    return out
