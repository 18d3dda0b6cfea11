"""CPU-only checks of the boundary and the host logic: the C-ABI library loads without a GPU
and exports everything the public header declares; argument validation that needs no
device; the op registrations and fake implementations; row sharding; workload generators."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "dtq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dtq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from driss_torch_b200 import _cabi

    lib = _cabi.load()
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/dtq_b200.h but not exported"
        assert name in _cabi.SIGNATURES, f"{name} has no ctypes prototype"
    assert set(_cabi.SIGNATURES) == set(names)


def test_version_status_strings_and_workspace_size():
    from driss_torch_b200 import _cabi

    lib = _cabi.load()
    assert b"sm_100a" in lib.dtq_version()
    assert lib.dtq_status_string(0) == b"ok"
    for code in range(1, 7):
        assert lib.dtq_status_string(code) not in (b"ok", b"unknown status")
    assert lib.dtq_workspace_bytes() >= 4096 and lib.dtq_workspace_bytes() % 256 == 0


def test_argument_validation_before_any_device_work():
    from driss_torch_b200 import _cabi

    lib = _cabi.load()
    one = ctypes.c_void_p(256)  # never dereferenced: these calls must fail on the checks before it
    assert lib.dtq_saturated_cast(one, one, one, -1, 0, 0, None) == 1
    assert lib.dtq_saturated_cast(one, one, None, 8, 0, 0, None) == 1
    assert lib.dtq_saturated_cast(one, one, one, 8, 2, 0, None) == 2
    assert lib.dtq_saturated_cast(one, one, one, 8, 0, 5, None) == 2
    assert lib.dtq_saturated_cast(one, one, one, 0, 0, 0, None) == 0  # empty: nothing to do
    assert lib.dtq_amax(one, one, 8, 0, None, 0, None) == 4
    assert lib.dtq_amax(one, one, 8, 0, one, 16, None) == 4
    assert lib.dtq_amax(one, None, 8, 0, one, 1 << 20, None) == 1
    assert lib.dtq_dynamic_scaled_quant(one, one, None, None, 8, 0, 0, None, 0, None) == 4
    assert lib.dtq_dynamic_scaled_quant(one, one, None, None, 8, 3, 0, one, 1 << 20, None) == 2
    assert lib.dtq_cast_with_amax(one, one, None, None, 8, 0, 0, None) == 1
    assert lib.dtq_mx_fp8_quantize(one, one, one, 4, 48, None) == 3
    assert lib.dtq_mx_fp8_quantize(one, one, one, 0, 64, None) == 0
    assert lib.dtq_mx_fp8_quantize(None, one, one, 4, 64, None) == 1
    assert lib.dtq_dynamic_scaled_quant_rowwise(one, one, None, None, 4, 0, 0, 0, None) == 3
    # the added entry points
    assert lib.dtq_saturated_cast_transposed(one, None, one, None, 4, 4, 0, 0, None) == 1   # no scale
    assert lib.dtq_saturated_cast_transposed(one, None, one, one, 4, 4, 5, 0, None) == 2
    assert lib.dtq_saturated_cast_transposed(one, None, None, one, 4, 4, 0, 0, None) == 1   # no transposed output
    assert lib.dtq_saturated_cast_transposed(one, None, one, one, 0, 4, 0, 0, None) == 0
    assert lib.dtq_mx_quantize(one, one, one, 4, 64, 3, 0, None) == 2
    assert lib.dtq_mx_quantize(one, one, one, 4, 64, 0, 3, None) == 2
    assert lib.dtq_mx_quantize(one, one, one, 4, 48, 0, 2, None) == 3
    assert lib.dtq_mx_quantize(one, None, one, 4, 64, 2, 2, None) == 1
    assert lib.dtq_mx_quantize(one, one, one, 0, 64, 1, 1, None) == 0
    for fn in (lib.dtq_mx_fp8_quantize_dual, lib.dtq_mx_fp8_quantize_dual_blocked):
        assert fn(one, one, one, one, one, 48, 64, None) == 3   # rows not a multiple of 32
        assert fn(one, one, one, one, one, 64, 48, None) == 3
        assert fn(one, one, one, None, one, 64, 64, None) == 1
        assert fn(one, one, one, one, one, 0, 64, None) == 0
    assert lib.dtq_mx_fp8_quantize_amax(one, one, one, one, 4, 64, None, 0, None) == 4      # no workspace
    assert lib.dtq_mx_fp8_quantize_amax(one, one, one, None, 4, 64, one, 1 << 20, None) == 1  # no amax output
    assert lib.dtq_mx_fp8_quantize_amax(one, one, one, one, 4, 48, one, 1 << 20, None) == 3
    assert lib.dtq_mx_fp8_quantize_amax_p2p(one, one, one, one, 4, 64, one, 1 << 20, None, 0, 1, 1, 0, None) == 1
    ptrs = (ctypes.c_void_p * 2)(256, 512)
    assert lib.dtq_mx_fp8_quantize_amax_p2p(one, one, one, one, 4, 64, one, 1 << 20, ptrs, 2, 2, 1, 0, None) == 1  # rank
    assert lib.dtq_mx_fp8_quantize_amax_p2p(one, one, one, one, 4, 64, one, 1 << 20, ptrs, 0, 17, 1, 0, None) == 1  # world
    assert lib.dtq_dynamic_scaled_quant_rowwise(one, one, None, None, 0, 16, 0, 0, None) == 0
    assert lib.dtq_dynamic_scaled_quant_rowwise(one, one, None, None, 4, 16, 9, 0, None) == 2
    assert lib.dtq_workspace_init(None, 0, None) == 4


def test_ops_are_registered_with_the_reference_schemas():
    import driss_torch_b200  # noqa: F401

    def schema(name):
        return str(getattr(torch.ops.DrissTorch, name).default._schema)

    assert schema("saturated_cast") == (
        "DrissTorch::saturated_cast(Tensor input, Tensor scale, ScalarType dtype, bool transpose) -> Tensor")
    assert schema("amax") == "DrissTorch::amax(Tensor input) -> Tensor"
    assert schema("dynamic_scaled_quant") == "DrissTorch::dynamic_scaled_quant(Tensor input, ScalarType dtype) -> Tensor"
    assert schema("mx_fp8_quantize") == (
        "DrissTorch::mx_fp8_quantize(Tensor input, int block_size, int axis, bool transpose, ScalarType fp8_type)"
        " -> (Tensor, Tensor)")


def test_no_cpu_kernel_no_fallback():
    import driss_torch_b200 as dt

    a = torch.zeros(4, 32, dtype=torch.bfloat16)
    s = torch.ones(1)
    with pytest.raises(NotImplementedError):
        dt.saturated_cast(a, s, torch.float8_e4m3fn)
    with pytest.raises(NotImplementedError):
        dt.amax(a)
    with pytest.raises(NotImplementedError):
        dt.dynamic_scaled_quant(a, torch.float8_e4m3fn)
    with pytest.raises((NotImplementedError, RuntimeError)):
        dt.mx_fp8_quantize(a)


def test_fake_implementations():
    import driss_torch_b200 as dt

    x = torch.empty(256, 128, dtype=torch.bfloat16, device="meta")
    s = torch.empty(1, dtype=torch.float32, device="meta")
    y = dt.saturated_cast(x, s, torch.float8_e5m2)
    assert y.shape == x.shape and y.dtype == torch.float8_e5m2
    assert dt.saturated_cast(x.t(), s, torch.float8_e5m2).stride() == x.t().stride()
    assert dt.amax(x).shape == (1,) and dt.amax(x).dtype == torch.float32
    assert dt.dynamic_scaled_quant(x, torch.float8_e4m3fn).dtype == torch.float8_e4m3fn
    p, sc = dt.mx_fp8_quantize(x)
    assert p.shape == x.shape and p.dtype == torch.float8_e4m3fn
    assert sc.shape == (256 * 4,) and sc.dtype == torch.float8_e8m0fnu
    p, am, scale = dt.dynamic_scaled_quant_with_scale(x, torch.float8_e4m3fn)
    assert am.shape == (1,) and scale.shape == (1,)
    p, am, scale = dt.dynamic_scaled_quant_rowwise(x, torch.float8_e4m3fn)
    assert p.shape == x.shape and am.shape == (256, 1) and scale.shape == (256, 1)
    p, scale = dt.cast_with_amax(x, s, torch.float8_e4m3fn)
    assert p.shape == x.shape and scale.shape == (1,)
    # the additions
    e8m0 = torch.float8_e8m0fnu
    p, sc = dt.mx_fp8_quantize_blocked(x)
    assert p.shape == x.shape and sc.dtype == e8m0 and sc.numel() == 2 * 1 * 512
    p, sc, p_t, sc_t = dt.mx_fp8_quantize_dual(x)
    assert p.shape == (256, 128) and p_t.shape == (128, 256) and sc.shape == (1024,) and sc_t.shape == (1024,)
    assert p_t.dtype == torch.float8_e4m3fn and sc_t.dtype == e8m0
    p, sc, am = dt.mx_fp8_quantize_with_amax(x)
    assert p.shape == x.shape and sc.shape == (1024,) and am.shape == (1,) and am.dtype == torch.float32
    p4, sc = dt.mx_fp4_quantize(x)
    assert p4.shape == (256, 64) and p4.dtype == torch.uint8 and sc.shape == (1024,)
    p5, sc = dt.mx_fp8_quantize(x.float(), ScalarType=torch.float8_e5m2)
    assert p5.dtype == torch.float8_e5m2 and p5.shape == x.shape
    y_t = dt.saturated_cast_transposed(x, s, torch.float8_e4m3fn)
    assert y_t.shape == (128, 256) and y_t.dtype == torch.float8_e4m3fn
    p, p_t, scale = dt.cast_with_amax_dual(x, s, torch.float8_e4m3fn)
    assert p.shape == (256, 128) and p_t.shape == (128, 256) and scale.shape == (1,)
    p, p_t, am, scale = dt.dynamic_scaled_quant_dual(x, torch.float8_e5m2)
    assert p_t.shape == (128, 256) and p_t.dtype == torch.float8_e5m2 and am.shape == (1,) and scale.shape == (1,)
    y, y_t = dt.saturated_cast_dual(x, s, torch.float8_e5m2)
    assert y.shape == (256, 128) and y_t.shape == (128, 256) and y.dtype == torch.float8_e5m2


def test_python_surface_matches_the_reference_wrappers():
    import inspect

    import driss_torch_b200 as dt

    assert list(inspect.signature(dt.saturated_cast).parameters) == ["x", "scale", "out_dtype", "transpose"]
    assert inspect.signature(dt.saturated_cast).parameters["transpose"].default is False
    assert list(inspect.signature(dt.amax).parameters) == ["x"]
    assert list(inspect.signature(dt.dynamic_scaled_quant).parameters) == ["inpt", "dtype"]
    sig = inspect.signature(dt.mx_fp8_quantize)
    assert list(sig.parameters) == ["input", "block_size", "axis", "transpose", "ScalarType"]
    assert [p.default for p in sig.parameters.values()][1:] == [32, 1, False, torch.float8_e4m3fn]
    with pytest.raises(AssertionError):
        dt.saturated_cast(torch.zeros(2, 2), torch.ones(1), torch.float8_e4m3fn, transpose=True)


@pytest.mark.parametrize("rows,world,multiple", [(262144, 8, 128), (262144, 1, 128), (1000, 3, 128), (5, 8, 1),
                                                  (0, 4, 128), (129, 2, 128), (4096, 4, 32), (7, 7, 1)])
def test_shard_rows_partitions_exactly(rows, world, multiple):
    from driss_torch_b200.sharded import shard_rows

    spans = [shard_rows(rows, world, r, multiple) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == rows
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [b - a for a, b in spans]
    assert sum(sizes) == rows
    for a, b in spans:
        if b < rows:
            assert (b - a) % multiple == 0 and a % multiple == 0
    nonzero = [s for s in sizes if s]
    if nonzero:
        assert max(nonzero) - min(nonzero) < 2 * multiple
    with pytest.raises(ValueError):
        shard_rows(rows, world, world, multiple)


def test_workload_generators_are_deterministic_and_shaped_as_described():
    from driss_torch_b200 import workloads as w

    a, b = w.make_cfg2(rows=256, cols=512), w.make_cfg2(rows=256, cols=512)
    assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    assert a.abs().max().item() > 50  # outliers x100 present
    c3 = w.make_cfg3(rows=256, cols=512)
    assert 0.002 < (c3 == 0).float().mean().item() < 0.03
    assert c3.abs().max().item() > 1e3 and (c3 < 0).any() and (c3 > 0).any()
    c4 = w.make_cfg4(rows=512, cols=64)
    row_max = c4.float().abs().amax(dim=1)
    assert row_max.max().item() / row_max.min().item() > 1e3
    s0 = w.make_cfg5_shard(0, 1, chunk_rows=16, cols=64, total_chunks=4)
    parts = torch.cat([w.make_cfg5_shard(r, 2, chunk_rows=16, cols=64, total_chunks=4) for r in range(2)])
    assert s0.shape == (64, 64) and torch.equal(s0, parts)
    with pytest.raises(ValueError):
        w.make_cfg5_shard(0, 3, chunk_rows=16, cols=64, total_chunks=4)
    assert set(w.WORKLOADS) == {"cfg1", "cfg2", "cfg3", "cfg4", "cfg5"}
    sc = w.tensor_scale(w.make_cfg1(rows=64, cols=64), torch.float8_e4m3fn)
    assert sc.shape == (1,) and sc.dtype == torch.float32


def test_the_reference_package_name_resolves_to_the_same_ops():
    # existing callers write `import driss_torch` (driss_torch/__init__.py in the reference)
    import driss_torch
    import driss_torch.abstract_impls  # noqa: F401  (the module name the reference's library declares)
    import driss_torch_b200 as dt

    for name in ("saturated_cast", "amax", "dynamic_scaled_quant", "mx_fp8_quantize", "mx_cast"):
        assert getattr(driss_torch, name) is getattr(dt, name)
    assert driss_torch.ops is torch.ops.DrissTorch
