import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"
REF_LIB = ROOT / "oracle" / "_ref" / "libdriss_torch_ref.so"

FP8_DTYPES = [torch.float8_e4m3fn, torch.float8_e5m2]
IN_DTYPES = [torch.bfloat16, torch.float32]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def as_bytes(t: torch.Tensor) -> torch.Tensor:
    """fp8 / e8m0 tensor -> uint8 CPU tensor of its bytes."""
    return t.detach().contiguous().view(torch.uint8).cpu()


def assert_fp8_equal(got: torch.Tensor, want: torch.Tensor, fp8_dtype=None, what: str = ""):
    """Byte equality, except that any NaN encoding matches any other NaN encoding."""
    g, w = as_bytes(got), as_bytes(want)
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} != {tuple(w.shape)}"
    diff = g != w
    if diff.any() and fp8_dtype is not None:
        gn = g.view(fp8_dtype).float().isnan()
        wn = w.view(fp8_dtype).float().isnan()
        diff = diff & ~(gn & wn)
    if diff.any():
        idx = diff.flatten().nonzero().flatten()[:8].tolist()
        gf, wf = g.flatten(), w.flatten()
        detail = ", ".join(f"[{i}] got 0x{int(gf[i]):02x} want 0x{int(wf[i]):02x}" for i in idx)
        raise AssertionError(f"{what}: {int(diff.sum())} of {g.numel()} bytes differ: {detail}")


@pytest.fixture(scope="session")
def ref_ops():
    """The unmodified reference CUDA ops (torch.ops.DrissTorchRef), if they were built."""
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref not built (make -f oracle/Makefile.ref)")
    torch.ops.load_library(str(REF_LIB))
    return torch.ops.DrissTorchRef


@pytest.fixture(scope="session")
def ref_gemm_ops():
    """The unmodified reference MX GEMMs (torch.ops.DrissTorchRefGemm: the reference's CUTLASS instantiations built
    from its own source), if they were built.  That library never travels with a multi-GPU run."""
    lib = REF_LIB.parent / "libdriss_torch_ref_gemm.so"
    if not lib.exists():
        pytest.skip("oracle/_ref/libdriss_torch_ref_gemm.so not built (make -f oracle/Makefile.ref gemm)")
    torch.ops.load_library(str(lib))
    return torch.ops.DrissTorchRefGemm
