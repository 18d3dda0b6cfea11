"""The host-buffer path (GPU): matrices in pinned host memory in, quantised outputs in host memory
out, chunked over copy and compute streams, several matrices in flight.  Every output must equal
the CPU oracle's result on the whole matrix, byte for byte."""
import pytest
import torch

from conftest import as_bytes
from driss_torch_b200 import workloads
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu
E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


def _host_outputs(rows, cols, fp8_dtype):
    return (torch.empty(rows, cols, dtype=fp8_dtype, pin_memory=True), torch.empty(rows, cols, dtype=E4M3, pin_memory=True),
            torch.empty(rows * cols // 32, dtype=torch.float8_e8m0fnu, pin_memory=True))


@pytest.mark.parametrize("rows,chunk_rows,depth", [(1024, 256, 1), (1000, 384, 2), (96, 4096, 2), (2048, 128, 3)])
@pytest.mark.parametrize("fp8_dtype", [E4M3, E5M2])
def test_matrices_in_flight_equal_the_oracle(rows, chunk_rows, depth, fp8_dtype):
    from driss_torch_b200.host_pipeline import HostQuantizer

    cols = 512
    hq = HostQuantizer(rows, cols, "cuda", chunk_rows=chunk_rows, fp8_dtype=fp8_dtype, depth=depth)
    # different data per matrix (different amax), more matrices than slots, outputs per matrix
    xs = [(workloads.make_cfg2(rows=rows, cols=cols).float() * (0.25 * (k + 1))).to(torch.bfloat16).pin_memory()
          for k in range(depth + 2)]
    xs[1][rows // 2, 17] = 3e4  # the amax sits in a late chunk
    outs = [_host_outputs(rows, cols, fp8_dtype) for _ in xs]
    tickets = [hq.submit(x, *o) for x, o in zip(xs, outs)]
    results = []
    for t in tickets:
        amax, scale = hq.wait(t)
        results.append((amax.item(), scale.item()))
    # amax / scale tensors belong to the slot: read right after each wait only while the slot is not reused;
    # with more matrices than slots the early ones were overwritten, so only the payloads are checked for those
    for k, (x, (p, mp, ms)) in enumerate(zip(xs, outs)):
        want, want_amax, want_scale = qo.dynamic_scaled_quant(x, fp8_dtype)
        want_mp, want_ms = qo.mx_fp8_quantize(x)
        assert torch.equal(as_bytes(p), as_bytes(want)), f"matrix {k}: tensor-wise payload"
        assert torch.equal(as_bytes(mp), as_bytes(want_mp)), f"matrix {k}: MX payload"
        assert torch.equal(as_bytes(ms), as_bytes(want_ms)), f"matrix {k}: MX scales"
    want, want_amax, want_scale = qo.dynamic_scaled_quant(xs[-1], fp8_dtype)
    assert results[-1] == (want_amax.item(), want_scale.item())
    # run() = submit + wait, and its amax / scale are current
    amax, scale = hq.run(xs[0], *outs[0])
    want, want_amax, want_scale = qo.dynamic_scaled_quant(xs[0], fp8_dtype)
    assert (amax.item(), scale.item()) == (want_amax.item(), want_scale.item())
    assert torch.equal(as_bytes(outs[0][0]), as_bytes(want))
    assert hq.launches == 3 * hq.nchunks + 1


def test_constructor_rejects_bad_arguments():
    from driss_torch_b200.host_pipeline import HostQuantizer

    with pytest.raises(ValueError):
        HostQuantizer(64, 48, "cuda")
    with pytest.raises(ValueError):
        HostQuantizer(64, 64, "cuda", depth=0)
