"""dtq_amax_static_scratch (GPU): the amax entry point for callers that are not allowed to
allocate device memory.

Such callers exist: a host runtime whose own pool owns the whole device heap and that forbids
cudaMalloc inside plugins, or a latency-critical section that cannot take the device-wide
synchronisation cudaMalloc / cudaFree imply.  For them the reduction's scratch is a fixed
array inside the library image instead of a caller-provided workspace.

The check is against the ordinary entry point, bit for bit, on two calls in a row (the array
keeps the previous call's contents, so the second call is the interesting one), and that an
input larger than the array can serve is rejected before anything is launched.  This file is
collected last so that a failure here cannot hide a failure anywhere else; it must also pass
when run on its own in a fresh process (its first call does the per-device address look-up).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().cpu().view(torch.int32).item()


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float32])
def test_two_calls_in_a_row_match_the_workspace_entry_point(in_dtype):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(20)
    first = (torch.randn(2048, 4096, generator=g) * 3.0).to(in_dtype).cuda()
    second = (torch.randn(777, 1031, generator=g) * 0.01).to(in_dtype).cuda()  # ragged, smaller maximum
    out = torch.full((1,), -7.0, device="cuda")
    from oracle import quant_oracle as qo

    for x in (first, second):
        want = _cabi.amax(x)                       # existing entry point, caller-provided workspace
        got = _cabi.amax_static_scratch(x, out=out)  # new entry point, nothing allocated by the library
        torch.cuda.synchronize()
        assert _bits(got) == _bits(want), f"{tuple(x.shape)} {in_dtype}"
        assert _bits(got) == _bits(qo.amax(x.cpu())), "against the CPU restatement of the reference kernel"
    # and once more on the first input: the array now holds the second call's partials
    assert _bits(_cabi.amax_static_scratch(first, out=out)) == _bits(_cabi.amax(first))


def test_empty_input_and_specials():
    from driss_torch_b200 import _cabi

    assert _cabi.amax_static_scratch(torch.zeros(1, 0, dtype=torch.bfloat16, device="cuda")).item() == -float("inf")
    x = torch.tensor([[1.0, float("nan"), -2.5, 0.0]], device="cuda")
    assert _cabi.amax_static_scratch(x).item() == 2.5


def test_inputs_beyond_the_array_are_rejected_without_a_launch():
    from driss_torch_b200 import _cabi

    lib = _cabi.load()
    limit_bytes = 256 * 1024 * 1024  # DTQ_AMAX_STATIC_MAX_BYTES
    x = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.full((1,), 5.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # one element more than fits: refused with DTQ_ERR_TOO_LARGE (6); `out` is left untouched
    assert lib.dtq_amax_static_scratch(x.data_ptr(), out.data_ptr(), limit_bytes // 2 + 1, _cabi.BF16, stream) == 6
    assert lib.dtq_amax_static_scratch(x.data_ptr(), out.data_ptr(), limit_bytes // 4 + 1, _cabi.F32, stream) == 6
    torch.cuda.synchronize()
    assert out.item() == 5.0
    assert b"exceeds" in lib.dtq_status_string(6)
    # exactly at the limit is accepted
    big = torch.zeros(limit_bytes // 2, dtype=torch.bfloat16, device="cuda").view(1, -1)
    big[0, -1] = -9.0
    assert _cabi.amax_static_scratch(big, out=out).item() == 9.0
