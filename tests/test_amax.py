"""amax parity (GPU) on the reference test's grid (test/test_amax.py:10-19) and beyond."""
import pytest
import torch

from conftest import IN_DTYPES
from driss_torch_b200 import workloads
from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().cpu().view(torch.int32).item()


@pytest.mark.parametrize("num_rows", [4, 64, 512, 4096])
@pytest.mark.parametrize("num_cols", [7, 17, 127, 512, 3212, 4097])
@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_amax(num_rows, num_cols, in_dtype):
    import driss_torch_b200 as dt
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(num_rows * 31 + num_cols)
    a = torch.randn(num_rows, num_cols, generator=g).to(in_dtype)
    want = qo.amax(a)
    eager = a.abs().max().to(torch.float32).reshape(1)  # the reference test's expectation
    assert _bits(want) == _bits(eager)
    ad = a.cuda()
    got = _cabi.amax(ad)
    assert got.shape == (1,) and got.dtype == torch.float32
    assert _bits(got) == _bits(want)
    assert _bits(dt.amax(ad)) == _bits(want)
    # repeated calls reuse the workspace and must keep working
    assert _bits(_cabi.amax(ad)) == _bits(want)


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
def test_position_of_the_maximum(in_dtype):
    from driss_torch_b200 import _cabi

    n = 1 << 20
    for pos in (0, 1, 7, 8, 4095, 4096, n // 2 + 3, n - 9, n - 1):
        a = torch.zeros(1, n, dtype=in_dtype)
        a[0, pos] = -3.5
        assert _cabi.amax(a.cuda()).item() == 3.5, pos


@pytest.mark.parametrize("in_dtype", IN_DTYPES)
@pytest.mark.parametrize("numel", [1, 2, 3, 7, 8, 9, 17, 4095, 4097, 1_000_003])
def test_ragged_and_misaligned(in_dtype, numel):
    from driss_torch_b200 import _cabi

    g = torch.Generator().manual_seed(numel)
    base = torch.randn(numel + 8, generator=g).to(in_dtype)
    for off in (0, 1, 3):
        a = base[off : off + numel].view(1, numel)
        got = _cabi.amax(a.cuda()[:, :] if off == 0 else base.cuda()[off : off + numel].view(1, numel))
        assert _bits(got) == _bits(qo.amax(a.contiguous())), (numel, off)


def test_specials():
    from driss_torch_b200 import _cabi

    # NaNs are dropped (src/amax.cu:60-65), infinities win, an all-NaN or empty input gives -inf
    a = torch.tensor([[1.0, float("nan"), -2.0, 0.5]])
    for dt_ in IN_DTYPES:
        assert _cabi.amax(a.to(dt_).cuda()).item() == 2.0
        assert _cabi.amax(torch.tensor([[1.0, -float("inf")]]).to(dt_).cuda()).item() == float("inf")
        assert _cabi.amax(torch.full((1, 64), float("nan")).to(dt_).cuda()).item() == -float("inf")
        assert _cabi.amax(torch.zeros(1, 0).to(dt_).cuda()).item() == -float("inf")
        assert _bits(_cabi.amax(torch.full((2, 64), -0.0).to(dt_).cuda())) == 0  # +0.0
        sub = torch.tensor([[1e-40, -3e-40]], dtype=torch.float32).to(dt_)
        assert _bits(_cabi.amax(sub.cuda())) == _bits(qo.amax(sub))


def test_cfg2_shape_distribution():
    from driss_torch_b200 import _cabi

    a = workloads.make_cfg2(rows=1024, cols=8192)
    assert _bits(_cabi.amax(a.cuda())) == _bits(qo.amax(a))


def test_non_contiguous_and_errors():
    import driss_torch_b200 as dt

    a = torch.randn(128, 96, device="cuda").to(torch.bfloat16)
    want = a.abs().max().float().item()
    assert dt.amax(a.t()).item() == want  # dense: reduced over storage
    assert dt.amax(a[::2, 5:]).item() == a[::2, 5:].abs().max().float().item()
    with pytest.raises(RuntimeError):
        dt.amax(a.view(-1))
    with pytest.raises(RuntimeError):
        dt.amax(a.half())
    for backend in ("aot_eager", "inductor"):  # the reference compiles with the default backend
        torch._dynamo.reset()
        fn = torch.compile(dt.amax, fullgraph=True, backend=backend)
        assert fn(a).item() == want
