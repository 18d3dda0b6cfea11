"""Pins the plain-C oracle (CPU only) against golden outputs of the unmodified reference CUDA
kernels, recorded on a B200 by tests/golden/make_golden.py."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import GOLDEN, assert_fp8_equal
from oracle import quant_oracle as qo

_spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

FIXTURE = GOLDEN / "reference_kernels.npz"
CASES = make_golden.cases()


@pytest.fixture(scope="module")
def golden():
    assert FIXTURE.exists(), f"{FIXTURE} is missing: regenerate it with tests/golden/make_golden.py on a GPU box"
    return np.load(FIXTURE)


def test_fixture_covers_every_case(golden):
    names = set(golden.files)
    for name, op, _ in CASES:
        if op == "mx_fp8_quantize":
            assert name + "__payload" in names and name + "__scales" in names
        else:
            assert name in names


@pytest.mark.parametrize("name,op,args", CASES, ids=[c[0] for c in CASES])
def test_oracle_reproduces_reference_kernel(golden, name, op, args):
    if op == "saturated_cast":
        x, s, dt = args
        want = torch.from_numpy(golden[name]).view(dt)
        assert_fp8_equal(qo.saturated_cast(x, s, dt), want, dt, name)
    elif op == "dynamic_scaled_quant":
        x, dt = args
        want = torch.from_numpy(golden[name]).view(dt)
        got, _, _ = qo.dynamic_scaled_quant(x, dt)
        assert_fp8_equal(got, want, dt, name)
        # the definition used for bf16 input: same arithmetic on float(x)
        if bool((x.to(torch.bfloat16).float() == x).all()):
            got16, _, _ = qo.dynamic_scaled_quant(x.to(torch.bfloat16), dt)
            assert_fp8_equal(got16, want, dt, name + " (bf16 input)")
    elif op == "amax":
        want = torch.from_numpy(golden[name])
        assert qo.amax(args[0]).view(torch.int32).item() == want.view(torch.int32).item()
    else:
        p, s = qo.mx_fp8_quantize(args[0])
        assert_fp8_equal(p, torch.from_numpy(golden[name + "__payload"]).view(torch.float8_e4m3fn), torch.float8_e4m3fn, name)
        assert np.array_equal(s.view(torch.uint8).numpy(), golden[name + "__scales"]), name + " scales"
