"""Generates ``reference_kernels.npz``: outputs of the UNMODIFIED reference CUDA kernels
(built by oracle/Makefile.ref, bound as torch.ops.DrissTorchRef) on deterministic inputs.

Run on a machine with a B200 and the reference checkout built:

    make -f oracle/Makefile.ref && python tests/golden/make_golden.py [out.npz]

``cases()`` is also imported by tests/test_oracle_golden.py, which rebuilds the same
inputs on CPU and checks the plain-C oracle against the stored outputs, so only outputs
are stored.  Inputs are integer-pattern or seeded-CPU-generator tensors.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
SAT_SCALES = [1.0, 0.3330078125, 448.0 / 5.21875, 57344.0, 3.0e-5]


def all_bf16() -> torch.Tensor:
    return torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).view(256, 256)


def finite_bf16() -> torch.Tensor:
    """Every finite bf16 value (NaN and inf patterns replaced by 1.0), for ops whose NaN handling is unpinned."""
    x = all_bf16().clone()
    bad = ~torch.isfinite(x.float())
    x[bad] = 1.0
    return x


def rand_f32(seed: int, shape, lo=0.0, hi=1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=g) * (hi - lo) + lo


def randn_f32(seed: int, shape) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g)


def mx_inputs():
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    fin = bits.clone()
    fin[~torch.isfinite(fin.float())] = 0.5
    g = torch.Generator().manual_seed(4)
    lognorm = (torch.exp(3.0 * torch.randn(256, 256, generator=g)) * torch.where(torch.rand(256, 256, generator=g) < 0.5, -1.0, 1.0))
    zeros = torch.zeros(128, 64)
    zeros[:, 32:] = 2.0**-121
    return {
        "mx_dense_patterns": fin.view(128, 512),
        "mx_shuffled_patterns": fin[torch.randperm(65536, generator=g)].view(128, 512),
        "mx_lognormal": lognorm.to(torch.bfloat16),
        "mx_rand": rand_f32(5, (256, 128)).to(torch.bfloat16),
        "mx_zero_and_tiny_blocks": zeros.to(torch.bfloat16),
    }


def cases():
    """(name, op, args) for every golden case; tensors are CPU tensors."""
    out = []
    for kname, dt in FP8.items():
        for i, s in enumerate(SAT_SCALES):
            out.append((f"sat_bf16_all_{kname}_s{i}", "saturated_cast", (all_bf16(), s, dt)))
        out.append((f"sat_f32_rand_{kname}", "saturated_cast", (rand_f32(1, (128, 512), -600.0, 600.0), 0.9, dt)))
        out.append((f"sat_f32_wide_{kname}", "saturated_cast", (randn_f32(2, (128, 512)) * 3.0e4, 1.7, dt)))
        out.append((f"dsq_f32_rand_{kname}", "dynamic_scaled_quant", (rand_f32(3, (128, 512)), dt)))
        out.append((f"dsq_f32_randn_{kname}", "dynamic_scaled_quant", (randn_f32(6, (256, 384)) * 17.0, dt)))
        out.append((f"dsq_f32_bf16vals_{kname}", "dynamic_scaled_quant", (finite_bf16().float(), dt)))
    out.append(("amax_bf16_randn", "amax", (randn_f32(7, (512, 4097 - 1)).to(torch.bfloat16),)))
    out.append(("amax_f32_randn", "amax", (randn_f32(8, (64, 3212)),)))
    out.append(("amax_bf16_finite_patterns", "amax", (finite_bf16(),)))
    for name, x in mx_inputs().items():
        out.append((name, "mx_fp8_quantize", (x,)))
    return out


def main() -> None:
    dst = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE / "reference_kernels.npz"
    torch.ops.load_library(str(ROOT / "oracle" / "_ref" / "libdriss_torch_ref.so"))
    ref = torch.ops.DrissTorchRef
    blobs = {}
    for name, op, args in cases():
        if op == "saturated_cast":
            x, s, dt = args
            y = ref.saturated_cast(x.cuda(), torch.tensor([s], dtype=torch.float32, device="cuda"), dt, False)
            blobs[name] = y.view(torch.uint8).cpu().numpy()
        elif op == "dynamic_scaled_quant":
            x, dt = args
            blobs[name] = ref.dynamic_scaled_quant(x.cuda(), dt).view(torch.uint8).cpu().numpy()
        elif op == "amax":
            blobs[name] = ref.amax(args[0].cuda()).cpu().numpy()
        elif op == "mx_fp8_quantize":
            p, s = ref.mx_fp8_quantize(args[0].cuda(), 32, 1, False, torch.float8_e4m3fn)
            blobs[name + "__payload"] = p.view(torch.uint8).cpu().numpy()
            blobs[name + "__scales"] = s.view(torch.uint8).cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(dst, **blobs)
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(blobs)} arrays) on {torch.cuda.get_device_name(0)}")


if __name__ == "__main__":
    main()
