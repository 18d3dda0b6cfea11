"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on ``torch.randn`` only (benchmarks/benchmark_saturated_casting.py:80-85)
and publishes no data set; these generators give every configuration a value distribution that
exercises what it is about (outliers for the tensor-wise scale, a wide exponent range for MX
blocks, per-row magnitudes for the row-wise scale).  Values are drawn in fp32 from a
``torch.Generator`` seeded per configuration and cast to bf16.  A CPU generator and a CUDA
generator give different streams, so a comparison must generate once and copy.

Shapes can be overridden (tests use small ones); ``rows``/``cols`` default to the full size.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    rows: int
    cols: int
    seed: int
    what: str


WORKLOADS = {
    "cfg1": Workload("cfg1", 4096, 4096, 1001, "saturated_cast bf16->e4m3, N(0,1), scale=448/amax"),
    "cfg2": Workload("cfg2", 8192, 8192, 1002, "amax + dynamic_scaled_quant bf16, N(0,1) with 0.1% x100 outliers"),
    "cfg3": Workload("cfg3", 16384, 8192, 1003, "mx_fp8_quantize bf16, sign x lognormal(0,3), 1% zeros"),
    "cfg4": Workload("cfg4", 32768, 4096, 1004, "row-wise dynamic quant bf16, rows scaled by 10^U(-3,3)"),
    "cfg5": Workload("cfg5", 262144, 8192, 1005, "row-sharded tensor-wise quant + MX cast bf16, N(0,1) with 0.01% x1000"),
}

CFG5_CHUNK_ROWS = 32768  # cfg5 is defined as 8 row chunks, chunk c seeded seed + c


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_cfg1(rows=None, cols=None, device="cpu") -> torch.Tensor:
    w = WORKLOADS["cfg1"]
    g = _gen(w.seed, device)
    return torch.randn(rows or w.rows, cols or w.cols, generator=g, device=device).to(torch.bfloat16)


def make_cfg2(rows=None, cols=None, device="cpu") -> torch.Tensor:
    w = WORKLOADS["cfg2"]
    g = _gen(w.seed, device)
    shape = (rows or w.rows, cols or w.cols)
    x = torch.randn(shape, generator=g, device=device)
    outlier = torch.rand(shape, generator=g, device=device) < 1e-3
    return torch.where(outlier, x * 100.0, x).to(torch.bfloat16)


def make_cfg3(rows=None, cols=None, device="cpu") -> torch.Tensor:
    """Lognormal magnitudes, random signs, 1 % exact zeros.  On the CPU two calls can differ in the last bit of a few
    elements (``exp`` runs as vector or scalar code depending on where its buffer starts): generate once and hand
    the same tensor to everything that is to be compared.  The same holds for ``make_cfg4`` (``pow``)."""
    w = WORKLOADS["cfg3"]
    g = _gen(w.seed, device)
    shape = (rows or w.rows, cols or w.cols)
    mag = torch.exp(3.0 * torch.randn(shape, generator=g, device=device))
    sign = torch.where(torch.rand(shape, generator=g, device=device) < 0.5, -1.0, 1.0)
    zero = torch.rand(shape, generator=g, device=device) < 0.01
    return torch.where(zero, torch.zeros((), device=device), mag * sign).to(torch.bfloat16)


def make_cfg4(rows=None, cols=None, device="cpu") -> torch.Tensor:
    w = WORKLOADS["cfg4"]
    g = _gen(w.seed, device)
    shape = (rows or w.rows, cols or w.cols)
    x = torch.randn(shape, generator=g, device=device)
    factor = torch.pow(10.0, torch.rand(shape[0], 1, generator=g, device=device) * 6.0 - 3.0)
    return (x * factor).to(torch.bfloat16)


def make_cfg5_chunk(chunk: int, rows: Optional[int] = None, cols: Optional[int] = None, device="cpu") -> torch.Tensor:
    """Row chunk ``chunk`` (of 8) of cfg5; ``rows`` is the chunk height (default 32768)."""
    w = WORKLOADS["cfg5"]
    g = _gen(w.seed + chunk, device)
    shape = (rows or CFG5_CHUNK_ROWS, cols or w.cols)
    x = torch.randn(shape, generator=g, device=device)
    outlier = torch.rand(shape, generator=g, device=device) < 1e-4
    return torch.where(outlier, x * 1000.0, x).to(torch.bfloat16)


def make_cfg5_shard(rank: int, world_size: int, chunk_rows: Optional[int] = None, cols: Optional[int] = None,
                    device="cpu", total_chunks: int = 8) -> torch.Tensor:
    """The rows of cfg5 that ``rank`` of ``world_size`` owns: ``total_chunks / world_size`` whole chunks,
    so the matrix content is the same for every world size that divides ``total_chunks``."""
    if total_chunks % world_size:
        raise ValueError("world_size must divide the number of chunks")
    per = total_chunks // world_size
    parts = [make_cfg5_chunk(c, chunk_rows, cols, device) for c in range(rank * per, (rank + 1) * per)]
    return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)


MAKERS = {"cfg1": make_cfg1, "cfg2": make_cfg2, "cfg3": make_cfg3, "cfg4": make_cfg4}


def tensor_scale(x: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """cfg1's tensor-wise fp32 scale ``fp8_max / max(amax, 1e-12)`` as a [1] tensor on ``x.device``."""
    amax = x.abs().max().to(torch.float64).clamp_min(1e-12)
    return (torch.finfo(fp8_dtype).max / amax).to(torch.float32).reshape(1)
