"""``import driss_torch`` for existing callers of the reference's quantization ops.

The reference package is called ``driss_torch`` (driss_torch/__init__.py:1-47,:114-122); the
B200 implementation lives in ``driss_torch_b200``.  This package re-exports it under the
reference's name, so ``driss_torch.saturated_cast`` / ``amax`` / ``dynamic_scaled_quant`` /
``mx_fp8_quantize`` keep working unchanged, with the same ``torch.ops.DrissTorch`` operators
behind them.  The reference's GEMM and RNG wrappers are not part of this path and are absent.
"""
from driss_torch_b200 import *  # noqa: F401,F403
from driss_torch_b200 import __all__, lib_path, ops  # noqa: F401
