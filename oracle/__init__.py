"""TEST INFRASTRUCTURE ONLY.

CPU checkers for the quantization path.  Nothing under this package is part of
the product: only the tests, the smoke check and the benchmark's CPU-baseline
legs may import it.

* ``quant_oracle`` -- ctypes front end of the plain-C restatement
  (``quant_oracle.c``) of the reference CUDA kernels' arithmetic.
* ``eager`` -- the PyTorch-eager formulas the reference's own tests compare
  against (test/test_sat_cast.py:7-24, test/test_amax.py:6-7), for CPU tensors.
* ``cute_sf_layout.cpp`` -- CUTLASS's own blocked scale-factor layout evaluated on the host
  (pins the index map of the blocked MX scales).
* ``_ref/`` -- (built by ``Makefile.ref``) the unmodified reference CUDA ops,
  bound under ``torch.ops.DrissTorchRef`` by ``ref_binding.cpp``.
"""
