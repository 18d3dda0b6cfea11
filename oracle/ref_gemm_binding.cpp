// TEST INFRASTRUCTURE ONLY: binds the unmodified reference MX GEMMs under their own dispatcher
// namespace, in a library of their own, so that the benchmark can time "the kernel to beat" next to
// the product's and the tests can compare results with it.
//
// The two functions are the reference's own host entry points, compiled from the reference checkout
// where it lies (see Makefile.ref, target `gemm`):
//   src/mx_fp8_bf16.cu:217   driss_torch::mx_fp8_bf16
//   src/mx_fp8_bf16.cu:243   driss_torch::mx_fp4_bf16
// The schema strings repeat src/register_ops.cpp:35-38 under `DrissTorchRefGemm`.
//
// The reference instantiates a CUTLASS collective on a 2x1 thread-block cluster; that library is
// therefore kept out of every multi-GPU run of this repository (the ignore list for such runs names it) and is only
// ever given this GPU's own memory.
#include <ATen/ATen.h>
#include <c10/core/DispatchKey.h>
#include <torch/library.h>

namespace driss_torch {
at::Tensor mx_fp8_bf16(at::Tensor a, at::Tensor b, at::Tensor a_scale, at::Tensor b_scale);
at::Tensor mx_fp4_bf16(at::Tensor a, at::Tensor b, at::Tensor a_scale, at::Tensor b_scale);
} // namespace driss_torch

TORCH_LIBRARY(DrissTorchRefGemm, m) {
  m.def("mx_fp8_bf16(Tensor a, Tensor b, Tensor a_scale, Tensor b_scale) -> Tensor");
  m.impl("mx_fp8_bf16", c10::DispatchKey::CUDA, TORCH_FN(driss_torch::mx_fp8_bf16));
  m.def("mx_fp4_bf16(Tensor a, Tensor b, Tensor a_scale, Tensor b_scale) -> Tensor");
  m.impl("mx_fp4_bf16", c10::DispatchKey::CUDA, TORCH_FN(driss_torch::mx_fp4_bf16));
}
