// TEST INFRASTRUCTURE ONLY: binds the unmodified reference CUDA ops under a
// separate dispatcher namespace so they can be loaded next to the product
// library (which owns the `DrissTorch` namespace) and used as ground truth by
// the GPU parity tests and as the "kernel to beat" in the benchmark.
//
// The four functions are the reference's own host entry points, compiled from
// the reference checkout where it lies (see Makefile.ref):
//   src/saturated_cast.cu:227        driss_torch::saturated_cast
//   src/amax.cu:106                  driss_torch::amax
//   src/dynamic_scaled_quant.cu:157  driss_torch::dynamic_scaled_quant
//   src/mx_cast.cu:168               driss_torch::mx_fp8_quantize
// The schema strings repeat src/register_ops.cpp:20-41 under `DrissTorchRef`.
#include <ATen/ATen.h>
#include <c10/core/DispatchKey.h>
#include <torch/library.h>

#include <tuple>

namespace driss_torch {
at::Tensor saturated_cast(const at::Tensor &input, const at::Tensor &scale,
                          at::ScalarType dtype, bool transpose);
at::Tensor amax(const at::Tensor &input);
at::Tensor dynamic_scaled_quant(const at::Tensor &input, at::ScalarType fp8_dtype);
std::tuple<at::Tensor, at::Tensor> mx_fp8_quantize(at::Tensor input, int64_t block_size,
                                                   int64_t axis, bool transpose,
                                                   c10::ScalarType fp8_type);
} // namespace driss_torch

TORCH_LIBRARY(DrissTorchRef, m) {
  m.def("saturated_cast(Tensor input, Tensor scale, ScalarType dtype, bool transpose) -> Tensor");
  m.impl("saturated_cast", c10::DispatchKey::CUDA, TORCH_FN(driss_torch::saturated_cast));
  m.def("amax(Tensor input) -> Tensor");
  m.impl("amax", c10::DispatchKey::CUDA, TORCH_FN(driss_torch::amax));
  m.def("dynamic_scaled_quant(Tensor input, ScalarType dtype) -> Tensor");
  m.impl("dynamic_scaled_quant", c10::DispatchKey::CUDA,
         TORCH_FN(driss_torch::dynamic_scaled_quant));
#ifdef DTQ_REF_WITH_MX
  m.def("mx_fp8_quantize(Tensor input, int block_size, int axis, bool transpose, ScalarType fp8_type) -> (Tensor, Tensor)");
  m.impl("mx_fp8_quantize", c10::DispatchKey::CUDA, TORCH_FN(driss_torch::mx_fp8_quantize));
#endif
}
