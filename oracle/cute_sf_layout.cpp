// TEST INFRASTRUCTURE ONLY.  Evaluates, on the host, the scale-factor layout that the reference's
// MX GEMM hands to CUTLASS (src/mx_fp8_bf16.cu:97-110: Sm1xxBlkScaledConfig::tile_atom_to_shape_SFA
// on the problem shape), using the CUTLASS headers vendored in the image, and prints the offset
// of every (row, k-block) scale.  The tests compare the kernel's blocked layout with this table.
//
// Build: g++ -std=c++17 -O1 -I<cutlass>/include oracle/cute_sf_layout.cpp -o oracle/_build/cute_sf_layout
// Usage: cute_sf_layout M K   ->  "cosize <n>" then M*(K/32) lines "row kblock offset"
#include <cstdio>
#include <cstdlib>

#include <cute/tensor.hpp>
#include <cutlass/detail/sm100_blockscaled_layout.hpp>

int main(int argc, char **argv) {
  using namespace cute;
  if (argc < 3) return 2;
  const int M = std::atoi(argv[1]), K = std::atoi(argv[2]);
  using Config = cutlass::detail::Sm1xxBlockScaledConfig<32>;
  auto layout = Config::tile_atom_to_shape_SFA(make_shape(M, 128, K, 1));
  std::printf("cosize %lld\n", static_cast<long long>(cosize(layout)));
  for (int r = 0; r < M; ++r)
    for (int kb = 0; kb < K / 32; ++kb)
      std::printf("%d %d %lld\n", r, kb, static_cast<long long>(layout(r, kb * 32, 0)));
  return 0;
}
