// mx_fp8_quantize: bf16 -> (e4m3 payload, one E8M0 scale per 32 consecutive elements).
//
// Replaces src/mx_cast.cu:44-86, :96-161 (a 128x32 tile per CTA through shared memory, one
// element per thread, 16 block-wide syncs).  Because blocks run along the contiguous last
// dimension and cols % 32 == 0, the matrix is a flat array of 64-byte blocks, so this is a
// pure stream: each lane loads 16 bytes (8 elements), four neighbouring lanes form one MX
// block and agree on its exponent with two shuffles, each lane stores its 8 payload bytes
// with one instruction, and a warp emits the 32 scale bytes of the 2 KB it covered as one
// contiguous 32-byte store.  Nothing is staged in shared memory and there are no block syncs.
//
// Arithmetic (identical to the reference): e_i = ceil(log2 |x_i|) from the exponent field
// (+1 if the mantissa is non-zero; zero -> -128, subnormal -> -126); E = max e_i;
// biased = clamp(E - 8 + 127, 0, 255); scale = 2^(biased-127) (0.0 for biased == 0, +inf for
// 255); payload = e4m3_satfinite(x * (1/scale)); scale byte = ue8m0(scale) rounded up,
// saturating (255 -> 0xFE).  e is monotone in |x|, so the block max is taken on the raw
// 15-bit magnitudes with packed 16-bit integer max.
#include "dtq_host.h"
#include "mx_common.cuh"

namespace dtq {
namespace {

// Grid cap in blocks per SM; the default is "no cap" (one tile per block), see saturated_cast.cu.
constexpr int64_t kBlocksPerSmCap = 1 << 20;
constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // tied to the scale-byte mapping below: lane&3 picks the iteration

// nchunks = numel / 8 is a multiple of 4.  A warp owns kUnroll consecutive 512-byte rows of
// chunks; a CTA tile is kThreads * kUnroll chunks.
template <bool BLOCKED>
__global__ void __launch_bounds__(kThreads, 2048 / kThreads)
mx_stream_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
                 int64_t nchunks, int64_t kblocks, int64_t katoms) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int64_t kTile = int64_t(kThreads) * kUnroll;
  // may have become resident under the tail of the kernel before it on the stream: wait for that kernel
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t tile = blockIdx.x; tile * kTile < nchunks; tile += gridDim.x) {
    const int64_t warp_first = tile * kTile + int64_t(warp) * (32 * kUnroll);
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t c = warp_first + u * 32 + lane;
      v[u] = c < nchunks ? ldg_stream(in + c) : make_uint4(0, 0, 0, 0);
    }
    uint32_t my_scale_byte = 0;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      uint32_t mag = chunk_absmax_bits(v[u]);
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 1));
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 2));
      const int biased = block_biased_exponent(mag);
      const float inv = inverse_scale(biased);
      const int64_t c = warp_first + u * 32 + lane;
      if (c < nchunks) stg_stream(payload + c * 8, mx_payload(v[u], inv));
      if ((lane & 3) == u) my_scale_byte = mx_scale_byte(biased);
    }
    // lane = 4*k + j holds the scale of block (u = j, quad k): block index u*8 + k in the warp's span.
    const int64_t blk = warp_first / 4 + (lane & 3) * 8 + (lane >> 2);
    if (blk * 4 < nchunks) scales[scale_offset<BLOCKED>(blk, kblocks, katoms)] = static_cast<uint8_t>(my_scale_byte);
  }
}

// Any alignment: one thread per MX block.
template <bool BLOCKED>
__global__ void __launch_bounds__(kThreads)
mx_scalar_kernel(const uint16_t *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
                 int64_t nblocks, int64_t kblocks, int64_t katoms) {
  for (int64_t b = int64_t(blockIdx.x) * kThreads + threadIdx.x; b < nblocks; b += int64_t(gridDim.x) * kThreads) {
    const uint16_t *x = in + b * 32;
    uint32_t mag = 0;
    for (int i = 0; i < 32; ++i) mag = max(mag, uint32_t(x[i]) & 0x7FFFu);
    const int biased = block_biased_exponent(mag);
    const float scale = __int_as_float(biased << 23);
    const float inv = __frcp_rn(scale);
    for (int i = 0; i < 32; ++i)
      payload[b * 32 + i] = cvt_fp8<DTQ_E4M3>(__fmul_rn(__uint_as_float(uint32_t(x[i]) << 16), inv));
    scales[scale_offset<BLOCKED>(b, kblocks, katoms)] = cvt_ue8m0(scale);
  }
}

}  // namespace
}  // namespace dtq

namespace dtq {
namespace {
template <bool BLOCKED>
int launch_mx(const void *in_bf16, void *payload, void *scales_e8m0, int64_t rows, int64_t cols, cudaStream_t st) {
  if (rows < 0 || cols < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (cols % 32 != 0) return DTQ_ERR_SHAPE;
  const int64_t numel = rows * cols;
  if (numel == 0) return DTQ_OK;
  if (!in_bf16 || !payload || !scales_e8m0 || !aligned_to(in_bf16, 2)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  const int64_t kblocks = cols / 32, katoms = (kblocks + 3) / 4;
  const int64_t max_grid = int64_t(dev.sm_count) * kBlocksPerSmCap;
  if (aligned_to(in_bf16, 16) && aligned_to(payload, 8)) {
    const int64_t nchunks = numel / 8;
    const int64_t tiles = ceil_div64(nchunks, int64_t(kThreads) * kUnroll);
    const int grid = balanced_grid(tiles, max_grid);
    return cuda_status(launch_after_dependency(mx_stream_kernel<BLOCKED>, dim3(grid), dim3(kThreads), 0, st,
                                               static_cast<const uint4 *>(in_bf16), static_cast<uint8_t *>(payload),
                                               static_cast<uint8_t *>(scales_e8m0), nchunks, kblocks, katoms));
  } else {
    const int64_t blocks = ceil_div64(numel / 32, kThreads);
    const int grid = static_cast<int>(blocks < max_grid ? blocks : max_grid);
    mx_scalar_kernel<BLOCKED><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t *>(in_bf16),
                                                         static_cast<uint8_t *>(payload),
                                                         static_cast<uint8_t *>(scales_e8m0), numel / 32, kblocks, katoms);
  }
  return cuda_status(cudaGetLastError());
}
}  // namespace
}  // namespace dtq

extern "C" int dtq_mx_fp8_quantize(const void *in_bf16, void *payload, void *scales_e8m0, int64_t rows, int64_t cols,
                                   void *stream) {
  return dtq::launch_mx<false>(in_bf16, payload, scales_e8m0, rows, cols, static_cast<cudaStream_t>(stream));
}

extern "C" size_t dtq_mx_blocked_scale_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>((cols / 32 + 3) / 4) * 512;
}

extern "C" int dtq_mx_fp8_quantize_blocked(const void *in_bf16, void *payload, void *scales_blocked, int64_t rows,
                                           int64_t cols, void *stream) {
  return dtq::launch_mx<true>(in_bf16, payload, scales_blocked, rows, cols, static_cast<cudaStream_t>(stream));
}
