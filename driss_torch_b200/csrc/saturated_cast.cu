// saturated_cast: out[i] = fp8_satfinite(in[i] * scale) over flat storage.
//
// Replaces the reference's three kernels and their selector (src/saturated_cast.cu:38-57,
// :59-104, :106-153, :168-224) with one persistent, 128-bit-vectorised streaming kernel:
// every warp-wide load instruction reads 512 contiguous bytes, every store writes 256
// (bf16 input) or 128 (fp32 input) contiguous bytes, several loads are in flight per thread,
// and indices are 64-bit.  The arithmetic is the reference's, bit for bit:
//   bf16: scale -> bf16 (RNE); product = one bf16 multiply (mul.bf16x2); bf16 -> fp32 -> fp8.
//   fp32: product = one fp32 multiply; fp32 -> fp8.
#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {
namespace {

constexpr int kUnroll = 2;  // 128-bit loads in flight per thread: 8 KB tiles.  Measured 1 / 2 / 3 / 4 / 8: 2 is the fastest at
                            // every size (48 MB: 11.6 / 9.0 / 9.1 / 9.5 / 9.6 us; 3 GB: 602 / 451 / - / 459 us): the kernel is light
                            // enough that more, shorter-lived blocks keep the memory system busier than longer ones
// Blocks per SM that cap the grid.  The default is "no cap": one tile per block, so the hardware
// block scheduler hands out tiles in address order as SMs free up, which measured about 10%
// faster on B200 than a persistent grid-stride loop (whose blocks run in lock step: load burst,
// then store burst).  The in-kernel loop then only matters beyond 2^31-1 tiles.
constexpr int64_t kBlocksPerSmCap = 1 << 20;
constexpr int kThreads = 256;

// One 16-byte input chunk -> its fp8 bytes, stored with one instruction.
template <int IN, int OUT>
struct Chunk;

template <int OUT>
struct Chunk<DTQ_BF16, OUT> {
  static constexpr int kElems = 8;
  using Scale = __nv_bfloat162;
  __device__ static Scale load_scale(const float *s) { return __float2bfloat162_rn(*s); }
  __device__ static uint32_t pair(uint32_t w, Scale s) {
    const uint32_t p = as_u32(__hmul2(as_bf162(w), s));
    return cvt_fp8x2<OUT>(bf16_lo(p), bf16_hi(p));
  }
  __device__ static void convert_store(uint4 v, Scale s, uint8_t *out, int64_t chunk) {
    uint2 r;
    r.x = pair(v.x, s) | (pair(v.y, s) << 16);
    r.y = pair(v.z, s) | (pair(v.w, s) << 16);
    stg_stream(out + chunk * kElems, r);
  }
  __device__ static uint8_t one(const void *in, int64_t i, Scale s) {
    const __nv_bfloat16 p = __hmul(static_cast<const __nv_bfloat16 *>(in)[i], s.x);
    return cvt_fp8<OUT>(__bfloat162float(p));
  }
};

template <int OUT>
struct Chunk<DTQ_F32, OUT> {
  static constexpr int kElems = 4;
  using Scale = float;
  __device__ static Scale load_scale(const float *s) { return *s; }
  __device__ static void convert_store(uint4 v, Scale s, uint8_t *out, int64_t chunk) {
    const uint32_t r = cvt_fp8x4<OUT>(__fmul_rn(__uint_as_float(v.x), s), __fmul_rn(__uint_as_float(v.y), s),
                                      __fmul_rn(__uint_as_float(v.z), s), __fmul_rn(__uint_as_float(v.w), s));
    stg_stream(out + chunk * kElems, r);
  }
  __device__ static uint8_t one(const void *in, int64_t i, Scale s) {
    return cvt_fp8<OUT>(__fmul_rn(static_cast<const float *>(in)[i], s));
  }
};

template <int IN, int OUT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
saturated_cast_stream(const uint4 *__restrict__ in, uint8_t *__restrict__ out, const float *__restrict__ scale,
                      int64_t numel) {
  using C = Chunk<IN, OUT>;
  // launched so that its blocks may become resident under the tail of the kernel before it on the stream
  // (launch latency and block ramp hidden); nothing is read before that kernel has completed
  pdl_launch_dependents();
  pdl_wait();
  const typename C::Scale s = C::load_scale(scale);
  const int64_t nchunks = numel / C::kElems;
  constexpr int64_t kTile = int64_t(kThreads) * UNROLL;

  for (int64_t tile = blockIdx.x; tile * kTile < nchunks; tile += gridDim.x) {
    const int64_t first = tile * kTile + threadIdx.x;
    uint4 v[UNROLL];
    if ((tile + 1) * kTile <= nchunks) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(in + first + u * kThreads);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) C::convert_store(v[u], s, out, first + u * kThreads);
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (first + u * kThreads < nchunks) v[u] = ldg_stream(in + first + u * kThreads);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (first + u * kThreads < nchunks) C::convert_store(v[u], s, out, first + u * kThreads);
    }
  }
  // The few elements past the last whole chunk.
  if (blockIdx.x == 0) {
    const int64_t i = nchunks * C::kElems + threadIdx.x;
    if (i < numel) out[i] = C::one(in, i, s);
  }
}

// Any alignment, one element per thread per step: only for pointers that are not 16/8-byte aligned.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads)
saturated_cast_scalar(const void *__restrict__ in, uint8_t *__restrict__ out, const float *__restrict__ scale,
                      int64_t numel) {
  using C = Chunk<IN, OUT>;
  const typename C::Scale s = C::load_scale(scale);
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < numel; i += int64_t(gridDim.x) * kThreads)
    out[i] = C::one(in, i, s);
}

template <int IN, int OUT>
int launch(const void *in, void *out, const float *scale, int64_t numel, const DeviceInfo &dev, cudaStream_t st) {
  using C = Chunk<IN, OUT>;
  const int64_t max_grid = int64_t(dev.sm_count) * kBlocksPerSmCap;
  if (aligned_to(in, 16) && aligned_to(out, 8)) {
    const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kThreads) * kUnroll);
    const int grid = balanced_grid(tiles, max_grid);
    return cuda_status(launch_after_dependency(saturated_cast_stream<IN, OUT, kUnroll>, dim3(grid), dim3(kThreads), 0, st,
                                               static_cast<const uint4 *>(in), static_cast<uint8_t *>(out), scale, numel));
  } else {
    const int64_t blocks = ceil_div64(numel, kThreads);
    const int grid = static_cast<int>(blocks < max_grid ? blocks : max_grid);
    saturated_cast_scalar<IN, OUT><<<grid, kThreads, 0, st>>>(in, static_cast<uint8_t *>(out), scale, numel);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_saturated_cast(const void *in, void *out, const float *scale, int64_t numel, int in_dtype,
                                  int out_dtype, void *stream) {
  using namespace dtq;
  if (numel < 0 || !scale || (numel > 0 && (!in || !out))) return DTQ_ERR_INVALID_ARGUMENT;
  if ((in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) || (out_dtype != DTQ_E4M3 && out_dtype != DTQ_E5M2))
    return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (numel == 0) return DTQ_OK;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3 ? launch<DTQ_BF16, DTQ_E4M3>(in, out, scale, numel, dev, st)
                                 : launch<DTQ_BF16, DTQ_E5M2>(in, out, scale, numel, dev, st);
  return out_dtype == DTQ_E4M3 ? launch<DTQ_F32, DTQ_E4M3>(in, out, scale, numel, dev, st)
                               : launch<DTQ_F32, DTQ_E5M2>(in, out, scale, numel, dev, st);
}
