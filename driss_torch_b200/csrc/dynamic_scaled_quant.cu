// Tensor-wise dynamic quantisation: amax -> scale -> fp8 cast.
//
//   amax = max |x| (>= 0);  scale_d = fp8_max / ((double)amax + 1e-12);
//   out[i] = fp8_satfinite((float)(scale_d * (double)x[i]))
//
// which is the arithmetic of the reference's cooperative kernel
// (src/dynamic_scaled_quant.cu:83-118), restated for bf16 and fp32 inputs.
//
// dtq_dynamic_scaled_quant is one cooperative launch of a persistent grid:
//   phase 1  every block streams its tiles (128-bit loads, several in flight), keeps its LAST
//            tile in registers, and publishes a partial max;
//   finish   the last-arriving block reduces the partials, writes amax / scale and releases
//            a generation word; the others wait on it with a bounded spin;
//   phase 2  every block converts the tile it kept, then walks its remaining tiles in REVERSE
//            order, so the most recently read part of the tensor is re-read while it is still
//            in the 126 MB L2.
// The reference reads the tensor twice with scalar loads, writes single bytes and needs a
// separate memset launch for its scratch.
//
// dtq_cast_with_amax is phase 2 alone for an amax that already sits in device memory (the
// sharded path: local amax -> max all-reduce -> cast).
#include <atomic>
#include <cmath>

#include "dtq_device.cuh"
#include "dtq_grid.cuh"
#include "dtq_host.h"

namespace dtq {

// from amax.cu
template <int IN>
struct AbsMax;
int64_t head_elems(const void *p, int elem_bytes, int64_t numel);

namespace {

#ifndef DTQ_DSQ_UNROLL
#define DTQ_DSQ_UNROLL 4
#endif
#ifndef DTQ_DSQ_COOP
#define DTQ_DSQ_COOP 1
#endif
#ifndef DTQ_DSQ_THREADS
#define DTQ_DSQ_THREADS 256
#endif
// Grid cap of the stand-alone cast kernel; default "no cap" (one tile per block), see saturated_cast.cu.
#ifndef DTQ_CAST_BLOCKS_PER_SM
#define DTQ_CAST_BLOCKS_PER_SM (1 << 20)
#endif
constexpr int kThreads = DTQ_DSQ_THREADS;

// ---- per-chunk arithmetic ----------------------------------------------------------------------
template <int IN, int OUT>
struct DsqChunk;

template <int OUT>
struct DsqChunk<DTQ_BF16, OUT> {
  static constexpr int kElems = 8;
  static constexpr int kElemBytes = 2;
  static constexpr int kOutAlign = 8;
  __device__ static void convert_store(uint4 v, const DsqScale &s, uint8_t *out, int64_t chunk) {
    stg_stream(out + chunk * kElems, dsq_convert_bf16x8<OUT>(v, s));
  }
  __device__ static float load_one(const void *in, int64_t i) {
    return __uint_as_float(uint32_t(static_cast<const uint16_t *>(in)[i]) << 16);
  }
  __device__ static void absmax(float &a, float &b, uint4 v) {
    // packed |x| and max on bf16 pairs, NaNs dropped
    __nv_bfloat162 m = __hmax2(as_bf162(v.x & 0x7FFF7FFFu), as_bf162(v.y & 0x7FFF7FFFu));
    __nv_bfloat162 n = __hmax2(as_bf162(v.z & 0x7FFF7FFFu), as_bf162(v.w & 0x7FFF7FFFu));
    m = __hmax2(m, n);
    a = fmaxf(a, __bfloat162float(m.x));
    b = fmaxf(b, __bfloat162float(m.y));
  }
};

template <int OUT>
struct DsqChunk<DTQ_F32, OUT> {
  static constexpr int kElems = 4;
  static constexpr int kElemBytes = 4;
  static constexpr int kOutAlign = 4;
  __device__ static void convert_store(uint4 v, const DsqScale &s, uint8_t *out, int64_t chunk) {
    stg_stream(out + chunk * kElems, dsq_convert_f32x4<OUT>(v, s));
  }
  __device__ static float load_one(const void *in, int64_t i) { return static_cast<const float *>(in)[i]; }
  __device__ static void absmax(float &a, float &b, uint4 v) {
    a = fmaxf(a, fmaxf(fabsf(__uint_as_float(v.x)), fabsf(__uint_as_float(v.y))));
    b = fmaxf(b, fmaxf(fabsf(__uint_as_float(v.z)), fabsf(__uint_as_float(v.w))));
  }
};

// ---- fused single launch -------------------------------------------------------------------------
// Requires `in` 16-byte aligned and `out` aligned for the packed store; numel may be anything
// (block 0 handles the elements past the last whole chunk).
template <int IN, int OUT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
dsq_fused_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ out, float *__restrict__ amax_out,
                 float *__restrict__ scale_out, int64_t numel, Workspace *ws) {
  using C = DsqChunk<IN, OUT>;
  __shared__ float smem32[32];
  __shared__ int flag;
  unsigned int gen0 = 0;
  if (threadIdx.x == 0) gen0 = ld_acquire(&ws->generation);

  const int64_t nchunks = numel / C::kElems;
  constexpr int64_t kTile = int64_t(kThreads) * UNROLL;
  const int64_t ntiles = (nchunks + kTile - 1) / kTile;
  const int64_t tail0 = nchunks * C::kElems;

  // phase 1
  float a = 0.0f, b = 0.0f;
  uint4 v[UNROLL];
  int64_t tile = blockIdx.x;
  int64_t last_tile = -1;
  for (; tile < ntiles; tile += gridDim.x) {
    const int64_t first = tile * kTile + threadIdx.x;
    if ((tile + 1) * kTile <= nchunks) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(in + first + u * kThreads);
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        v[u] = (first + u * kThreads < nchunks) ? ldg_stream(in + first + u * kThreads) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) C::absmax(a, b, v[u]);
    last_tile = tile;
  }
  if (blockIdx.x == 0 && tail0 + threadIdx.x < numel) a = fmaxf(a, fabsf(C::load_one(in, tail0 + threadIdx.x)));

  // finish
  const float block_value = block_max_nonneg(fmaxf(a, b), smem32, 0.0f);
  if (publish_and_ticket(ws, block_value, &flag)) {
    const float total = reduce_partials(ws, smem32, 0.0f);
    if (threadIdx.x == 0) {
      ws->amax = total;
      if (amax_out) *amax_out = total;
      if (scale_out) *scale_out = static_cast<float>(dsq_scale<OUT>(total));
      ws->arrivals = 0;
      __threadfence();
      atomicAdd(&ws->generation, 1u);
    }
    __syncthreads();
  } else if (!wait_generation(ws, gen0, &flag)) {
    return;  // status word says why; nothing more is written
  }
  const float amax = ld_relaxed_f32(&ws->amax);
  const DsqScale sd = make_dsq_scale<OUT>(amax);

  // phase 2: the kept tile from registers, the rest newest-first
  if (last_tile >= 0) {
    const int64_t first = last_tile * kTile + threadIdx.x;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (first + u * kThreads < nchunks) C::convert_store(v[u], sd, out, first + u * kThreads);
    for (tile = last_tile - gridDim.x; tile >= 0; tile -= gridDim.x) {
      const int64_t f = tile * kTile + threadIdx.x;  // always a whole tile
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(in + f + u * kThreads);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) C::convert_store(v[u], sd, out, f + u * kThreads);
    }
  }
  if (blockIdx.x == 0 && tail0 + threadIdx.x < numel)
    out[tail0 + threadIdx.x] = cvt_fp8<OUT>(dsq_mul(sd.sd, C::load_one(in, tail0 + threadIdx.x)));
}

// ---- cast phase alone ---------------------------------------------------------------------------------
template <int IN, int OUT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
cast_with_amax_stream(const uint4 *__restrict__ in, uint8_t *__restrict__ out, const float *__restrict__ amax_p,
                      float *__restrict__ scale_out, int64_t numel) {
  using C = DsqChunk<IN, OUT>;
  const float amax = fmaxf(*amax_p, 0.0f);
  const DsqScale sd = make_dsq_scale<OUT>(amax);
  if (scale_out && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = static_cast<float>(sd.sd);
  const int64_t nchunks = numel / C::kElems;
  constexpr int64_t kTile = int64_t(kThreads) * UNROLL;
  for (int64_t tile = blockIdx.x; tile * kTile < nchunks; tile += gridDim.x) {
    const int64_t first = tile * kTile + threadIdx.x;
    uint4 v[UNROLL];
    if ((tile + 1) * kTile <= nchunks) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(in + first + u * kThreads);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) C::convert_store(v[u], sd, out, first + u * kThreads);
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (first + u * kThreads < nchunks) C::convert_store(ldg_stream(in + first + u * kThreads), sd, out,
                                                             first + u * kThreads);
    }
  }
  const int64_t tail0 = nchunks * C::kElems;
  if (blockIdx.x == 0 && tail0 + threadIdx.x < numel)
    out[tail0 + threadIdx.x] = cvt_fp8<OUT>(dsq_mul(sd.sd, C::load_one(in, tail0 + threadIdx.x)));
}

template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads)
cast_with_amax_scalar(const void *__restrict__ in, uint8_t *__restrict__ out, const float *__restrict__ amax_p,
                      float *__restrict__ scale_out, int64_t numel) {
  using C = DsqChunk<IN, OUT>;
  const double sd = dsq_scale<OUT>(fmaxf(*amax_p, 0.0f));
  if (scale_out && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = static_cast<float>(sd);
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < numel; i += int64_t(gridDim.x) * kThreads)
    out[i] = cvt_fp8<OUT>(dsq_mul(sd, C::load_one(in, i)));
}

// Unaligned inputs to the fused op: |x| max of any-alignment data into ws->amax (one block per
// grid slot, last-block finish), followed by the scalar cast.
template <int IN>
__global__ void __launch_bounds__(kThreads)
amax_scalar_kernel(const void *__restrict__ in, int64_t numel, float *__restrict__ amax_out, Workspace *ws) {
  __shared__ float smem32[32];
  __shared__ int flag;
  float a = 0.0f;
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < numel; i += int64_t(gridDim.x) * kThreads) {
    const float x = IN == DTQ_BF16 ? __uint_as_float(uint32_t(static_cast<const uint16_t *>(in)[i]) << 16)
                                   : static_cast<const float *>(in)[i];
    a = fmaxf(a, fabsf(x));
  }
  const float block_value = block_max_nonneg(a, smem32, 0.0f);
  if (publish_and_ticket(ws, block_value, &flag)) {
    const float total = reduce_partials(ws, smem32, 0.0f);
    if (threadIdx.x == 0) {
      ws->amax = total;
      if (amax_out) *amax_out = total;
      ws->arrivals = 0;
    }
  }
}

// Largest grid the cooperative launch accepts for this kernel on this device, cached.
template <typename Kernel>
int coop_grid_limit(Kernel kernel, const DeviceInfo &dev, std::atomic<int> *cache) {
  int dev_id = 0;
  if (cudaGetDevice(&dev_id) != cudaSuccess) return 0;
  int v = cache[dev_id & 63].load(std::memory_order_relaxed);
  if (v == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess) return 0;
    v = per_sm * dev.sm_count;
    if (v > kMaxGridBlocks) v = kMaxGridBlocks;
    cache[dev_id & 63].store(v, std::memory_order_relaxed);
  }
  return v;
}

template <int IN, int OUT>
int launch_fused(const void *in, void *out, float *amax_out, float *scale_out, int64_t numel, Workspace *ws,
                 const DeviceInfo &dev, cudaStream_t st) {
  using C = DsqChunk<IN, OUT>;
  uint8_t *o = static_cast<uint8_t *>(out);
  if (aligned_to(in, 16) && aligned_to(out, C::kOutAlign) && dev.cooperative) {
    static std::atomic<int> cache[64];
    auto kernel = dsq_fused_kernel<IN, OUT, DTQ_DSQ_UNROLL>;
    const int limit = coop_grid_limit(kernel, dev, cache);
    if (limit <= 0) return DTQ_ERR_CUDA_BASE + static_cast<int>(cudaErrorLaunchFailure);
    const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kThreads) * DTQ_DSQ_UNROLL);
    const int grid = balanced_grid(tiles, limit);
    const uint4 *in4 = static_cast<const uint4 *>(in);
    void *args[] = {&in4, &o, &amax_out, &scale_out, &numel, &ws};
#if DTQ_DSQ_COOP
    DTQ_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kernel), dim3(grid), dim3(kThreads), args, 0, st));
    return DTQ_OK;
#else
    kernel<<<grid, kThreads, 0, st>>>(in4, o, amax_out, scale_out, numel, ws);
    return cuda_status(cudaGetLastError());
#endif
  }
  const int64_t blocks = ceil_div64(numel, kThreads);
  const int64_t max_grid = int64_t(dev.sm_count) * 8;
  const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks < max_grid ? blocks : max_grid));
  amax_scalar_kernel<IN><<<grid, kThreads, 0, st>>>(in, numel, amax_out, ws);
  cast_with_amax_scalar<IN, OUT><<<grid, kThreads, 0, st>>>(in, o, &ws->amax, scale_out, numel);
  return cuda_status(cudaGetLastError());
}

template <int IN, int OUT>
int launch_cast(const void *in, void *out, const float *amax, float *scale_out, int64_t numel, const DeviceInfo &dev,
                cudaStream_t st) {
  using C = DsqChunk<IN, OUT>;
  uint8_t *o = static_cast<uint8_t *>(out);
  const int64_t max_grid = int64_t(dev.sm_count) * DTQ_CAST_BLOCKS_PER_SM;
  if (aligned_to(in, 16) && aligned_to(out, C::kOutAlign)) {
    const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kThreads) * DTQ_DSQ_UNROLL);
    const int grid = balanced_grid(tiles, max_grid);
    cast_with_amax_stream<IN, OUT, DTQ_DSQ_UNROLL><<<grid, kThreads, 0, st>>>(static_cast<const uint4 *>(in), o, amax,
                                                                             scale_out, numel);
  } else {
    const int64_t blocks = ceil_div64(numel, kThreads);
    const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks < max_grid ? blocks : max_grid));
    cast_with_amax_scalar<IN, OUT><<<grid, kThreads, 0, st>>>(in, o, amax, scale_out, numel);
  }
  return cuda_status(cudaGetLastError());
}

int check_dtypes(int in_dtype, int out_dtype) {
  if ((in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) || (out_dtype != DTQ_E4M3 && out_dtype != DTQ_E5M2))
    return DTQ_ERR_UNSUPPORTED_DTYPE;
  return DTQ_OK;
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_dynamic_scaled_quant(const void *in, void *out, float *amax_out, float *scale_out, int64_t numel,
                                        int in_dtype, int out_dtype, void *workspace, size_t workspace_bytes,
                                        void *stream) {
  using namespace dtq;
  if (numel < 0 || (numel > 0 && (!in || !out))) return DTQ_ERR_INVALID_ARGUMENT;
  if (int e = check_dtypes(in_dtype, out_dtype)) return e;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  if (numel > 0 && !aligned_to(in, in_dtype == DTQ_BF16 ? 2 : 4)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace *ws = static_cast<Workspace *>(workspace);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3
               ? launch_fused<DTQ_BF16, DTQ_E4M3>(in, out, amax_out, scale_out, numel, ws, dev, st)
               : launch_fused<DTQ_BF16, DTQ_E5M2>(in, out, amax_out, scale_out, numel, ws, dev, st);
  return out_dtype == DTQ_E4M3 ? launch_fused<DTQ_F32, DTQ_E4M3>(in, out, amax_out, scale_out, numel, ws, dev, st)
                               : launch_fused<DTQ_F32, DTQ_E5M2>(in, out, amax_out, scale_out, numel, ws, dev, st);
}

extern "C" int dtq_cast_with_amax(const void *in, void *out, const float *amax, float *scale_out, int64_t numel,
                                  int in_dtype, int out_dtype, void *stream) {
  using namespace dtq;
  if (numel < 0 || !amax || (numel > 0 && (!in || !out))) return DTQ_ERR_INVALID_ARGUMENT;
  if (int e = check_dtypes(in_dtype, out_dtype)) return e;
  if (numel > 0 && !aligned_to(in, in_dtype == DTQ_BF16 ? 2 : 4)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3 ? launch_cast<DTQ_BF16, DTQ_E4M3>(in, out, amax, scale_out, numel, dev, st)
                                 : launch_cast<DTQ_BF16, DTQ_E5M2>(in, out, amax, scale_out, numel, dev, st);
  return out_dtype == DTQ_E4M3 ? launch_cast<DTQ_F32, DTQ_E4M3>(in, out, amax, scale_out, numel, dev, st)
                               : launch_cast<DTQ_F32, DTQ_E5M2>(in, out, amax, scale_out, numel, dev, st);
}
