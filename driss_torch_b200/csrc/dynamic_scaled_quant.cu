// Tensor-wise dynamic quantisation: amax -> scale -> fp8 cast.
//
//   amax = max |x| (>= 0);  scale_d = fp8_max / ((double)amax + 1e-12);
//   out[i] = fp8_satfinite((float)(scale_d * (double)x[i]))
//
// which is the arithmetic of the reference's cooperative kernel
// (src/dynamic_scaled_quant.cu:83-118), restated for bf16 and fp32 inputs.
//
// dtq_dynamic_scaled_quant is one cooperative launch of a persistent grid (block b owns tiles
// b, b+G, b+2G, ...).  The tensor-wise dependency forces a second look at every element; the
// kernel makes as little of that second look as possible come from HBM:
//   phase 1  each block keeps its FIRST tile in registers and its next few tiles in shared
//            memory (filled through the registers the max is taken from), then streams the rest;
//   finish   every block folds its maximum into one word with an atomic max and takes a ticket;
//            all wait, with a bounded spin, until the ticket count reaches the grid size;
//   phase 2  each block converts its streamed tiles newest-first, so the re-read starts with
//            what L2 still holds (about 50 MB on B200, measured), with the next tile's loads in
//            flight while the current one is converted and stored; then the tiles it kept in
//            shared memory and registers, which cost no memory traffic at all.
// Keeping the OLDEST tiles on chip matters: L2 retains the most recently read lines, and those
// must be lines phase 2 will actually ask for.
// The reference reads the tensor twice from HBM with scalar loads, writes single bytes and needs
// a separate memset launch for its scratch.
//
// dtq_cast_with_amax is phase 2 alone for an amax that already sits in device memory (the
// sharded path: local amax -> max all-reduce -> cast).
#include <atomic>
#include <cmath>
#include <mutex>

#include "dtq_device.cuh"
#include "dtq_grid.cuh"
#include "dtq_host.h"

namespace dtq {

// from amax.cu
int launch_amax(const void *in, float *out, int64_t numel, int in_dtype, Workspace *ws, const DeviceInfo &dev,
                cudaStream_t st);

namespace {

constexpr int kUnroll = 4;  // 128-bit loads in flight per thread, all kernels of this file
// The fused kernel: threads per block, resident blocks per SM it is sized for, and how many
// tiles (of kFusedThreads * kUnroll 16-byte chunks) a block keeps in shared memory at most.
constexpr int kFusedThreads = 512;
constexpr int kFusedBlocksPerSm = 2;
constexpr int kFusedSmemTiles = 3;
// A block's first tile stays in registers across the barrier: one more tile kept on chip for
// 4 * kUnroll registers per thread.
constexpr int kFusedRegTiles = 1;
// Inputs above this many bytes are quantised as amax kernel + cast kernel instead of the single
// fused launch: what the chip can keep between the two looks (about 140 MB) no longer matters at
// that size, and the two stream kernels run at higher occupancy than the persistent fused one
// (measured at 512 MiB: 199 us against 209 us; at 128 MiB the fused launch wins 48 us to 60 us).
constexpr int64_t kFusedMaxBytes = int64_t(320) << 20;
// The stand-alone cast kernel: one tile per block (no grid cap), see saturated_cast.cu.
constexpr int kThreads = 256;
constexpr int64_t kCastBlocksPerSmCap = 1 << 20;

// ---- per-chunk arithmetic ----------------------------------------------------------------------
// BOUNDED: |x| <= amax is guaranteed (amax was computed from the same data in this launch).
template <int IN, int OUT, bool BOUNDED = false>
struct DsqChunk;

template <int OUT, bool BOUNDED>
struct DsqChunk<DTQ_BF16, OUT, BOUNDED> {
  static constexpr int kElems = 8;
  static constexpr int kElemBytes = 2;
  static constexpr int kOutAlign = 8;
  __device__ static void convert_store(uint4 v, const DsqScale &s, uint8_t *out, int64_t chunk) {
    stg_stream(out + chunk * kElems, dsq_convert_bf16x8<OUT, BOUNDED>(v, s));
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

template <int OUT, bool BOUNDED>
struct DsqChunk<DTQ_F32, OUT, BOUNDED> {
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
// (block 0 handles the elements past the last whole chunk).  Dynamic shared memory holds
// `smem_tiles` tiles.
// Phase 1 loads the newest kFusedL2KeepMB of the tiles it cannot keep on chip with an L2 evict_last
// policy, so that they survive the rest of the streaming traffic until phase 2 comes back for them (newest
// first).  Measured on B200, 128 MiB input: 53.2 us without the hint, 52.6 / 50.9 / 50.0 / 49.3 us with
// 32 / 48 / 64 / 80 MB, 49.8 us with every streamed tile marked (more than L2 holds: the marked lines evict
// each other).
constexpr int64_t kFusedL2KeepMB = 80;

template <int UNROLL>
__device__ __forceinline__ void load_tile(uint4 (&v)[UNROLL], const uint4 *__restrict__ in, int64_t tile,
                                          int64_t nchunks) {
  constexpr int64_t kTile = int64_t(kFusedThreads) * UNROLL;
  const int64_t first = tile * kTile + threadIdx.x;
  if ((tile + 1) * kTile <= nchunks) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(in + first + u * kFusedThreads);
  } else {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      v[u] = (first + u * kFusedThreads < nchunks) ? ldg_stream(in + first + u * kFusedThreads) : make_uint4(0, 0, 0, 0);
  }
}

// The same with an L2 eviction policy on every load.
template <int UNROLL>
__device__ __forceinline__ void load_tile_hint(uint4 (&v)[UNROLL], const uint4 *__restrict__ in, int64_t tile,
                                               int64_t nchunks, uint64_t policy) {
  constexpr int64_t kTile = int64_t(kFusedThreads) * UNROLL;
  const int64_t first = tile * kTile + threadIdx.x;
#pragma unroll
  for (int u = 0; u < UNROLL; ++u)
    v[u] = (first + u * kFusedThreads < nchunks) ? ldg_stream_hint(in + first + u * kFusedThreads, policy)
                                                 : make_uint4(0, 0, 0, 0);
}

template <typename C, int UNROLL>
__device__ __forceinline__ void store_tile(const uint4 (&v)[UNROLL], const DsqScale &sd, uint8_t *__restrict__ out,
                                           int64_t tile, int64_t nchunks) {
  constexpr int64_t kTile = int64_t(kFusedThreads) * UNROLL;
  const int64_t first = tile * kTile + threadIdx.x;
  if ((tile + 1) * kTile <= nchunks) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) C::convert_store(v[u], sd, out, first + u * kFusedThreads);
  } else {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (first + u * kFusedThreads < nchunks) C::convert_store(v[u], sd, out, first + u * kFusedThreads);
  }
}

// P2P: the tensor is row-sharded over several GPUs running this same launch; the barrier between
// the phases also exchanges the per-GPU maxima through peer memory (see grid_max_barrier_exchange).
template <int IN, int OUT, int UNROLL, bool P2P>
__global__ void __launch_bounds__(kFusedThreads, kFusedBlocksPerSm)
dsq_fused_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ out, float *__restrict__ amax_out,
                 float *__restrict__ scale_out, int64_t numel, Workspace *ws, int smem_tiles, PeerExchange px) {
  using C = DsqChunk<IN, OUT, true>;
  extern __shared__ uint4 kept_smem[];  // [smem_tiles][UNROLL][kFusedThreads]
  __shared__ float smem32[32];
  __shared__ int flag;
  unsigned int gen0 = 0;
  if (threadIdx.x == 0) gen0 = ld_acquire(&ws->generation);

  const int64_t nchunks = numel / C::kElems;
  constexpr int64_t kTile = int64_t(kFusedThreads) * UNROLL;
  const int64_t ntiles = (nchunks + kTile - 1) / kTile;
  const int64_t tail0 = nchunks * C::kElems;
  const int64_t G = gridDim.x;
  // this block's tiles: blockIdx.x + k * G for k in [0, count)
  const int64_t count = blockIdx.x < ntiles ? (ntiles - blockIdx.x + G - 1) / G : 0;
  constexpr int kRegTiles = kFusedRegTiles;  // tile k = 0 lives in registers
  // tiles k in [kRegTiles, kept) live in shared memory, tiles k >= kept are streamed
  const int64_t kept = count < smem_tiles + kRegTiles ? count : smem_tiles + kRegTiles;

  // phase 1
  const uint64_t keep_policy = l2_policy_evict_last();
  // the newest kFusedL2KeepMB of the streamed tiles (phase 2 starts with them); never a kept tile
  const int64_t hint_tiles = (kFusedL2KeepMB << 20) / (G * kTile * 16);
  const int64_t hint_from = count - hint_tiles > kept ? count - hint_tiles : kept;
  float a = 0.0f, b = 0.0f;
  uint4 first_tile[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) first_tile[u] = make_uint4(0, 0, 0, 0);
  if (kRegTiles && count > 0) {
    load_tile<UNROLL>(first_tile, in, blockIdx.x, nchunks);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) C::absmax(a, b, first_tile[u]);
  }
  for (int64_t k = kRegTiles; k < count; k += 2) {  // two tiles (2 * UNROLL loads) in flight
    uint4 v[UNROLL], w[UNROLL];
    const bool second = k + 1 < count;
    // tiles that are not kept on chip come back in phase 2: ask L2 to hold on to them
    if (k >= hint_from) load_tile_hint<UNROLL>(v, in, blockIdx.x + k * G, nchunks, keep_policy);
    else load_tile<UNROLL>(v, in, blockIdx.x + k * G, nchunks);
    if (second) {
      if (k + 1 >= hint_from) load_tile_hint<UNROLL>(w, in, blockIdx.x + (k + 1) * G, nchunks, keep_policy);
      else load_tile<UNROLL>(w, in, blockIdx.x + (k + 1) * G, nchunks);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) C::absmax(a, b, v[u]);
    if (k < kept) {
      uint4 *slot = kept_smem + (k - kRegTiles) * kTile + threadIdx.x;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) slot[u * kFusedThreads] = v[u];
    }
    if (second) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) C::absmax(a, b, w[u]);
      if (k + 1 < kept) {
        uint4 *slot = kept_smem + (k + 1 - kRegTiles) * kTile + threadIdx.x;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) slot[u * kFusedThreads] = w[u];
      }
    }
  }
  if (blockIdx.x == 0 && tail0 + threadIdx.x < numel) a = fmaxf(a, fabsf(C::load_one(in, tail0 + threadIdx.x)));

  // finish
  const float block_value = block_max_nonneg(fmaxf(a, b), smem32, 0.0f);
  __shared__ float amax_shared;
  float amax;
  bool met;
  if constexpr (P2P) met = grid_max_barrier_exchange(ws, gen0, block_value, px, &flag, &amax_shared, &amax);
  else met = grid_max_barrier(ws, gen0, block_value, &flag, &amax_shared, &amax);
  if (!met) {  // a bounded wait gave up (the status word says so): no payload, and NaN where a maximum was expected
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      if (amax_out) *amax_out = __uint_as_float(0x7FC00000u);
      if (scale_out) *scale_out = __uint_as_float(0x7FC00000u);
    }
    return;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (amax_out) *amax_out = amax;
    if (scale_out) *scale_out = static_cast<float>(dsq_scale<OUT>(amax));
  }
  const DsqScale sd = make_dsq_scale<OUT>(amax);

  // phase 2a: streamed tiles, newest first
  for (int64_t k = count - 1; k >= kept; --k) {
    uint4 v[UNROLL];
    load_tile<UNROLL>(v, in, blockIdx.x + k * G, nchunks);
    store_tile<C, UNROLL>(v, sd, out, blockIdx.x + k * G, nchunks);
  }
  // phase 2b: tiles kept in shared memory, then the one kept in registers
  for (int64_t k = kept - 1; k >= kRegTiles; --k) {
    uint4 v[UNROLL];
    const uint4 *slot = kept_smem + (k - kRegTiles) * kTile + threadIdx.x;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) v[u] = slot[u * kFusedThreads];
    store_tile<C, UNROLL>(v, sd, out, blockIdx.x + k * G, nchunks);
  }
  if (kRegTiles && count > 0) store_tile<C, UNROLL>(first_tile, sd, out, blockIdx.x, nchunks);
  if (blockIdx.x == 0 && tail0 + threadIdx.x < numel)
    out[tail0 + threadIdx.x] = cvt_fp8<OUT>(dsq_mul(sd.sd, C::load_one(in, tail0 + threadIdx.x)));
}

// ---- cast phase alone ---------------------------------------------------------------------------------
constexpr int kCastPrefetchTiles = 6;  // tiles per block asked of L2 while the block waits for the amax
// BOUNDED: *amax_p is the maximum of this very input (no product can overflow).
template <int IN, int OUT, int UNROLL, bool BOUNDED>
__global__ void __launch_bounds__(kThreads, 2048 / kThreads)
cast_with_amax_stream(const uint4 *__restrict__ in, uint8_t *__restrict__ out, const float *__restrict__ amax_p,
                      float *__restrict__ scale_out, float *__restrict__ amax_out, int64_t numel) {
  using C = DsqChunk<IN, OUT, BOUNDED>;
  pdl_launch_dependents();
  const int64_t nchunks = numel / C::kElems;
  constexpr int64_t kTile = int64_t(kThreads) * UNROLL;
  const int64_t ntiles = (nchunks + kTile - 1) / kTile;
  // The amax may be a while in coming (behind it sits the end of a kernel, or an exchange between GPUs) and the
  // memory system idles meanwhile: ask L2 for this block's first tiles now.  Harmless whatever the kernel before
  // this one is still writing (see l2_prefetch_bulk).
  if (threadIdx.x < kCastPrefetchTiles) {
    const int64_t t = blockIdx.x + int64_t(threadIdx.x) * gridDim.x;
    if (t < ntiles && (ntiles - t) * kTile <= nchunks)
      l2_prefetch_bulk(in + (ntiles - 1 - t) * kTile, unsigned(kTile * sizeof(uint4)));
  }
  pdl_wait();  // launched so that it may become resident under the tail of the kernel that delivers the amax
  const float amax_in = *amax_p;
  const float amax = fmaxf(amax_in, 0.0f);
  const DsqScale sd = make_dsq_scale<OUT>(amax);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    // a NaN amax (an exchange that timed out upstream) is passed on, not silently turned into 0
    const bool bad = amax_in != amax_in;
    if (scale_out) *scale_out = bad ? amax_in : static_cast<float>(sd.sd);
    if (amax_out) *amax_out = bad ? amax_in : amax;
  }
  // highest addresses first: what the kernel before this one read last (an amax, an MX cast) may still be in L2
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t tile = ntiles - 1 - t;
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

// Per device and kernel instantiation: the shared memory the kernel may keep tiles in and the
// largest grid a cooperative launch accepts with it (cached after the first call).
constexpr int kMaxPlanDevices = 64;
struct FusedPlan {
  int smem_tiles = 0;
  int max_grid = 0;
};

template <typename Kernel>
int fused_plan(Kernel kernel, const DeviceInfo &dev, FusedPlan *cache, std::atomic<int> *ready, FusedPlan *plan) {
  int dev_id = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev_id));
  if (dev_id < 0 || dev_id >= kMaxPlanDevices) return DTQ_ERR_INVALID_ARGUMENT;
  if (!ready[dev_id].load(std::memory_order_acquire)) {
    static std::mutex mutex;
    std::lock_guard<std::mutex> lock(mutex);
    if (!ready[dev_id].load(std::memory_order_relaxed)) {
      int smem_per_sm = 0, reserved = 0;
      DTQ_CUDA_TRY(cudaDeviceGetAttribute(&smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev_id));
      DTQ_CUDA_TRY(cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev_id));
      const size_t tile_bytes = size_t(kFusedThreads) * kUnroll * 16;
      FusedPlan p;
      // what one of kFusedBlocksPerSm co-resident blocks can have, minus static use and reserve
      const size_t budget = size_t(smem_per_sm) / kFusedBlocksPerSm - reserved - 512;
      p.smem_tiles = static_cast<int>(budget / tile_bytes);
      if (p.smem_tiles > kFusedSmemTiles) p.smem_tiles = kFusedSmemTiles;
      const size_t dyn = size_t(p.smem_tiles) * tile_bytes;
      DTQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dyn)));
      int per_sm = 0;
      DTQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kFusedThreads, dyn));
      p.max_grid = per_sm * dev.sm_count;
      if (p.max_grid > kMaxGridBlocks) p.max_grid = kMaxGridBlocks;
      if (p.max_grid <= 0) return DTQ_ERR_CUDA_BASE + static_cast<int>(cudaErrorLaunchOutOfResources);
      cache[dev_id] = p;
      ready[dev_id].store(1, std::memory_order_release);
    }
  }
  *plan = cache[dev_id];
  return DTQ_OK;
}

// The single persistent launch (optionally with the cross-GPU exchange in its barrier).
template <int IN, int OUT, bool P2P>
int launch_fused_kernel(const void *in, void *out, float *amax_out, float *scale_out, int64_t numel, Workspace *ws,
                        const DeviceInfo &dev, const PeerExchange &px, cudaStream_t st) {
  using C = DsqChunk<IN, OUT>;
  static FusedPlan cache[kMaxPlanDevices];
  static std::atomic<int> ready[kMaxPlanDevices];
  auto kernel = dsq_fused_kernel<IN, OUT, kUnroll, P2P>;
  FusedPlan plan;
  if (int e = fused_plan(kernel, dev, cache, ready, &plan)) return e;
  const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kFusedThreads) * kUnroll);
  const int grid = balanced_grid(tiles, plan.max_grid);
  const uint4 *in4 = static_cast<const uint4 *>(in);
  uint8_t *o = static_cast<uint8_t *>(out);
  int smem_tiles = plan.smem_tiles;
  PeerExchange exchange = px;
  const size_t dyn = size_t(smem_tiles) * kFusedThreads * kUnroll * 16;
  void *args[] = {&in4, &o, &amax_out, &scale_out, &numel, &ws, &smem_tiles, &exchange};
  DTQ_CUDA_TRY(
      cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kernel), dim3(grid), dim3(kFusedThreads), args, dyn, st));
  return DTQ_OK;
}

template <int IN, int OUT>
int launch_fused(const void *in, void *out, float *amax_out, float *scale_out, int64_t numel, Workspace *ws,
                 const DeviceInfo &dev, cudaStream_t st) {
  using C = DsqChunk<IN, OUT>;
  uint8_t *o = static_cast<uint8_t *>(out);
  const bool vector_ok = aligned_to(in, 16) && aligned_to(out, C::kOutAlign);
  if (vector_ok && numel * C::kElemBytes > kFusedMaxBytes) {
    if (int e = launch_amax(in, &ws->amax, numel, IN, ws, dev, st)) return e;
    const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kThreads) * kUnroll);
    const int grid = balanced_grid(tiles, int64_t(dev.sm_count) * kCastBlocksPerSmCap);
    return cuda_status(launch_after_dependency(cast_with_amax_stream<IN, OUT, kUnroll, true>, dim3(grid), dim3(kThreads),
                                               0, st, static_cast<const uint4 *>(in), o, &ws->amax, scale_out, amax_out,
                                               numel));
  }
  if (vector_ok && dev.cooperative)
    return launch_fused_kernel<IN, OUT, false>(in, out, amax_out, scale_out, numel, ws, dev, PeerExchange{}, st);
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
  const int64_t max_grid = int64_t(dev.sm_count) * kCastBlocksPerSmCap;
  if (aligned_to(in, 16) && aligned_to(out, C::kOutAlign)) {
    const int64_t tiles = ceil_div64(numel / C::kElems, int64_t(kThreads) * kUnroll);
    const int grid = balanced_grid(tiles, max_grid);
    return cuda_status(launch_after_dependency(cast_with_amax_stream<IN, OUT, kUnroll, false>, dim3(grid),
                                               dim3(kThreads), 0, st, static_cast<const uint4 *>(in), o, amax, scale_out,
                                               static_cast<float *>(nullptr), numel));
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

extern "C" size_t dtq_p2p_exchange_bytes(void) { return sizeof(unsigned long long) * dtq::kPeerParities * dtq::kMaxPeers; }

extern "C" int dtq_dynamic_scaled_quant_p2p(const void *in, void *out, float *amax_out, float *scale_out, int64_t numel,
                                            int in_dtype, int out_dtype, void *workspace, size_t workspace_bytes,
                                            void *const *peer_exchange, int rank, int world, uint32_t epoch,
                                            uint32_t spin_limit, void *stream) {
  using namespace dtq;
  if (numel < 0 || (numel > 0 && (!in || !out)) || !peer_exchange) return DTQ_ERR_INVALID_ARGUMENT;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return DTQ_ERR_INVALID_ARGUMENT;
  if (int e = check_dtypes(in_dtype, out_dtype)) return e;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  // the exchange lives in the vector kernel: every rank must take it, so alignment is a requirement here
  const int out_align = in_dtype == DTQ_BF16 ? 8 : 4;
  if (!aligned_to(in, 16) || !aligned_to(out, out_align)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  if (!dev.cooperative) return DTQ_ERR_CUDA_BASE + static_cast<int>(cudaErrorNotSupported);
  PeerExchange px{};
  for (int r = 0; r < world; ++r) {
    if (!peer_exchange[r] || !aligned_to(peer_exchange[r], 8)) return DTQ_ERR_INVALID_ARGUMENT;
    px.buffer[r] = static_cast<unsigned long long *>(peer_exchange[r]);
  }
  px.rank = rank;
  px.world = world;
  px.epoch = epoch;
  px.spin_limit = spin_limit ? spin_limit : kSpinLimit;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace *ws = static_cast<Workspace *>(workspace);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3
               ? launch_fused_kernel<DTQ_BF16, DTQ_E4M3, true>(in, out, amax_out, scale_out, numel, ws, dev, px, st)
               : launch_fused_kernel<DTQ_BF16, DTQ_E5M2, true>(in, out, amax_out, scale_out, numel, ws, dev, px, st);
  return out_dtype == DTQ_E4M3
             ? launch_fused_kernel<DTQ_F32, DTQ_E4M3, true>(in, out, amax_out, scale_out, numel, ws, dev, px, st)
             : launch_fused_kernel<DTQ_F32, DTQ_E5M2, true>(in, out, amax_out, scale_out, numel, ws, dev, px, st);
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
