// mx_fp8_quantize, shared-memory-staged variant: the same arithmetic and outputs as mx_cast.cu,
// but the input reaches the SM through the bulk asynchronous copy engine (TMA, 1-D
// cp.async.bulk global -> shared, completion on an mbarrier) into a ring of stages, decoupled
// from the warps that convert.  A persistent CTA = one producer thread + eight consumer warps;
// full/empty mbarriers per stage; every wait is bounded and reports through a status word.
// No tensor map is needed (MX blocks run along the contiguous dimension, so a tile is a flat
// 16 KiB span); every copy is for the CTA that issues it, there is no cluster.
//
// Kept beside the register-path kernel as a measured alternative (the benchmark's per-op table
// times both): on B200 the register path is faster for this reuse-free stream, so the default
// entry point uses it.
#include <atomic>

#include "dtq_host.h"
#include "mx_common.cuh"

namespace dtq {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreadsTma = kConsumerThreads + 32;  // + one producer warp (lane 0 issues)
constexpr int kUnroll = 4;                          // 16-byte chunks per consumer thread per tile
constexpr int kTileChunks = kConsumerThreads * kUnroll;
constexpr int kTileBytes = kTileChunks * 16;  // 16 KiB
constexpr int kStages = 4;
constexpr int kTmaBlocksPerSm = 3;
constexpr unsigned int kWaitLimit = 1u << 20;  // polls of try_wait (each already waits a while in hardware)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity to complete; false if it never did.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity) {
  const uint32_t addr = smem_u32(bar);
  for (unsigned int spins = 0; spins < kWaitLimit; ++spins) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct __align__(128) TmaSmem {
  uint4 stage[kStages][kTileChunks];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int abort;  // set by whoever gives up a wait: everybody else stops at its next tile
};

// Tiles blockIdx.x, blockIdx.x + gridDim.x, ... of kTileChunks chunks each; nchunks % 4 == 0.
__global__ void __launch_bounds__(kThreadsTma)
mx_tma_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
              int64_t nchunks, int *status) {
  extern __shared__ unsigned char smem_raw[];
  TmaSmem &sm = *reinterpret_cast<TmaSmem *>(smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t ntiles = (nchunks + kTileChunks - 1) / kTileChunks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kConsumerWarps);
    }
    sm.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kConsumerWarps) {  // producer warp
    if (lane == 0) {
      volatile int *abort = &sm.abort;
      int64_t k = 0;
      for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++k) {
        const int s = static_cast<int>(k % kStages);
        const unsigned round = static_cast<unsigned>(k / kStages);
        if (*abort || (round > 0 && !mbar_wait(&sm.empty[s], (round - 1) & 1u))) {
          // Give up, but not with copies still on their way into this CTA's shared memory: wait
          // (bounded) for the newest copy of every stage; they complete without the consumers' help.
          atomicExch(status, DTQ_ERR_TIMEOUT);
          *abort = 1;
          for (int64_t j = k - 1; j >= 0 && j > k - 1 - kStages; --j)
            mbar_wait(&sm.full[j % kStages], static_cast<unsigned>(j / kStages) & 1u);
          return;
        }
        const int64_t first = tile * kTileChunks;
        const int64_t left = nchunks - first;
        const unsigned bytes = static_cast<unsigned>((left < kTileChunks ? left : kTileChunks) * 16);
        mbar_expect_tx(&sm.full[s], bytes);
        bulk_load(sm.stage[s], in + first, bytes, &sm.full[s]);
      }
    }
    return;
  }

  // consumers
  int64_t k = 0;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++k) {
    const int s = static_cast<int>(k % kStages);
    const unsigned round = static_cast<unsigned>(k / kStages);
    if (*static_cast<volatile int *>(&sm.abort)) return;  // the producer drains its copies before the CTA ends
    if (!mbar_wait(&sm.full[s], round & 1u)) {
      // the copy never landed: nothing can be drained; after this status the outputs are not to be trusted
      if (lane == 0) {
        atomicExch(status, DTQ_ERR_TIMEOUT);
        *static_cast<volatile int *>(&sm.abort) = 1;
      }
      return;
    }
    const int64_t warp_first = tile * kTileChunks + int64_t(warp) * (32 * kUnroll);
    const uint4 *src = sm.stage[s] + warp * (32 * kUnroll);
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = src[u * 32 + lane];  // bytes past the end of the input are stale: masked below
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);  // the stage may be refilled while this warp converts

    uint32_t my_scale_byte = 0;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t c = warp_first + u * 32 + lane;
      uint32_t mag = c < nchunks ? chunk_absmax_bits(v[u]) : 0u;
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 1));
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 2));
      const int biased = block_biased_exponent(mag);
      const float inv = inverse_scale(biased);
      if (c < nchunks) {
        uint2 r;
        r.x = mx_pair(v[u].x, inv) | (mx_pair(v[u].y, inv) << 16);
        r.y = mx_pair(v[u].z, inv) | (mx_pair(v[u].w, inv) << 16);
        stg_stream(payload + c * 8, r);
      }
      if ((lane & 3) == u) my_scale_byte = mx_scale_byte(biased);
    }
    const int64_t blk = warp_first / 4 + (lane & 3) * 8 + (lane >> 2);
    if (blk * 4 < nchunks) scales[blk] = static_cast<uint8_t>(my_scale_byte);
  }
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_mx_fp8_quantize_tma(const void *in_bf16, void *payload, void *scales_e8m0, int64_t rows,
                                       int64_t cols, int *status_dev, void *stream) {
  using namespace dtq;
  if (rows < 0 || cols < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (cols % 32 != 0) return DTQ_ERR_SHAPE;
  const int64_t numel = rows * cols;
  if (numel == 0) return DTQ_OK;
  if (!in_bf16 || !payload || !scales_e8m0 || !status_dev) return DTQ_ERR_INVALID_ARGUMENT;
  // the bulk copy needs 16-byte aligned sources; the packed stores 8-byte aligned destinations
  if (!aligned_to(in_bf16, 16) || !aligned_to(payload, 8)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  constexpr int kMaxDevices = 64;
  static std::atomic<int> configured[kMaxDevices];
  int dev_id = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev_id));
  if (dev_id < 0 || dev_id >= kMaxDevices) return DTQ_ERR_INVALID_ARGUMENT;
  const int smem = static_cast<int>(sizeof(TmaSmem)) + 128;
  if (!configured[dev_id].load(std::memory_order_acquire)) {  // setting the attribute twice is harmless
    DTQ_CUDA_TRY(cudaFuncSetAttribute(mx_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev_id].store(1, std::memory_order_release);
  }
  const int64_t nchunks = numel / 8;
  const int64_t tiles = ceil_div64(nchunks, kTileChunks);
  const int grid = balanced_grid(tiles, int64_t(dev.sm_count) * kTmaBlocksPerSm);
  mx_tma_kernel<<<grid, kThreadsTma, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(in_bf16), static_cast<uint8_t *>(payload), static_cast<uint8_t *>(scales_e8m0), nchunks,
      status_dev);
  return cuda_status(cudaGetLastError());
}
