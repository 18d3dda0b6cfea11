// Grid-wide finish of a max reduction inside one launch, and a bounded grid barrier.
//
// Each block publishes one partial and takes a ticket; the block that draws the last ticket
// reduces all partials.  No output has to be pre-initialised and the workspace is left ready for
// the next launch.  Waiting (only the fused ops wait) is a bounded spin: if the generation word
// does not move within the limit, the waiter records DTQ_ERR_TIMEOUT in the workspace and the
// block returns, so a launch can never hang the device.
#pragma once

#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_relaxed_f32(const float *p) {
  float v;
  asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Publishes `block_value` (meaningful in thread 0) and returns, in every thread of the block,
// whether this block arrived last.  `flag` is one int of shared memory.
__device__ __forceinline__ bool publish_and_ticket(Workspace *ws, float block_value, int *flag) {
  if (threadIdx.x == 0) {
    ws->partials[blockIdx.x] = block_value;
    __threadfence();
    const unsigned int ticket = atomicAdd(&ws->arrivals, 1u);
    *flag = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  const bool last = *flag != 0;
  __syncthreads();
  return last;
}

// Run by every thread of the last block: max over all blocks' partials (valid in warp 0).
__device__ __forceinline__ float reduce_partials(const Workspace *ws, float *smem32, float identity) {
  __threadfence();
  float v = identity;
  for (unsigned int i = threadIdx.x; i < gridDim.x; i += blockDim.x) v = fmaxf(v, ld_relaxed_f32(&ws->partials[i]));
  return block_max_nonneg(v, smem32, identity);
}

constexpr unsigned int kSpinLimit = 1u << 23;  // x ~100 ns sleep: gives up after about a second

// Thread 0 waits until the generation word differs from `gen0`; every thread gets the verdict.
__device__ __forceinline__ bool wait_generation(Workspace *ws, unsigned int gen0, int *flag) {
  if (threadIdx.x == 0) {
    unsigned int spins = 0;
    bool ok = true;
    while (ld_acquire(&ws->generation) == gen0) {
      if (++spins > kSpinLimit) {
        ok = false;
        atomicExch(&ws->status, DTQ_ERR_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
    *flag = ok;
  }
  __syncthreads();
  const bool ok = *flag != 0;
  __syncthreads();
  return ok;
}

}  // namespace dtq
