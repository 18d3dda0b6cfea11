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

constexpr unsigned int kSpinLimit = 1u << 20;  // polls, each an L2 round trip plus a short sleep: gives up after about a second

// Grid barrier that also reduces a non-negative float maximum, for kernels whose blocks are all
// co-resident.  `gen0` is the generation word as read by thread 0 BEFORE the block did anything
// else; its parity picks the counter pair.  Thread 0 folds the block's value into the running
// maximum, fences, takes a ticket; the last arriver clears the other parity's pair (the previous
// launch is long over) and bumps the generation for the next launch.  Everybody then waits for
// the count to reach gridDim.x (bounded spin) and reads the maximum.  Returns false on timeout
// (status word set, nothing may be assumed about `*result`).
__device__ __forceinline__ bool grid_max_barrier(Workspace *ws, unsigned int gen0, float block_value, int *flag,
                                                 float *shared_result, float *result) {
  if (threadIdx.x == 0) {
    const unsigned int slot = gen0 & 1u;
    atomicMax(&ws->bar_max[slot], __float_as_uint(block_value));
    __threadfence();
    const unsigned int ticket = atomicAdd(&ws->bar_count[slot], 1u);
    bool ok = true;
    if (ticket == gridDim.x - 1) {
      ws->bar_count[slot ^ 1u] = 0;
      ws->bar_max[slot ^ 1u] = 0;
      atomicAdd(&ws->generation, 1u);
    } else {
      unsigned int spins = 0;
      while (ld_acquire(&ws->bar_count[slot]) != gridDim.x) {
        if (++spins > kSpinLimit) {
          ok = false;
          atomicExch(&ws->status, DTQ_ERR_TIMEOUT);
          break;
        }
        __nanosleep(20);
      }
    }
    __threadfence();
    *shared_result = __uint_as_float(ld_acquire(&ws->bar_max[slot]));
    *flag = ok;
  }
  __syncthreads();
  *result = *shared_result;
  const bool ok = *flag != 0;
  __syncthreads();
  return ok;
}

}  // namespace dtq
