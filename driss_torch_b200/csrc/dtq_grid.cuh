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

// ---- the same barrier with an exchange across GPUs in its serial section -------------------------
// Every rank (one process per GPU, same launch on each) owns a small exchange buffer that all
// peers can address over NVLink: kPeerParities x kMaxPeers 64-bit slots.  The last block to arrive
// at the local barrier stores {epoch, local maximum} into its slot of EVERY rank's buffer
// (st.release.sys, plain peer stores) and then reads its own buffer until all `world` slots carry
// this launch's epoch (ld.acquire.sys, bounded spin).  The slot parity alternates with the epoch,
// so a fast peer's next launch can never overwrite a value a slow rank has not read yet (a rank
// cannot get two launches ahead: it needs this rank's next value first).  Nothing is ever reset.
constexpr int kMaxPeers = 16;
constexpr int kPeerParities = 2;

struct PeerExchange {
  unsigned long long *buffer[kMaxPeers];  // entry r: rank r's exchange buffer as mapped on this device
  int rank, world;
  unsigned int epoch;       // same on every rank for the same launch, increasing by one per launch
  unsigned int spin_limit;  // polls before a wait gives up
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// The exchange alone, for a kernel without a grid barrier: run by all 32 lanes of one warp of one
// block per rank.  Stores {epoch, local_bits} into this rank's slot on every rank and returns the
// maximum of all ranks' values for this epoch (unsigned order); *ok is false if a peer's value did
// not arrive within the spin limit.
__device__ __forceinline__ unsigned int peer_exchange_max(const PeerExchange &px, unsigned int local_bits, bool *ok) {
  const int lane = threadIdx.x & 31;
  const int parity = px.epoch & 1u;
  unsigned int value = 0;
  bool mine_ok = true;
  if (lane < px.world) {
    // The 64-bit word {epoch, value} is the whole message: one store, one load, nothing else to order against it
    // (a release / acquire pair at system scope costs a fence on each side of the link).
    st_relaxed_sys(px.buffer[lane] + parity * kMaxPeers + px.rank,
                   (static_cast<unsigned long long>(px.epoch) << 32) | local_bits);
    const unsigned long long *mine = px.buffer[px.rank] + parity * kMaxPeers + lane;
    unsigned int spins = 0;
    unsigned long long v = ld_relaxed_sys(mine);
    while (static_cast<unsigned int>(v >> 32) != px.epoch) {
      if (++spins > px.spin_limit) {
        mine_ok = false;
        break;
      }
      __nanosleep(40);
      v = ld_relaxed_sys(mine);
    }
    value = static_cast<unsigned int>(v);
  }
  *ok = __all_sync(0xFFFFFFFFu, mine_ok);
  return __reduce_max_sync(0xFFFFFFFFu, value);
}

// As grid_max_barrier, but the value every block leaves with is the maximum over all ranks.
// Waiting blocks watch the local count reach gridDim.x + 1: the last arriver adds the extra one
// after the exchange, when ws->amax holds the global value.
__device__ __forceinline__ bool grid_max_barrier_exchange(Workspace *ws, unsigned int gen0, float block_value,
                                                          const PeerExchange &px, int *flag, float *shared_result,
                                                          float *result) {
  if (threadIdx.x < 32) {  // warp 0; lane 0 runs the local protocol, lanes < world the exchange
    const unsigned int slot = gen0 & 1u;
    const int lane = threadIdx.x;
    unsigned int ticket = 0;
    if (lane == 0) {
      atomicMax(&ws->bar_max[slot], __float_as_uint(block_value));
      __threadfence();
      ticket = atomicAdd(&ws->bar_count[slot], 1u);
    }
    ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
    bool ok = true;
    if (ticket == gridDim.x - 1) {
      unsigned int local_bits = 0;
      if (lane == 0) {
        __threadfence();
        local_bits = ld_acquire(&ws->bar_max[slot]);
      }
      local_bits = __shfl_sync(0xFFFFFFFFu, local_bits, 0);
      const int parity = px.epoch & 1u;
      unsigned int global_bits = 0;
      if (lane < px.world) {
        st_release_sys(px.buffer[lane] + parity * kMaxPeers + px.rank,
                       (static_cast<unsigned long long>(px.epoch) << 32) | local_bits);
        const unsigned long long *mine = px.buffer[px.rank] + parity * kMaxPeers + lane;
        unsigned int spins = 0;
        unsigned long long v = ld_acquire_sys(mine);
        while (static_cast<unsigned int>(v >> 32) != px.epoch) {
          if (++spins > px.spin_limit) {
            ok = false;
            break;
          }
          __nanosleep(40);
          v = ld_acquire_sys(mine);
        }
        global_bits = static_cast<unsigned int>(v);
      }
      ok = __all_sync(0xFFFFFFFFu, ok);
      global_bits = __reduce_max_sync(0xFFFFFFFFu, global_bits);  // non-negative floats order like their bits
      if (lane == 0) {
        if (!ok) atomicExch(&ws->status, DTQ_ERR_TIMEOUT);
        ws->amax = ok ? __uint_as_float(global_bits) : 0.0f;
        ws->bar_count[slot ^ 1u] = 0;
        ws->bar_max[slot ^ 1u] = 0;
        atomicAdd(&ws->generation, 1u);
        __threadfence();
        // release the local waiters; on failure with a count they recognise as "gave up"
        atomicAdd(&ws->bar_count[slot], ok ? 1u : 2u);
      }
    } else if (lane == 0) {
      unsigned int spins = 0;
      unsigned int c = ld_acquire(&ws->bar_count[slot]);
      while (c <= gridDim.x) {
        if (++spins > kSpinLimit + px.spin_limit) {
          atomicExch(&ws->status, DTQ_ERR_TIMEOUT);
          break;
        }
        __nanosleep(20);
        c = ld_acquire(&ws->bar_count[slot]);
      }
      ok = c == gridDim.x + 1;
    }
    if (lane == 0) {
      __threadfence();
      *shared_result = ld_relaxed_f32(&ws->amax);
      *flag = ok;
    }
  }
  __syncthreads();
  *result = *shared_result;
  const bool ok = *flag != 0;
  __syncthreads();
  return ok;
}

}  // namespace dtq
