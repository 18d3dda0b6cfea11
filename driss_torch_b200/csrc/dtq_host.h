// Host-side helpers shared by the launchers: status mapping, per-device facts, the workspace
// layout that kernels and launchers agree on.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/dtq_b200.h"

namespace dtq {

constexpr int kMaxGridBlocks = 4096;  // upper bound on any persistent grid (148 SMs x 16 CTAs fits)

// Scratch shared by the single-launch reductions.  Zero-filled once by dtq_workspace_init;
// every kernel leaves `arrivals` at zero again and only ever advances `generation`.
struct alignas(256) Workspace {
  unsigned int arrivals;    // blocks that have published their partial in the current launch
  unsigned int generation;  // bumped by the last-arriving block; waiters spin on it (bounded)
  int status;               // sticky: DTQ_ERR_TIMEOUT if a bounded wait ever gave up
  float amax;               // the reduced value of the current launch, valid after the bump
  // The fused kernel's grid barrier: arrival count and running maximum (as float bits), one pair
  // per parity of `generation`; a launch uses the pair of its parity and clears the other.
  unsigned int bar_count[2];
  unsigned int bar_max[2];
  // Running maxima of kernels whose blocks fold their value into a few words (atomicMax, block b
  // into word b % 32) instead of publishing partials; a one-warp finishing launch takes them and
  // leaves zeros behind.
  unsigned int slot_max[32];
  unsigned int pad[24];
  float partials[kMaxGridBlocks];
};

struct DeviceInfo {
  int sm_count = 0;
  int cooperative = 0;
};

// Facts about the current device, queried once per device and cached (thread-safe).
int current_device_info(DeviceInfo *info);

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? DTQ_OK : DTQ_ERR_CUDA_BASE + static_cast<int>(e); }

#define DTQ_CUDA_TRY(expr)                             \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) return dtq::cuda_status(_e); \
  } while (0)

// Launches `kernel` so that it may start while the kernel queued before it on `st` is still
// draining (programmatic dependent launch).  The kernel must call pdl_wait() before its first
// access to memory that its predecessor on the stream may read or write.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_dependency(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes,
                                           cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned_to(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Grid for a persistent kernel that walks `tiles` tiles grid-stride: at most `max_grid` blocks,
// and when every block needs several tiles, as few blocks as keep the number of rounds, so that
// all blocks run the same number of tiles (no straggler round with most of the GPU idle).
inline int balanced_grid(int64_t tiles, int64_t max_grid) {
  if (tiles < 1) return 1;
  if (tiles <= max_grid) return static_cast<int>(tiles);
  const int64_t rounds = ceil_div64(tiles, max_grid);
  return static_cast<int>(ceil_div64(tiles, rounds));
}

}  // namespace dtq
