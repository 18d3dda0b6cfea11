// Status strings, per-device facts and workspace management for the C ABI.
#include <atomic>
#include <mutex>

#include "dtq_host.h"

namespace dtq {

namespace {
constexpr int kMaxDevices = 64;
DeviceInfo g_info[kMaxDevices];
std::atomic<int> g_ready[kMaxDevices];
std::mutex g_mutex;
}  // namespace

int current_device_info(DeviceInfo *info) {
  int dev = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return DTQ_ERR_INVALID_ARGUMENT;
  if (!g_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_ready[dev].load(std::memory_order_relaxed)) {
      DeviceInfo d;
      DTQ_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
      DTQ_CUDA_TRY(cudaDeviceGetAttribute(&d.cooperative, cudaDevAttrCooperativeLaunch, dev));
      g_info[dev] = d;
      g_ready[dev].store(1, std::memory_order_release);
    }
  }
  *info = g_info[dev];
  return DTQ_OK;
}

}  // namespace dtq

extern "C" const char *dtq_status_string(int status) {
  switch (status) {
    case DTQ_OK: return "ok";
    case DTQ_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer or negative size)";
    case DTQ_ERR_UNSUPPORTED_DTYPE: return "unsupported element type";
    case DTQ_ERR_SHAPE: return "unsupported shape";
    case DTQ_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
    case DTQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case DTQ_ERR_TOO_LARGE: return "size exceeds the limit of this entry point";
    default: break;
  }
  if (status >= DTQ_ERR_CUDA_BASE) return cudaGetErrorString(static_cast<cudaError_t>(status - DTQ_ERR_CUDA_BASE));
  return "unknown status";
}

extern "C" const char *dtq_version(void) { return "dtq_b200 0.1 (sm_100a)"; }

extern "C" size_t dtq_workspace_bytes(void) { return sizeof(dtq::Workspace); }

extern "C" int dtq_workspace_init(void *workspace, size_t workspace_bytes, void *stream) {
  if (!workspace || workspace_bytes < sizeof(dtq::Workspace) || !dtq::aligned_to(workspace, 256))
    return DTQ_ERR_WORKSPACE;
  return dtq::cuda_status(cudaMemsetAsync(workspace, 0, sizeof(dtq::Workspace), static_cast<cudaStream_t>(stream)));
}

extern "C" int dtq_workspace_status_async(const void *workspace, int *status_host, void *stream) {
  if (!workspace || !status_host) return DTQ_ERR_INVALID_ARGUMENT;
  const dtq::Workspace *ws = static_cast<const dtq::Workspace *>(workspace);
  return dtq::cuda_status(cudaMemcpyAsync(status_host, &ws->status, sizeof(int), cudaMemcpyDeviceToHost,
                                          static_cast<cudaStream_t>(stream)));
}

extern "C" int dtq_workspace_status(const void *workspace, int *status_host, void *stream) {
  if (!workspace || !status_host) return DTQ_ERR_INVALID_ARGUMENT;
  const dtq::Workspace *ws = static_cast<const dtq::Workspace *>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DTQ_CUDA_TRY(cudaMemcpyAsync(status_host, &ws->status, sizeof(int), cudaMemcpyDeviceToHost, st));
  return dtq::cuda_status(cudaStreamSynchronize(st));
}
