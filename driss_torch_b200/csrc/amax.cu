// amax: out[0] = max |in[i]| as fp32, finished grid-wide in a single launch.
//
// Replaces src/amax.cu:50-80 (+ the -inf fill launch at :115): a persistent grid streams the
// input with several 128-bit loads in flight per thread, reduces with packed bf16 max, one
// integer warp-max instruction per warp, and a last-block finish instead of one same-address
// atomic per block on a pre-filled output.  The value is order independent, so the result is
// bit-identical; NaNs are dropped and an empty input gives -inf, as in the reference.
#include <atomic>
#include <cmath>
#include <mutex>

#include "dtq_device.cuh"
#include "dtq_grid.cuh"
#include "dtq_host.h"

namespace dtq {

constexpr int kAmaxUnroll = 8;       // 128-bit loads in flight per thread
constexpr int kAmaxBlocksPerSm = 4;  // persistent grid: blocks per SM
constexpr int kAmaxThreads = 512;

template <int IN>
struct AbsMax;

template <>
struct AbsMax<DTQ_BF16> {
  static constexpr int kElemBytes = 2;
  __nv_bfloat162 a, b;
  __device__ explicit AbsMax(float identity) { a = b = __float2bfloat162_rn(identity); }
  __device__ void chunk(uint4 v) {
    a = absmax_bf162(a, v.x);
    b = absmax_bf162(b, v.y);
    a = absmax_bf162(a, v.z);
    b = absmax_bf162(b, v.w);
  }
  __device__ void one(const void *p, int64_t i) {
    const uint32_t h = static_cast<const uint16_t *>(p)[i];
    a = absmax_bf162(a, h | (h << 16));
  }
  __device__ float result() const { return bf162_hmax_to_float(__hmax2(a, b)); }
};

template <>
struct AbsMax<DTQ_F32> {
  static constexpr int kElemBytes = 4;
  float a, b;
  __device__ explicit AbsMax(float identity) { a = b = identity; }
  __device__ void chunk(uint4 v) {
    a = fmaxf(a, fabsf(__uint_as_float(v.x)));
    b = fmaxf(b, fabsf(__uint_as_float(v.y)));
    a = fmaxf(a, fabsf(__uint_as_float(v.z)));
    b = fmaxf(b, fabsf(__uint_as_float(v.w)));
  }
  __device__ void one(const void *p, int64_t i) { a = fmaxf(a, fabsf(static_cast<const float *>(p)[i])); }
  __device__ float result() const { return fmaxf(a, b); }
};

// Streams chunks [0, nchunks) of `body` grid-stride in tiles of blockDim.x * UNROLL chunks.
template <int IN, int UNROLL>
__device__ __forceinline__ void absmax_stream(AbsMax<IN> &acc, const uint4 *__restrict__ body, int64_t nchunks) {
  const int64_t tile_chunks = int64_t(blockDim.x) * UNROLL;
  for (int64_t tile = blockIdx.x; tile * tile_chunks < nchunks; tile += gridDim.x) {
    const int64_t first = tile * tile_chunks + threadIdx.x;
    uint4 v[UNROLL];
    if ((tile + 1) * tile_chunks <= nchunks) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ldg_stream(body + first + int64_t(u) * blockDim.x);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc.chunk(v[u]);
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t c = first + int64_t(u) * blockDim.x;
        if (c < nchunks) acc.chunk(ldg_stream(body + c));
      }
    }
  }
}

// `in` may have any element alignment: up to `head` leading and `tail` trailing elements are
// read one by one by block 0, the 16-byte aligned middle is streamed.
template <int IN, int UNROLL>
__global__ void __launch_bounds__(kAmaxThreads)
amax_kernel(const void *__restrict__ in, float *__restrict__ out, int64_t numel, int64_t head, Workspace *ws) {
  __shared__ float smem32[32];
  __shared__ int flag;
  constexpr int kElems = 16 / AbsMax<IN>::kElemBytes;
  pdl_launch_dependents();  // a cast queued behind this launch with launch_after_dependency may become resident early
  pdl_wait();               // and this launch itself may have started under the tail of its predecessor
  const float identity = -INFINITY;
  AbsMax<IN> acc(identity);

  const char *base = static_cast<const char *>(in);
  const int64_t nchunks = (numel - head) / kElems;
  absmax_stream<IN, UNROLL>(acc, reinterpret_cast<const uint4 *>(base + head * AbsMax<IN>::kElemBytes), nchunks);
  if (blockIdx.x == 0) {
    const int64_t tail0 = head + nchunks * kElems;
    if (threadIdx.x < head) acc.one(in, threadIdx.x);
    if (tail0 + threadIdx.x < numel) acc.one(in, tail0 + threadIdx.x);
  }

  const float block_value = block_max_nonneg(acc.result(), smem32, identity);
  if (publish_and_ticket(ws, block_value, &flag)) {
    const float total = reduce_partials(ws, smem32, identity);
    if (threadIdx.x == 0) {
      out[0] = total;
      ws->arrivals = 0;
    }
  }
}

int amax_grid(int64_t numel, int elem_bytes, const DeviceInfo &dev) {
  const int64_t tiles = ceil_div64(numel * elem_bytes / 16, int64_t(kAmaxThreads) * kAmaxUnroll);
  const int64_t max_grid = int64_t(dev.sm_count) * kAmaxBlocksPerSm;
  return balanced_grid(tiles, max_grid);
}

int64_t head_elems(const void *p, int elem_bytes, int64_t numel) {
  const int64_t h = static_cast<int64_t>((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / elem_bytes;
  return h < numel ? h : numel;
}

// Arguments already validated; `out` may be any device float (the fused op points it into its
// workspace when it splits a very large tensor into amax + cast).
int launch_amax(const void *in, float *out, int64_t numel, int in_dtype, Workspace *ws, const DeviceInfo &dev,
                cudaStream_t st) {
  const int eb = in_dtype == DTQ_BF16 ? 2 : 4;
  const int grid = amax_grid(numel, eb, dev);
  const int64_t head = head_elems(in, eb, numel);
  if (in_dtype == DTQ_BF16)
    return cuda_status(launch_after_dependency(amax_kernel<DTQ_BF16, kAmaxUnroll>, dim3(grid), dim3(kAmaxThreads), 0, st, in,
                                               out, numel, head, ws));
  return cuda_status(launch_after_dependency(amax_kernel<DTQ_F32, kAmaxUnroll>, dim3(grid), dim3(kAmaxThreads), 0, st, in, out,
                                             numel, head, ws));
}

}  // namespace dtq

extern "C" int dtq_amax(const void *in, float *out, int64_t numel, int in_dtype, void *workspace,
                        size_t workspace_bytes, void *stream) {
  using namespace dtq;
  if (numel < 0 || !out || (numel > 0 && !in)) return DTQ_ERR_INVALID_ARGUMENT;
  if (in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  if (numel > 0 && !aligned_to(in, in_dtype == DTQ_BF16 ? 2 : 4)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  return launch_amax(in, out, numel, in_dtype, static_cast<Workspace *>(workspace), dev, static_cast<cudaStream_t>(stream));
}

// ---- amax without any caller- or library-allocated scratch -------------------------------------------------
//
// Some hosts may not allocate device memory at the point where they need an amax: a runtime that
// hands the whole device heap to its own pool and forbids cudaMalloc in plugins, or a
// latency-critical section that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply.  For them the scratch of the reduction lives in this library's image: one
// Workspace in a file-scope __device__ array, present on every GPU that loads the library until
// the process exits.
//
// In host code the array's NAME is only a host-side handle, not a device address, so the address
// is looked up once per device with cudaGetSymbolAddress (with that device current) and cached.
// One block per tile is launched, so the array's kMaxGridBlocks partial slots bound the input:
// kMaxGridBlocks tiles of kAmaxThreads * kAmaxUnroll 16-byte chunks = DTQ_AMAX_STATIC_MAX_BYTES.
namespace dtq {
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[sizeof(Workspace)];

constexpr int kStaticMaxDevices = 64;
void *g_static_scratch_ptr[kStaticMaxDevices];
std::atomic<int> g_static_scratch_ready[kStaticMaxDevices];
std::mutex g_static_scratch_mutex;

// Device address of the scratch array on the current device (looked up on first use).
int static_scratch_address(Workspace **ws) {
  int dev = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kStaticMaxDevices) return DTQ_ERR_INVALID_ARGUMENT;
  if (!g_static_scratch_ready[dev].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ready[dev].load(std::memory_order_relaxed)) {
      void *ptr = nullptr;
      DTQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
      g_static_scratch_ptr[dev] = ptr;
      g_static_scratch_ready[dev].store(1, std::memory_order_release);
    }
  }
  *ws = static_cast<Workspace *>(g_static_scratch_ptr[dev]);
  return DTQ_OK;
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_amax_static_scratch(const void *in, float *out, int64_t numel, int in_dtype, void *stream) {
  using namespace dtq;
  static_assert(int64_t(kMaxGridBlocks) * kAmaxThreads * kAmaxUnroll * 16 == DTQ_AMAX_STATIC_MAX_BYTES,
                "the documented limit must match the scratch array");
  if (numel < 0 || !out || (numel > 0 && !in)) return DTQ_ERR_INVALID_ARGUMENT;
  if (in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) return DTQ_ERR_UNSUPPORTED_DTYPE;
  const int eb = in_dtype == DTQ_BF16 ? 2 : 4;
  if (numel > DTQ_AMAX_STATIC_MAX_BYTES / eb) return DTQ_ERR_TOO_LARGE;  // needs more partial slots than the array has
  if (numel > 0 && !aligned_to(in, eb)) return DTQ_ERR_INVALID_ARGUMENT;
  Workspace *ws = nullptr;
  if (int e = static_scratch_address(&ws)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: start the arrival counter from zero.
  DTQ_CUDA_TRY(cudaMemsetAsync(&ws->arrivals, 0, sizeof(ws->arrivals), st));
  const int64_t tiles = ceil_div64(numel * eb / 16, int64_t(kAmaxThreads) * kAmaxUnroll);
  const int grid = static_cast<int>(tiles < 1 ? 1 : tiles);  // <= kMaxGridBlocks by the size check
  const int64_t head = head_elems(in, eb, numel);
  if (in_dtype == DTQ_BF16)
    amax_kernel<DTQ_BF16, kAmaxUnroll><<<grid, kAmaxThreads, 0, st>>>(in, out, numel, head, ws);
  else
    amax_kernel<DTQ_F32, kAmaxUnroll><<<grid, kAmaxThreads, 0, st>>>(in, out, numel, head, ws);
  return cuda_status(cudaGetLastError());
}
