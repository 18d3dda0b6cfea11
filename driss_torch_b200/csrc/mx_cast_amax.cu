// mx_fp8_quantize that also returns max|x| of the whole tensor, from the same read.
//
// A step that quantises one tensor both ways -- tensor-wise (amax -> scale -> cast) and MX block-32 --
// reads it three times when the ops run one after the other: amax, cast, MX cast.  The MX cast
// already computes every 16-byte chunk's largest magnitude for its block scale, so the tensor's
// amax is a by-product: this kernel is mx_stream_kernel (same bytes out, see mx_cast.cu) plus a
// per-thread running maximum, folded per block into one of 32 words of the workspace (atomicMax,
// and only when the block's value exceeds what the word already holds, so that tens of thousands of
// blocks do not queue up on one address); a one-warp launch behind it reduces the 32 words, writes
// the result and leaves the workspace clean.  The step then needs two reads (this kernel, then
// dtq_cast_with_amax) instead of three.
//
// amax is the fused tensor-wise op's (src/dynamic_scaled_quant.cu:83-110: running maximum of |x|
// starting from 0, NaNs never win a comparison): the largest non-NaN magnitude, 0 if there is none;
// equal to dtq_amax's result clamped at 0.  The MX arithmetic wants the opposite for NaNs (a NaN is
// the largest magnitude), so a chunk whose largest magnitude is a NaN takes a slow path that folds
// its non-NaN elements one by one.
//
// P2P: the tensor is row-sharded over several GPUs each making this call on its shard; the
// finishing warp also exchanges the local maximum with all peers through peer-addressable memory
// (peer_exchange_max: plain st.release.sys / ld.acquire.sys over NVLink, bounded wait), so amax_out
// is the maximum over the whole tensor on every rank and the cast can follow on the same stream
// with no collective call in between.
#include "dtq_grid.cuh"
#include "dtq_host.h"
#include "mx_common.cuh"

namespace dtq {
namespace {

constexpr int64_t kL2KeepMB = 48;  // how much of the end of the input is asked to stay in L2 for the cast behind
constexpr int kThreadsA = 256;
constexpr int kUnrollA = 4;  // tied to the scale-byte mapping: lane & 3 picks the iteration

// Candidates are 15-bit bf16 magnitudes (non-negative floats order like their bits).
__device__ __forceinline__ uint32_t fold_chunk(uint32_t cand, uint4 v, uint32_t chunk_mag) {
  if (chunk_mag <= 0x7F80u) return max(cand, chunk_mag);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = w[i] & 0x7FFFu, hi = (w[i] >> 16) & 0x7FFFu;
    if (lo <= 0x7F80u) cand = max(cand, lo);
    if (hi <= 0x7F80u) cand = max(cand, hi);
  }
  return cand;
}

__device__ __forceinline__ unsigned int ld_relaxed_u32(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreadsA, 2048 / kThreadsA)
mx_amax_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
               int64_t nchunks, Workspace *ws) {
  __shared__ uint32_t warp_cand[kThreadsA / 32];
  pdl_launch_dependents();  // the finishing warp may become resident now; it waits for this grid to complete
  pdl_wait();               // and this grid itself may have become resident under the tail of the kernel before it
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int64_t kTile = int64_t(kThreadsA) * kUnrollA;
  uint32_t cand = 0;
  // The cast that follows reads the same input again, newest tiles first: the last tiles of this read are
  // loaded under an L2 evict_last policy so that they are still there.
  const uint64_t keep_policy = l2_policy_evict_last();
  const int64_t keep_from = nchunks - (kL2KeepMB << 20) / 16;
  for (int64_t tile = blockIdx.x; tile * kTile < nchunks; tile += gridDim.x) {
    const int64_t warp_first = tile * kTile + int64_t(warp) * (32 * kUnrollA);
    uint4 v[kUnrollA];
#pragma unroll
    for (int u = 0; u < kUnrollA; ++u) {
      const int64_t c = warp_first + u * 32 + lane;
      v[u] = c < nchunks ? (warp_first >= keep_from ? ldg_stream_hint(in + c, keep_policy) : ldg_stream(in + c))
                         : make_uint4(0, 0, 0, 0);
    }
    uint32_t my_scale_byte = 0;
#pragma unroll
    for (int u = 0; u < kUnrollA; ++u) {
      const int64_t c = warp_first + u * 32 + lane;
      uint32_t mag = chunk_absmax_bits(v[u]);
      cand = fold_chunk(cand, v[u], mag);  // chunks past the end were loaded as zeros
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 1));
      mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 2));
      const int biased = block_biased_exponent(mag);
      if (c < nchunks) stg_stream(payload + c * 8, mx_payload(v[u], inverse_scale(biased)));
      if ((lane & 3) == u) my_scale_byte = mx_scale_byte(biased);
    }
    // lane = 4*k + j holds the scale of block (u = j, quad k): block index u*8 + k in the warp's span.
    const int64_t blk = warp_first / 4 + (lane & 3) * 8 + (lane >> 2);
    if (blk * 4 < nchunks) scales[blk] = static_cast<uint8_t>(my_scale_byte);
  }

  // ---- fold the block's maximum into its word of the workspace
  cand = __reduce_max_sync(0xFFFFFFFFu, cand);
  if (lane == 0) warp_cand[warp] = cand;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t b = 0;
#pragma unroll
    for (int w = 0; w < kThreadsA / 32; ++w) b = max(b, warp_cand[w]);
    unsigned int *slot = &ws->slot_max[blockIdx.x & 31];
    if (b > ld_relaxed_u32(slot)) atomicMax(slot, b);  // the word only grows during a launch: a stale read costs one atomic
  }
}

// One warp, launched behind mx_amax_kernel on the same stream: reduces and clears the 32 words,
// exchanges with the peers if asked to, writes the result.
template <bool P2P>
__global__ void __launch_bounds__(32)
mx_amax_finish_kernel(float *__restrict__ amax_out, Workspace *ws, PeerExchange px) {
  const int lane = threadIdx.x;
  pdl_launch_dependents();  // a cast queued behind this launch may become resident while the maxima meet
  pdl_wait();               // every block of the MX kernel has folded its maximum
  uint32_t total = atomicExch(&ws->slot_max[lane], 0u);
  total = __reduce_max_sync(0xFFFFFFFFu, total);
  bool ok = true;
  if constexpr (P2P) total = peer_exchange_max(px, total, &ok);
  if (lane == 0) {
    if (!ok) atomicExch(&ws->status, DTQ_ERR_TIMEOUT);
    // a peer never arrived: NaN, so that nothing downstream can take the value for a maximum
    amax_out[0] = ok ? __uint_as_float(total << 16) : __uint_as_float(0x7FC00000u);
  }
}

template <bool P2P>
int launch_mx_amax(const void *in_bf16, void *payload, void *scales, float *amax_out, int64_t rows, int64_t cols,
                   void *workspace, size_t workspace_bytes, const PeerExchange &px, cudaStream_t st) {
  if (rows < 0 || cols < 0 || !amax_out) return DTQ_ERR_INVALID_ARGUMENT;
  if (cols % 32 != 0) return DTQ_ERR_SHAPE;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  const int64_t numel = rows * cols;
  if (numel > 0 && (!in_bf16 || !payload || !scales)) return DTQ_ERR_INVALID_ARGUMENT;
  // every rank must take the same kernel, so the vector path's alignment is a requirement here
  if (numel > 0 && (!aligned_to(in_bf16, 16) || !aligned_to(payload, 8))) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  const int64_t nchunks = numel / 8;
  const int64_t tiles = ceil_div64(nchunks, int64_t(kThreadsA) * kUnrollA);
  const int grid = balanced_grid(tiles, int64_t(dev.sm_count) * (1 << 20));
  Workspace *ws = static_cast<Workspace *>(workspace);
  if (numel > 0)
    DTQ_CUDA_TRY(launch_after_dependency(mx_amax_kernel, dim3(grid), dim3(kThreadsA), 0, st, static_cast<const uint4 *>(in_bf16),
                                         static_cast<uint8_t *>(payload), static_cast<uint8_t *>(scales), nchunks, ws));
  // an empty shard still takes part in the exchange
  return cuda_status(launch_after_dependency(mx_amax_finish_kernel<P2P>, dim3(1), dim3(32), 0, st, amax_out, ws, px));
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_mx_fp8_quantize_amax(const void *in_bf16, void *payload, void *scales_e8m0, float *amax_out,
                                        int64_t rows, int64_t cols, void *workspace, size_t workspace_bytes,
                                        void *stream) {
  return dtq::launch_mx_amax<false>(in_bf16, payload, scales_e8m0, amax_out, rows, cols, workspace, workspace_bytes,
                                    dtq::PeerExchange{}, static_cast<cudaStream_t>(stream));
}

extern "C" int dtq_mx_fp8_quantize_amax_p2p(const void *in_bf16, void *payload, void *scales_e8m0, float *amax_out,
                                            int64_t rows, int64_t cols, void *workspace, size_t workspace_bytes,
                                            void *const *peer_exchange, int rank, int world, uint32_t epoch,
                                            uint32_t spin_limit, void *stream) {
  using namespace dtq;
  if (!peer_exchange || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return DTQ_ERR_INVALID_ARGUMENT;
  PeerExchange px{};
  for (int r = 0; r < world; ++r) {
    if (!peer_exchange[r] || !aligned_to(peer_exchange[r], 8)) return DTQ_ERR_INVALID_ARGUMENT;
    px.buffer[r] = static_cast<unsigned long long *>(peer_exchange[r]);
  }
  px.rank = rank;
  px.world = world;
  px.epoch = epoch;
  px.spin_limit = spin_limit ? spin_limit : kSpinLimit;
  return launch_mx_amax<true>(in_bf16, payload, scales_e8m0, amax_out, rows, cols, workspace, workspace_bytes, px,
                              static_cast<cudaStream_t>(stream));
}
