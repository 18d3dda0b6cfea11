// Row-wise dynamic quantisation of a contiguous [rows, cols] matrix: per row r
//   amax_r = max |x[r,:]|;  scale_d = fp8_max / ((double)amax_r + 1e-12);
//   out[r,c] = fp8_satfinite((float)(scale_d * (double)x[r,c])).
// The reference has no such op; the arithmetic is its tensor-wise kernel's
// (src/dynamic_scaled_quant.cu:111-117) applied per row, and the per-row fp32 scales are what
// its row-wise scaled GEMM consumes (src/sweep_mm.cu:28-40).
//
// Single pass over HBM: a row is loaded into the registers of a warp (short rows) or of a CTA
// sized to the row, with all its 128-bit loads in flight at once; the row maximum is agreed by
// shuffle or through shared memory, and the payload is produced from the registers.  Rows too
// long for registers (> 32768 bf16 / 16384 fp32 elements) or not 16-byte aligned take a
// two-pass CTA-per-row kernel whose second read is served by L2.
#include <cmath>

#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <int IN>
struct RowIn;
template <>
struct RowIn<DTQ_BF16> {
  static constexpr int kElems = 8, kElemBytes = 2;
  // Running per-half max(|acc|, |w|) of packed bf16; the sign bit is garbage until `finish` masks it.
  // A NaN operand is dropped (the other operand is returned), and acc starts at 0, so acc is never NaN.
  using Acc = uint32_t;
  __device__ static Acc fold1(Acc acc, uint32_t w) {
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(acc) : "r"(acc), "r"(w));
    return acc;
  }
  __device__ static void fold(Acc &a, Acc &b, uint4 v) {
    a = fold1(fold1(a, v.x), v.z);
    b = fold1(fold1(b, v.y), v.w);
  }
  __device__ static float finish(Acc a, Acc b) {
    const uint32_t m = fold1(a, b) & 0x7FFF7FFFu;
    return fmaxf(bf16_lo(m), bf16_hi(m));
  }
  __device__ static float absmax(uint4 v) {
    Acc a = 0, b = 0;
    fold(a, b, v);
    return finish(a, b);
  }
  template <int OUT>
  __device__ static void convert_store(uint4 v, const DsqScale &s, uint8_t *dst) {
    stg_stream(dst, dsq_convert_bf16x8<OUT, true>(v, s));
  }
  __device__ static float load_one(const void *p, int64_t i) {
    return __uint_as_float(uint32_t(static_cast<const uint16_t *>(p)[i]) << 16);
  }
};
template <>
struct RowIn<DTQ_F32> {
  static constexpr int kElems = 4, kElemBytes = 4;
  using Acc = float;
  __device__ static void fold(Acc &a, Acc &b, uint4 v) {
    a = fmaxf(fmaxf(a, fabsf(__uint_as_float(v.x))), fabsf(__uint_as_float(v.z)));
    b = fmaxf(fmaxf(b, fabsf(__uint_as_float(v.y))), fabsf(__uint_as_float(v.w)));
  }
  __device__ static float finish(Acc a, Acc b) { return fmaxf(a, b); }
  __device__ static float absmax(uint4 v) {
    return fmaxf(fmaxf(fabsf(__uint_as_float(v.x)), fabsf(__uint_as_float(v.y))),
                 fmaxf(fabsf(__uint_as_float(v.z)), fabsf(__uint_as_float(v.w))));
  }
  template <int OUT>
  __device__ static void convert_store(uint4 v, const DsqScale &s, uint8_t *dst) {
    stg_stream(dst, dsq_convert_f32x4<OUT>(v, s));
  }
  __device__ static float load_one(const void *p, int64_t i) { return static_cast<const float *>(p)[i]; }
};

// A team of TEAM_WARPS warps shares a row; each thread holds up to CHUNKS 16-byte chunks of it
// (chunks_per_row = cols / kElems <= 32 * TEAM_WARPS * CHUNKS).  TEAM_WARPS == 1: a CTA is eight
// independent warps, one row each, and never synchronises.  TEAM_WARPS > 1: the CTA is the team
// (one row per CTA), so short rows get small CTAs, many of which are resident per SM and drift
// out of phase -- some loading while others convert -- which keeps HBM busy.
template <int IN, int OUT, int CHUNKS, int TEAM_WARPS>
__global__ void __launch_bounds__(TEAM_WARPS == 1 ? kThreads : 32 * TEAM_WARPS)
rowwise_regs_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ out, float *__restrict__ amax_out,
                    float *__restrict__ scale_out, int64_t rows, int chunks_per_row) {
  using R = RowIn<IN>;
  constexpr int kTeam = 32 * TEAM_WARPS;
  __shared__ float smem32[32];
  // programmatic dependent launch, both ways (see dtq_device.cuh): blocks may become resident under the tail of the
  // kernel before this one, and what is queued behind this one under its own tail
  pdl_launch_dependents();
  pdl_wait();
  int64_t row;
  int t;
  if constexpr (TEAM_WARPS == 1) {
    row = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    t = threadIdx.x & 31;
  } else {
    row = blockIdx.x;
    t = threadIdx.x;
  }
  const bool live = row < rows;

  const uint4 *src = in + row * chunks_per_row;
  uint4 v[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = t + j * kTeam;
    v[j] = (live && c < chunks_per_row) ? ldg_stream(src + c) : make_uint4(0, 0, 0, 0);
  }
  typename R::Acc acc0 = 0, acc1 = 0;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) R::fold(acc0, acc1, v[j]);
  const float a = R::finish(acc0, acc1);

  DsqScale sd;
  if constexpr (TEAM_WARPS == 1) {
    const float amax = warp_max_nonneg(a);
    if (!live) return;
    sd = make_dsq_scale<OUT>(amax);
    if (t == 0) {
      if (amax_out) amax_out[row] = amax;
      if (scale_out) scale_out[row] = static_cast<float>(sd.sd);
    }
  } else {
    float amax = block_max_nonneg(a, smem32, 0.0f);
    if (threadIdx.x == 0) smem32[0] = amax;
    __syncthreads();
    amax = smem32[0];
    sd = make_dsq_scale<OUT>(amax);
    if (t == 0) {
      if (amax_out) amax_out[row] = amax;
      if (scale_out) scale_out[row] = static_cast<float>(sd.sd);
    }
  }
  uint8_t *dst = out + row * chunks_per_row * R::kElems;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = t + j * kTeam;
    if (c < chunks_per_row) R::template convert_store<OUT>(v[j], sd, dst + int64_t(c) * R::kElems);
  }
}

// One CTA per row, two passes, any cols and any alignment (VEC = rows are 16-byte aligned and
// cols is a whole number of chunks).
template <int IN, int OUT, bool VEC>
__global__ void __launch_bounds__(kThreads)
rowwise_looped_kernel(const void *__restrict__ in, uint8_t *__restrict__ out, float *__restrict__ amax_out,
                      float *__restrict__ scale_out, int64_t rows, int64_t cols) {
  using R = RowIn<IN>;
  __shared__ float smem32[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const char *src = static_cast<const char *>(in) + row * cols * R::kElemBytes;
    uint8_t *dst = out + row * cols;
    float a = 0.0f;
    if constexpr (VEC) {
      const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
      for (int64_t c = threadIdx.x; c < cols / R::kElems; c += kThreads) a = fmaxf(a, R::absmax(ldg_keep(s4 + c)));
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += kThreads) a = fmaxf(a, fabsf(R::load_one(src, c)));
    }
    float amax = block_max_nonneg(a, smem32, 0.0f);
    __syncthreads();
    if (threadIdx.x == 0) smem32[0] = amax;
    __syncthreads();
    amax = smem32[0];
    __syncthreads();
    const DsqScale sd = make_dsq_scale<OUT>(amax);
    if (threadIdx.x == 0) {
      if (amax_out) amax_out[row] = amax;
      if (scale_out) scale_out[row] = static_cast<float>(sd.sd);
    }
    if constexpr (VEC) {
      const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
      for (int64_t c = threadIdx.x; c < cols / R::kElems; c += kThreads)
        R::template convert_store<OUT>(ldg_stream(s4 + c), sd, dst + c * R::kElems);
    } else {
      for (int64_t c = threadIdx.x; c < cols; c += kThreads) dst[c] = cvt_fp8<OUT>(dsq_mul(sd.sd, R::load_one(src, c)));
    }
  }
}

template <int IN, int OUT, int CHUNKS, int TEAM_WARPS>
int launch_regs(const void *in, void *out, float *amax_out, float *scale_out, int64_t rows, int chunks_per_row,
                cudaStream_t st) {
  const unsigned grid = static_cast<unsigned>(TEAM_WARPS == 1 ? ceil_div64(rows, kWarps) : rows);
  const int threads = TEAM_WARPS == 1 ? kThreads : 32 * TEAM_WARPS;
  return cuda_status(launch_after_dependency(rowwise_regs_kernel<IN, OUT, CHUNKS, TEAM_WARPS>, dim3(grid), dim3(threads), 0, st,
                                             static_cast<const uint4 *>(in), static_cast<uint8_t *>(out), amax_out, scale_out,
                                             rows, chunks_per_row));
}

// Smallest team that keeps a thread at <= 4 chunks (64 bytes in flight); the largest team may
// hold up to 16.
template <int IN, int OUT>
int dispatch_regs(const void *in, void *out, float *amax_out, float *scale_out, int64_t rows, int chunks,
                  cudaStream_t st) {
#define DTQ_ROW(C, W) return launch_regs<IN, OUT, C, W>(in, out, amax_out, scale_out, rows, chunks, st)
  if (chunks <= 32) DTQ_ROW(1, 1);
  if (chunks <= 64) DTQ_ROW(2, 1);
  if (chunks <= 128) DTQ_ROW(4, 1);
  if (chunks <= 256) DTQ_ROW(4, 2);
  if (chunks <= 512) DTQ_ROW(4, 4);
  if (chunks <= 1024) DTQ_ROW(4, 8);
  if (chunks <= 2048) DTQ_ROW(8, 8);
  DTQ_ROW(16, 8);
#undef DTQ_ROW
}

template <int IN, int OUT>
int launch(const void *in, void *out, float *amax_out, float *scale_out, int64_t rows, int64_t cols,
           const DeviceInfo &dev, cudaStream_t st) {
  using R = RowIn<IN>;
  const bool vec = aligned_to(in, 16) && aligned_to(out, R::kElems) && cols % R::kElems == 0;
  const int64_t chunks = cols / R::kElems;
  if (vec && chunks <= kThreads * 16)
    return dispatch_regs<IN, OUT>(in, out, amax_out, scale_out, rows, int(chunks), st);
  const int64_t max_grid = int64_t(dev.sm_count) * 8;
  const unsigned grid = static_cast<unsigned>(rows < max_grid ? rows : max_grid);
  uint8_t *o = static_cast<uint8_t *>(out);
  if (vec)
    rowwise_looped_kernel<IN, OUT, true><<<grid, kThreads, 0, st>>>(in, o, amax_out, scale_out, rows, cols);
  else
    rowwise_looped_kernel<IN, OUT, false><<<grid, kThreads, 0, st>>>(in, o, amax_out, scale_out, rows, cols);
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_dynamic_scaled_quant_rowwise(const void *in, void *out, float *amax_out, float *scale_out,
                                                int64_t rows, int64_t cols, int in_dtype, int out_dtype, void *stream) {
  using namespace dtq;
  if (rows < 0 || cols < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if ((in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) || (out_dtype != DTQ_E4M3 && out_dtype != DTQ_E5M2))
    return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (rows == 0) return DTQ_OK;
  if (cols == 0) return DTQ_ERR_SHAPE;
  if (rows > 0x7FFFFFFFLL * 8) return DTQ_ERR_TOO_LARGE;
  if (!in || !out || !aligned_to(in, in_dtype == DTQ_BF16 ? 2 : 4)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3 ? launch<DTQ_BF16, DTQ_E4M3>(in, out, amax_out, scale_out, rows, cols, dev, st)
                                 : launch<DTQ_BF16, DTQ_E5M2>(in, out, amax_out, scale_out, rows, cols, dev, st);
  return out_dtype == DTQ_E4M3 ? launch<DTQ_F32, DTQ_E4M3>(in, out, amax_out, scale_out, rows, cols, dev, st)
                               : launch<DTQ_F32, DTQ_E5M2>(in, out, amax_out, scale_out, rows, cols, dev, st);
}
