// MX block-32 quantisation for the element formats and input types the reference's schema names
// but its kernel does not compute: the reference accepts fp8_type = e5m2 and fp16 / fp32 inputs
// and then runs the bf16 -> e4m3 arithmetic on whatever bytes it was given
// (src/mx_cast.cu:148,175-184,204), and its MXFP4 GEMM (src/mx_fp8_bf16.cu:243-271) has no
// producer kernel at all.  This file applies the reference's scale rule, generalised only in the
// element format's largest exponent:
//   e_i = ceil(log2 |float(x_i)|) from the fp32 exponent field (+1 if the mantissa is non-zero;
//         zero -> -128, fp32 subnormal -> -126)                      (src/mx_cast.cu:50-65)
//   biased = clamp(max_i e_i - EMAX + 127, 0, 255),  scale = 2^(biased-127)   (:68-85)
//   payload_i = convert_satfinite(float(x_i) * (1 / scale))           (:146-149)
//   scale byte = biased                                               (:153)
// with EMAX = 8 for e4m3 (the reference's constant), 15 for e5m2, 2 for e2m1: the exponent of the
// format's largest power of two, so that |x| / scale <= 2^EMAX never saturates.  The reference's
// behaviour for blocks that are all zero or tiny (scale 0 -> 1/scale = inf -> 0 * inf = NaN) is
// kept: NaN bytes (0x7F) in the fp8 formats; e2m1 has no NaN and the conversion gives +6 (0x7).
// For bf16 input and e4m3 this is dtq_mx_fp8_quantize's arithmetic (tested equal).
// e2m1 payloads are packed two per byte, the element with the lower index in the low nibble.
//
// Structure: the flat stream of mx_cast.cu.  A lane owns a 16-byte chunk (8 bf16 / fp16 or 4 fp32
// values), 4 or 8 neighbouring lanes form a block and agree on the largest magnitude with 2 or 3
// shuffles; magnitudes are compared as integers (monotone in |x| for each input format).
#include <cuda_fp16.h>

#include "dtq_host.h"
#include "mx_common.cuh"

namespace dtq {
namespace {

constexpr int kThreadsF = 256;
constexpr int kUnrollF = 4;

// ---- input formats ------------------------------------------------------------------------------------
template <int IN>
struct MxIn;

template <>
struct MxIn<DTQ_BF16> {
  static constexpr int kElems = 8;
  __device__ static uint32_t key(uint4 v) { return chunk_absmax_bits(v); }
  // exponent field + (mantissa != 0) of the fp32 value of the block's largest magnitude
  __device__ static int exp_plus(uint32_t key) { return static_cast<int>((key + 0x7Fu) >> 7); }
  __device__ static void unpack(uint4 v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
};

template <>
struct MxIn<DTQ_F16> {
  static constexpr int kElems = 8;
  __device__ static uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t r;  // NaN-propagating like packed_mag_max; the canonical fp16 NaN 0x7FFF widens to an fp32 NaN
    asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
  }
  __device__ static uint32_t key(uint4 v) {
    const uint32_t m = max2(max2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu), max2(v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu));
    return max(m & 0xFFFFu, m >> 16);
  }
  __device__ static int exp_plus(uint32_t key) {
    const uint32_t bits = __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(key))));
    return static_cast<int>((bits + 0x7FFFFFu) >> 23);  // fp16 subnormals are fp32 normals
  }
  __device__ static void unpack(uint4 v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
};

template <>
struct MxIn<DTQ_F32> {
  static constexpr int kElems = 4;
  __device__ static uint32_t key(uint4 v) {
    return max(max(v.x & 0x7FFFFFFFu, v.y & 0x7FFFFFFFu), max(v.z & 0x7FFFFFFFu, v.w & 0x7FFFFFFFu));
  }
  __device__ static int exp_plus(uint32_t key) { return static_cast<int>((key + 0x7FFFFFu) >> 23); }
  __device__ static void unpack(uint4 v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};

// ---- element formats ----------------------------------------------------------------------------------
// Two fp32 -> two e2m1 nibbles in one byte, round-to-nearest-even, saturating; `lo` in bits 0-3.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t r;
  asm("{ .reg .b8 t;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\t"
      "mov.b16 %0, {t, 0}; }"
      : "=h"(r)
      : "f"(hi), "f"(lo));
  return r;
}

template <int FMT>
struct MxOut;
template <>
struct MxOut<DTQ_E4M3> {
  static constexpr int kEmax = 8, kBitsPerElem = 8;
  __device__ static uint32_t two(float a, float b) { return cvt_fp8x2<DTQ_E4M3>(a, b); }
};
template <>
struct MxOut<DTQ_E5M2> {
  static constexpr int kEmax = 15, kBitsPerElem = 8;
  __device__ static uint32_t two(float a, float b) { return cvt_fp8x2<DTQ_E5M2>(a, b); }
};
template <>
struct MxOut<DTQ_E2M1> {
  static constexpr int kEmax = 2, kBitsPerElem = 4;
  __device__ static uint32_t two(float a, float b) { return cvt_e2m1x2(a, b); }
};

// 1 / 2^(biased-127) for biased in [0, 254]: +inf for scale 0, the subnormal 2^-127 for biased 254.
__device__ __forceinline__ float inverse_scale_wide(int biased) {
  const int e = 254 - biased;
  return __uint_as_float(biased == 0 ? 0x7F800000u : (e > 0 ? static_cast<uint32_t>(e) << 23 : 0x00400000u));
}

// Stores the converted chunk: kElems * bits / 8 bytes.
template <int N, int FMT>
__device__ __forceinline__ void convert_store(const float (&f)[N], float inv, uint8_t *dst) {
  using O = MxOut<FMT>;
  uint32_t pair[N / 2];  // 16 bits (fp8) or 8 bits (e2m1) each
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float2 p = __fmul2_rn(make_float2(f[2 * i], f[2 * i + 1]), make_float2(inv, inv));
    pair[i] = O::two(p.x, p.y);
  }
  if constexpr (O::kBitsPerElem == 8 && N == 8) {
    stg_stream(dst, make_uint2(pair[0] | (pair[1] << 16), pair[2] | (pair[3] << 16)));
  } else if constexpr (O::kBitsPerElem == 8 && N == 4) {
    stg_stream(dst, pair[0] | (pair[1] << 16));
  } else if constexpr (N == 8) {
    stg_stream(dst, pair[0] | (pair[1] << 8) | (pair[2] << 16) | (pair[3] << 24));
  } else {
    *reinterpret_cast<uint16_t *>(dst) = static_cast<uint16_t>(pair[0] | (pair[1] << 8));
  }
}

// nchunks 16-byte chunks; a block of 32 elements is kLanes consecutive chunks (never split across warps).
template <int IN, int FMT>
__global__ void __launch_bounds__(kThreadsF, 2048 / kThreadsF)
mx_formats_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
                  int64_t nchunks, int64_t kblocks) {  // kblocks > 0: scales in the MX GEMM's blocked layout, that many per row
  // programmatic dependent launch, both ways (see dtq_device.cuh): blocks may become resident under the tail of the
  // kernel before this one, and what is queued behind this one under its own tail
  pdl_launch_dependents();
  pdl_wait();
  using I = MxIn<IN>;
  using O = MxOut<FMT>;
  constexpr int kLanes = 32 / I::kElems;                        // lanes per MX block
  constexpr int kChunkBytesOut = I::kElems * O::kBitsPerElem / 8;
  const int lane = threadIdx.x & 31;
  constexpr int64_t kTile = int64_t(kThreadsF) * kUnrollF;
  for (int64_t tile = blockIdx.x; tile * kTile < nchunks; tile += gridDim.x) {
    const int64_t first = tile * kTile + threadIdx.x;
    uint4 v[kUnrollF];
#pragma unroll
    for (int u = 0; u < kUnrollF; ++u) {
      const int64_t c = first + u * kThreadsF;  // nchunks % kLanes == 0: a block is inside or outside as a whole
      v[u] = c < nchunks ? ldg_stream(in + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnrollF; ++u) {
      const int64_t c = first + u * kThreadsF;
      uint32_t key = I::key(v[u]);
#pragma unroll
      for (int d = 1; d < kLanes; d <<= 1) key = max(key, __shfl_xor_sync(0xFFFFFFFFu, key, d));
      const int biased = max(0, I::exp_plus(key) - O::kEmax);  // at most 256 - 2 = 254: no upper clamp needed
      if (c < nchunks) {
        float f[I::kElems];
        I::unpack(v[u], f);
        convert_store<I::kElems, FMT>(f, inverse_scale_wide(biased), payload + c * kChunkBytesOut);
        if ((lane & (kLanes - 1)) == 0) {
          const int64_t blk = c / kLanes;
          scales[kblocks > 0 ? scale_offset<true>(blk, kblocks, (kblocks + 3) / 4) : blk] = static_cast<uint8_t>(biased);
        }
      }
    }
  }
}

template <int IN, int FMT>
int launch_formats(const void *in, void *payload, void *scales, int64_t numel, int64_t kblocks, const DeviceInfo &dev,
                   cudaStream_t st) {
  using I = MxIn<IN>;
  constexpr int kChunkBytesOut = I::kElems * MxOut<FMT>::kBitsPerElem / 8;
  if (!aligned_to(in, 16) || !aligned_to(payload, kChunkBytesOut)) return DTQ_ERR_INVALID_ARGUMENT;
  const int64_t nchunks = numel / I::kElems;
  const int64_t tiles = ceil_div64(nchunks, int64_t(kThreadsF) * kUnrollF);
  const int grid = balanced_grid(tiles, int64_t(dev.sm_count) * (1 << 20));
  return cuda_status(launch_after_dependency(mx_formats_kernel<IN, FMT>, dim3(grid), dim3(kThreadsF), 0, st,
                                             static_cast<const uint4 *>(in), static_cast<uint8_t *>(payload),
                                             static_cast<uint8_t *>(scales), nchunks, kblocks));
}

template <int IN>
int launch_by_format(int fmt, const void *in, void *payload, void *scales, int64_t numel, int64_t kblocks,
                     const DeviceInfo &dev, cudaStream_t st) {
  switch (fmt) {
    case DTQ_E4M3: return launch_formats<IN, DTQ_E4M3>(in, payload, scales, numel, kblocks, dev, st);
    case DTQ_E5M2: return launch_formats<IN, DTQ_E5M2>(in, payload, scales, numel, kblocks, dev, st);
    default: return launch_formats<IN, DTQ_E2M1>(in, payload, scales, numel, kblocks, dev, st);
  }
}

int mx_quantize_any(const void *in, void *payload, void *scales_e8m0, int64_t rows, int64_t cols, int in_dtype, int elem_format,
                    bool blocked, void *stream) {
  if (rows < 0 || cols < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (in_dtype != DTQ_BF16 && in_dtype != DTQ_F32 && in_dtype != DTQ_F16) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (elem_format != DTQ_E4M3 && elem_format != DTQ_E5M2 && elem_format != DTQ_E2M1) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (cols % 32 != 0) return DTQ_ERR_SHAPE;
  const int64_t numel = rows * cols;
  if (numel == 0) return DTQ_OK;
  if (!in || !payload || !scales_e8m0) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t kblocks = blocked ? cols / 32 : 0;
  switch (in_dtype) {
    case DTQ_BF16: return launch_by_format<DTQ_BF16>(elem_format, in, payload, scales_e8m0, numel, kblocks, dev, st);
    case DTQ_F16: return launch_by_format<DTQ_F16>(elem_format, in, payload, scales_e8m0, numel, kblocks, dev, st);
    default: return launch_by_format<DTQ_F32>(elem_format, in, payload, scales_e8m0, numel, kblocks, dev, st);
  }
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_mx_quantize(const void *in, void *payload, void *scales_e8m0, int64_t rows, int64_t cols,
                               int in_dtype, int elem_format, void *stream) {
  return dtq::mx_quantize_any(in, payload, scales_e8m0, rows, cols, in_dtype, elem_format, false, stream);
}

extern "C" int dtq_mx_quantize_blocked(const void *in, void *payload, void *scales_blocked, int64_t rows, int64_t cols,
                                       int in_dtype, int elem_format, void *stream) {
  return dtq::mx_quantize_any(in, payload, scales_blocked, rows, cols, in_dtype, elem_format, true, stream);
}
