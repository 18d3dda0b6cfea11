// MX (block-32, E8M0 scale, e4m3 payload) arithmetic shared by the MX kernels; identical to the
// reference's (src/mx_cast.cu:44-86 for the scale, :146-153 for payload and scale byte).
#pragma once

#include "dtq_device.cuh"

namespace dtq {

// Largest 15-bit magnitude among the eight bf16 of a 16-byte chunk.
__device__ __forceinline__ uint32_t chunk_absmax_bits(uint4 v) {
  const uint32_t m = __vmaxu2(__vmaxu2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu),
                              __vmaxu2(v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu));
  return max(m & 0xFFFFu, m >> 16);
}

// Biased exponent of the block scale from the block's largest magnitude bits:
// e = ceil(log2 |x|) from the exponent field (+1 if the mantissa is non-zero; zero -> -128,
// subnormal -> -126), biased = clamp(e - 8 + 127, 0, 255).  e is monotone in |x|, so taking the
// maximum of the raw magnitudes first gives the same block exponent as the maximum of the e_i.
__device__ __forceinline__ int block_biased_exponent(uint32_t mag) {
  const int be = static_cast<int>(mag >> 7);
  int e = be - 127 + ((mag & 0x7Fu) != 0);
  if (be == 0) e = (mag == 0) ? -128 : -126;
  return min(255, max(0, e - 8 + 127));
}

// 1 / scale for scale = 2^(biased-127), as the reference's rcp.rn gives it: exact for every power
// of two (2^-127 is the subnormal 0x00400000), +inf for scale 0 (biased 0), 0 for scale +inf
// (biased 255).  Built from the exponent instead of running the reciprocal sequence.
__device__ __forceinline__ float inverse_scale(int biased) {
  const int e = 254 - biased;  // exponent field of the reciprocal
  uint32_t bits = static_cast<uint32_t>(e) << 23;
  if (e <= 0) bits = e == 0 ? 0x00400000u : 0u;
  if (biased == 0) bits = 0x7F800000u;
  return __uint_as_float(bits);
}

// Two packed bf16 -> two e4m3 bytes of x * inv.
__device__ __forceinline__ uint32_t mx_pair(uint32_t w, float inv) {
  const float2 p = __fmul2_rn(make_float2(bf16_lo(w), bf16_hi(w)), make_float2(inv, inv));
  return cvt_fp8x2<DTQ_E4M3>(p.x, p.y);
}

__device__ __forceinline__ uint2 mx_payload(uint4 v, float inv) {
  uint2 r;
  r.x = mx_pair(v.x, inv) | (mx_pair(v.y, inv) << 16);
  r.y = mx_pair(v.z, inv) | (mx_pair(v.w, inv) << 16);
  return r;
}

// The scale byte: cvt.rp.satfinite.ue8m0 of 2^(biased-127) = biased, with 255 (+inf) clamped to 0xFE.
__device__ __forceinline__ uint8_t mx_scale_byte(int biased) { return cvt_ue8m0(__int_as_float(biased << 23)); }

}  // namespace dtq
