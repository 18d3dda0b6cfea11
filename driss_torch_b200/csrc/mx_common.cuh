// MX (block-32, E8M0 scale, e4m3 payload) arithmetic shared by the MX kernels; identical to the
// reference's (src/mx_cast.cu:44-86 for the scale, :146-153 for payload and scale byte).
#pragma once

#include "dtq_device.cuh"

namespace dtq {

// Per-half maximum of two words of packed 15-bit bf16 magnitudes (sign bits clear): one bf16x2
// max.  NaN-propagating, so a NaN (the largest magnitudes when read as integers) still wins; it
// comes out as the canonical 0x7FFF, which has the exponent field and the non-zero mantissa of
// every other NaN, hence the same block exponent.
__device__ __forceinline__ uint32_t packed_mag_max(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// The same on signed values: per-half max(|a|, |b|), with a sign bit that is the XOR of the operands'
// signs -- garbage to be masked off once at the end of a chain (a canonical NaN included).
__device__ __forceinline__ uint32_t packed_absmax_signed(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Largest 15-bit magnitude among the eight bf16 of a 16-byte chunk.
__device__ __forceinline__ uint32_t chunk_absmax_bits(uint4 v) {
  const uint32_t m = packed_absmax_signed(packed_absmax_signed(v.x, v.y), packed_absmax_signed(v.z, v.w)) & 0x7FFF7FFFu;
  return max(m & 0xFFFFu, m >> 16);
}

// Biased exponent of the block scale from the block's largest magnitude bits.  The reference:
// e = ceil(log2 |x|) from the exponent field (+1 if the mantissa is non-zero; zero -> -128,
// subnormal -> -126), biased = clamp(e - 8 + 127, 0, 255); e is monotone in |x|, so taking the
// maximum of the raw magnitudes first gives the same block exponent as the maximum of the e_i.
// Here: (mag + 0x7F) >> 7 = exponent field + (mantissa != 0), so biased = that - 8 clamped at 0.
// For the exponent field 0 (zero and subnormals) both forms are negative before the clamp, and
// the upper clamp never acts: mag <= 0x7FFF gives at most 248.
__device__ __forceinline__ int block_biased_exponent(uint32_t mag) {
  return max(0, static_cast<int>((mag + 0x7Fu) >> 7) - 8);
}

// 1 / scale for scale = 2^(biased-127), as the reference's rcp.rn gives it: the exact power of
// two (a normal number, since biased <= 248), and +inf for scale 0 (biased 0).  Built from the
// exponent instead of running the reciprocal sequence.
__device__ __forceinline__ float inverse_scale(int biased) {
  return __uint_as_float(biased == 0 ? 0x7F800000u : static_cast<uint32_t>(254 - biased) << 23);
}

// Two packed bf16 -> two e4m3 bytes of x * inv.
__device__ __forceinline__ uint32_t mx_pair(uint32_t w, float inv) {
  const float2 p = __fmul2_rn(make_float2(bf16_lo(w), bf16_hi(w)), make_float2(inv, inv));
  return cvt_fp8x2<DTQ_E4M3>(p.x, p.y);
}

// The same from two values already widened to fp32.
__device__ __forceinline__ uint32_t mx_pair_f32(float lo, float hi, float inv) {
  const float2 p = __fmul2_rn(make_float2(lo, hi), make_float2(inv, inv));
  return cvt_fp8x2<DTQ_E4M3>(p.x, p.y);
}

__device__ __forceinline__ uint2 mx_payload(uint4 v, float inv) {
  uint2 r;
  r.x = mx_pair(v.x, inv) | (mx_pair(v.y, inv) << 16);
  r.y = mx_pair(v.z, inv) | (mx_pair(v.w, inv) << 16);
  return r;
}

// The scale byte.  The reference converts 2^(biased-127) with cvt.rp.satfinite.ue8m0x2.f32; for a
// power of two in range that is the exponent field itself, 0.0 (biased 0) gives 0, and the
// saturating case (biased 255) cannot occur (biased <= 248).
__device__ __forceinline__ uint8_t mx_scale_byte(int biased) { return static_cast<uint8_t>(biased); }

// Where the scale of MX block `blk` (row-major index over [rows, kblocks]) goes.
// Row-major: scales[blk], the reference's layout (src/mx_cast.cu:199,210-211).
// Blocked: the layout the reference's MX GEMM consumes (src/mx_fp8_bf16.cu:97-110, CUTLASS
// Sm1xxBlockScaledConfig::tile_atom_to_shape_SFA; the reference gets there through a separate
// `to_blocked` pass, test/test_mx.py:28-32): 128-row x 4-k-block atoms of 512 bytes, atoms ordered
// k-block-major within a 128-row band; inside an atom row r, k-block c sit at
// (r % 32) * 16 + (r / 32) * 4 + c.
template <bool BLOCKED>
__device__ __forceinline__ int64_t scale_offset(int64_t blk, int64_t kblocks, int64_t katoms) {
  if constexpr (!BLOCKED) return blk;
  const int64_t r = blk / kblocks, c = blk - r * kblocks;
  const int64_t atom = (r >> 7) * katoms + (c >> 2);
  return atom * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3);
}

}  // namespace dtq
