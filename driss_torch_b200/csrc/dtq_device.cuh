// Device-side building blocks shared by the quantization kernels (sm_100a).
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/dtq_b200.h"

namespace dtq {

// ---- streaming global memory access ----------------------------------------------------------
// Inputs are read exactly once and outputs written exactly once, so neither should displace
// anything in L1; reads go through the non-coherent path, writes are marked evict-first.
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Same access without the streaming hint: for data that is read again later in the same launch.
__device__ __forceinline__ uint4 ldg_keep(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void stg_stream(void *p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void stg_stream(void *p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stg_stream(void *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- number formats --------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Two fp32 -> two fp8 bytes, round-to-nearest-even, saturating to the largest finite value.
// `lo` lands in bits 0-7 (lower address), `hi` in bits 8-15.
template <int OUT>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi) {
  uint16_t r;
  if constexpr (OUT == DTQ_E4M3) {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  }
  return r;
}
template <int OUT>
__device__ __forceinline__ uint32_t cvt_fp8x4(float a, float b, float c, float d) {
  return cvt_fp8x2<OUT>(a, b) | (cvt_fp8x2<OUT>(c, d) << 16);
}
template <int OUT>
__device__ __forceinline__ uint8_t cvt_fp8(float a) {
  return static_cast<uint8_t>(cvt_fp8x2<OUT>(a, 0.0f) & 0xFFu);
}

// fp32 power of two -> E8M0 byte, rounding towards +inf, saturating (inf -> 0xFE): sm_100a only.
__device__ __forceinline__ uint8_t cvt_ue8m0(float s) {
  uint16_t r;
  asm("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(r) : "f"(s), "f"(s));
  return static_cast<uint8_t>(r & 0xFFu);
}

template <int OUT>
__device__ __forceinline__ constexpr double fp8_max() {
  return OUT == DTQ_E4M3 ? 448.0 : 57344.0;
}

// The fused ops' scale: a double, because the reference adds the double literal 1e-12.
template <int OUT>
__device__ __forceinline__ double dsq_scale(float amax) {
  return fp8_max<OUT>() / (static_cast<double>(amax) + 1e-12);
}
// (float)(scale_d * (double)x): product in double, one narrowing to fp32.
__device__ __forceinline__ float dsq_mul(double sd, float x) {
  return __double2float_rn(__dmul_rn(sd, static_cast<double>(x)));
}

// The double-precision product costs two 64-bit conversions per element on the slow
// conversion pipe, which (not HBM) bounds a kernel that uses it for every element.  The final
// fp8 byte, however, only depends on which side of an fp8 rounding boundary the reference value
//   R = fp32_rne(fp64_rne(x * scale_d))
// falls, and fp8 conversion is monotone.  So bracket R in fp32:
//   lo = fp32(scale_d * (1 - 2^-21)),  hi = fp32(scale_d * (1 + 2^-21)),
//   p_lo = fp32(x * lo),  p_hi = fp32(x * hi).
// Every rounding involved is within 2^-24 relative, so R lies between p_lo and p_hi (for either
// sign of x; underflow keeps the sign and everything that small converts to a signed zero;
// overflow saturates on both sides; NaN stays NaN).  If both ends convert to the same fp8 byte,
// that byte is fp8(R) exactly.  Otherwise (about 2^-16 of random elements) the caller recomputes
// with the double product.
struct DsqScale {
  double sd;
  float lo, hi;
};
template <int OUT>
__device__ __forceinline__ DsqScale make_dsq_scale(float amax) {
  DsqScale s;
  s.sd = dsq_scale<OUT>(amax);
  s.lo = __double2float_rn(s.sd * (1.0 - 0x1p-21));
  s.hi = __double2float_rn(s.sd * (1.0 + 0x1p-21));
  return s;
}
// Two elements -> two fp8 bytes via the lower bracket end; `mismatch` collects (by OR) the
// difference to the upper end's bytes.
template <int OUT>
__device__ __forceinline__ uint32_t dsq_pair_bracket(float x0, float x1, const DsqScale &s, uint32_t &mismatch) {
  const float2 x = make_float2(x0, x1);
  const float2 pl = __fmul2_rn(x, make_float2(s.lo, s.lo));
  const float2 ph = __fmul2_rn(x, make_float2(s.hi, s.hi));
  const uint32_t a = cvt_fp8x2<OUT>(pl.x, pl.y);
  const uint32_t b = cvt_fp8x2<OUT>(ph.x, ph.y);
  mismatch |= a ^ b;
  return a;
}
// The exact recomputation lives in functions that are never inlined, so that it stays behind a
// real branch: were it merged into the caller as predicated code, its 64-bit conversions would
// occupy the conversion pipe for every element again.
template <int OUT>
__device__ __noinline__ uint2 dsq_exact_bf16x8(uint4 v, double sd) {
  uint2 r;
  r.x = cvt_fp8x2<OUT>(dsq_mul(sd, bf16_lo(v.x)), dsq_mul(sd, bf16_hi(v.x))) |
        (cvt_fp8x2<OUT>(dsq_mul(sd, bf16_lo(v.y)), dsq_mul(sd, bf16_hi(v.y))) << 16);
  r.y = cvt_fp8x2<OUT>(dsq_mul(sd, bf16_lo(v.z)), dsq_mul(sd, bf16_hi(v.z))) |
        (cvt_fp8x2<OUT>(dsq_mul(sd, bf16_lo(v.w)), dsq_mul(sd, bf16_hi(v.w))) << 16);
  return r;
}
template <int OUT>
__device__ __noinline__ uint32_t dsq_exact_f32x4(uint4 v, double sd) {
  return cvt_fp8x4<OUT>(dsq_mul(sd, __uint_as_float(v.x)), dsq_mul(sd, __uint_as_float(v.y)),
                        dsq_mul(sd, __uint_as_float(v.z)), dsq_mul(sd, __uint_as_float(v.w)));
}
// Eight bf16 (four packed words) -> eight fp8 bytes.
template <int OUT>
__device__ __forceinline__ uint2 dsq_convert_bf16x8(uint4 v, const DsqScale &s) {
  uint32_t mismatch = 0;
  uint2 r;
  r.x = dsq_pair_bracket<OUT>(bf16_lo(v.x), bf16_hi(v.x), s, mismatch) |
        (dsq_pair_bracket<OUT>(bf16_lo(v.y), bf16_hi(v.y), s, mismatch) << 16);
  r.y = dsq_pair_bracket<OUT>(bf16_lo(v.z), bf16_hi(v.z), s, mismatch) |
        (dsq_pair_bracket<OUT>(bf16_lo(v.w), bf16_hi(v.w), s, mismatch) << 16);
  if (__builtin_expect(mismatch != 0, 0)) r = dsq_exact_bf16x8<OUT>(v, s.sd);
  return r;
}
// Four fp32 -> four fp8 bytes.
template <int OUT>
__device__ __forceinline__ uint32_t dsq_convert_f32x4(uint4 v, const DsqScale &s) {
  uint32_t mismatch = 0;
  uint32_t r = dsq_pair_bracket<OUT>(__uint_as_float(v.x), __uint_as_float(v.y), s, mismatch) |
               (dsq_pair_bracket<OUT>(__uint_as_float(v.z), __uint_as_float(v.w), s, mismatch) << 16);
  if (__builtin_expect(mismatch != 0, 0)) r = dsq_exact_f32x4<OUT>(v, s.sd);
  return r;
}

// ---- reductions of non-negative floats (or -inf) ------------------------------------------------
// Such floats order like their bit patterns read as signed ints (-inf is negative), so the
// warp-wide integer max instruction does the job exactly.
__device__ __forceinline__ float warp_max_nonneg(float v) {
  int b = __reduce_max_sync(0xFFFFFFFFu, __float_as_int(v));
  return __int_as_float(b);
}

// Block-wide max for blockDim.x a multiple of 32, up to 1024; result valid in every thread
// of warp 0.  `smem` holds 32 floats.
__device__ __forceinline__ float block_max_nonneg(float v, float *smem, float identity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_max_nonneg(v);
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = identity;
  if (warp == 0) {
    r = lane < nwarps ? smem[lane] : identity;
    r = warp_max_nonneg(r);
  }
  return r;
}

// |x| of a packed bf16 pair and of eight packed pairs' running max; NaNs are dropped by max.
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t w) {
  return *reinterpret_cast<__nv_bfloat162 *>(&w);
}
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t *>(&v); }

__device__ __forceinline__ __nv_bfloat162 absmax_bf162(__nv_bfloat162 acc, uint32_t w) {
  return __hmax2(acc, as_bf162(w & 0x7FFF7FFFu));
}
__device__ __forceinline__ float bf162_hmax_to_float(__nv_bfloat162 acc) {
  return fmaxf(__bfloat162float(acc.x), __bfloat162float(acc.y));
}

}  // namespace dtq
