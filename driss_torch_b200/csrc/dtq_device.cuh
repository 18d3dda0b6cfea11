// Device-side building blocks shared by the quantization kernels (sm_100a).
#pragma once

#include <cmath>
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
// The same load with an L2 eviction policy attached (see l2_policy_evict_last): for data that the
// same launch reads again and that should therefore outlive the streaming traffic in L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ldg_stream_hint(const void *p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
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

// ---- programmatic dependent launch ------------------------------------------------------------
// Two kernels queued back to back on one stream normally run strictly one after the other: the
// second is launched when the first has drained.  A kernel launched with the programmatic-
// serialization attribute (launch_after_dependency in dtq_host.h) may instead become resident as
// soon as every block of its predecessor has executed pdl_launch_dependents (or exited); it must
// then execute pdl_wait before it touches anything the predecessor reads or writes: the wait
// returns when the predecessor has completed and its memory operations are visible.  Launch
// latency and the ramp of the second kernel hide under the tail of the first.  Both instructions
// are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Asks L2 to fetch `bytes` (a multiple of 16) from the 16-byte aligned global address `p`.  Nothing is
// delivered to the thread and nothing observable changes: L2 is where this GPU's memory is kept coherent,
// so a line fetched early is the line a later load would have fetched, whoever writes it in between.
__device__ __forceinline__ void l2_prefetch_bulk(const void *p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
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

// ---- the double-precision product without the 64-bit conversion pipe -----------------------------
// Done literally, (float)(scale_d * (double)x) costs two 64-bit conversions per element on the
// conversion (XU) pipe, and that pipe, not HBM, then bounds the kernel.  Two exact substitutes:
//
// (A) compensated fp32, for bf16 x and a bf16-valued amax in [0.25, 2^64] -- the normal case, amax
//     being an element of the tensor.  With head = fp32(sd), tail = fp32(sd - head):
//       r1 = fp32(x*head), c = fma(x, head, -r1) (exact), c2 = fma(x, tail, c), R' = fp32(r1 + c2).
//     r1 + c2 differs from P = x*sd by < 2^-46 |P|, so R' equals the reference
//     R = fp32(fp64(P)) unless P lies within 2^-46 of an fp32 rounding midpoint.  It cannot:
//     P = Q(1+theta) with Q = 7n 2^k / m (n, m <= 255 the integer mantissas of x and amax; both fp8
//     maxima are 7 * 2^j) and |theta| <= 1e-12/amax + 2^-51 <= 2^-36.9.  If m divides 7n 2^i, Q has
//     at most 11 significant bits, is an fp32 number, and P stays within 2^-36.9 of it; otherwise
//     |Q - M| >= 2^-33 |Q| for every 25-bit midpoint M (the difference of the two fractions is a
//     non-zero integer over m times a power of two).  Results below the fp32 normal range convert to
//     a signed zero either way; the sign is copied from x.  Products that overflow fp32 (possible
//     only when the caller's amax is smaller than |x|) are detected and left infinite.
//     This matters because with bf16 data about one e4m3 product in 128 sits exactly on an fp8
//     rounding tie (sd is a ratio of small integers), so any scheme that falls back to fp64 "near
//     a boundary" falls back in almost every warp.
// (B) bracket, for everything else (fp32 x, arbitrary amax): fp8 conversion is monotone, so if
//       fp8(fp32(x * fp32(sd(1 - 2^-21)))) == fp8(fp32(x * fp32(sd(1 + 2^-21))))
//     that byte is fp8(R) (every rounding involved is within 2^-24; underflow keeps the sign,
//     overflow saturates on both sides, NaN stays NaN); otherwise the pair is recomputed in fp64 by
//     a never-inlined function, so that the 64-bit conversions stay behind a real branch.
struct DsqScale {
  double sd;
  float lo, hi;      // (B) bracket ends
  float head, tail;  // (A) sd = head + tail + O(2^-48 sd)
  bool compensated;  // (A) is valid for bf16 inputs
};
template <int OUT>
__device__ __forceinline__ DsqScale make_dsq_scale(float amax) {
  DsqScale s;
  s.sd = dsq_scale<OUT>(amax);
  s.lo = __double2float_rn(s.sd * (1.0 - 0x1p-21));
  s.hi = __double2float_rn(s.sd * (1.0 + 0x1p-21));
  s.head = __double2float_rn(s.sd);
  s.tail = __double2float_rn(s.sd - static_cast<double>(s.head));
  s.compensated = (__float_as_uint(amax) & 0xFFFFu) == 0u && amax >= 0.25f && amax <= 0x1p64f;
  return s;
}

// (A) two bf16-valued elements -> two fp8 bytes.  BOUNDED: the caller guarantees |x| <= amax (or
// NaN), so no product overflows.
template <int OUT, bool BOUNDED>
__device__ __forceinline__ uint32_t dsq_pair_compensated(float x0, float x1, const DsqScale &s) {
  const float2 x = make_float2(x0, x1);
  const float2 h = make_float2(s.head, s.head);
  const float2 q = __fmul2_rn(x, make_float2(-s.head, -s.head));  // -r1
  const float2 c = __ffma2_rn(x, h, q);                           // x*head - r1, exact
  const float2 c2 = __ffma2_rn(x, make_float2(s.tail, s.tail), c);
  float2 r = __ffma2_rn(q, make_float2(-1.0f, -1.0f), c2);        // r1 + c2, one rounding
  if (!BOUNDED) {
    if (fabsf(q.x) == INFINITY) r.x = -q.x;
    if (fabsf(q.y) == INFINITY) r.y = -q.y;
  }
  return cvt_fp8x2<OUT>(copysignf(r.x, x0), copysignf(r.y, x1));
}

// (B) two elements -> the fp8 bytes of the lower bracket end and of the upper end.
template <int OUT>
__device__ __forceinline__ void dsq_pair_bracket(float x0, float x1, const DsqScale &s, uint32_t &lo_bytes,
                                                 uint32_t &hi_bytes) {
  const float2 x = make_float2(x0, x1);
  const float2 pl = __fmul2_rn(x, make_float2(s.lo, s.lo));
  const float2 ph = __fmul2_rn(x, make_float2(s.hi, s.hi));
  lo_bytes = cvt_fp8x2<OUT>(pl.x, pl.y);
  hi_bytes = cvt_fp8x2<OUT>(ph.x, ph.y);
}
// fp32 -> fp64 is exact, so normal numbers are widened on the integer pipe (re-bias the exponent,
// move the mantissa); zeros, subnormals, infinities and NaNs take the conversion instruction.
__device__ __forceinline__ double widen_exact(float x) {
  const uint32_t w = __float_as_uint(x);
  const uint32_t a = w & 0x7FFFFFFFu;
  const uint32_t e = a >> 23;
  if (e - 1u >= 254u) return static_cast<double>(x);
  return __hiloint2double(static_cast<int>((w & 0x80000000u) | ((a >> 3) + 0x38000000u)), static_cast<int>(w << 29));
}
template <int OUT>
__device__ __forceinline__ uint32_t dsq_pair_exact(float x0, float x1, double sd) {
  return cvt_fp8x2<OUT>(__double2float_rn(__dmul_rn(sd, widen_exact(x0))),
                        __double2float_rn(__dmul_rn(sd, widen_exact(x1))));
}
// `r` = bytes of the lower bracket end, `m` = xor with the upper end's bytes: a non-zero 16-bit
// half marks a pair to redo.
template <int OUT>
__device__ __noinline__ uint2 dsq_redo_bf16x8(uint4 v, uint2 r, uint2 m, double sd) {
  if (m.x & 0xFFFFu) r.x = (r.x & 0xFFFF0000u) | dsq_pair_exact<OUT>(bf16_lo(v.x), bf16_hi(v.x), sd);
  if (m.x >> 16) r.x = (r.x & 0xFFFFu) | (dsq_pair_exact<OUT>(bf16_lo(v.y), bf16_hi(v.y), sd) << 16);
  if (m.y & 0xFFFFu) r.y = (r.y & 0xFFFF0000u) | dsq_pair_exact<OUT>(bf16_lo(v.z), bf16_hi(v.z), sd);
  if (m.y >> 16) r.y = (r.y & 0xFFFFu) | (dsq_pair_exact<OUT>(bf16_lo(v.w), bf16_hi(v.w), sd) << 16);
  return r;
}
template <int OUT>
__device__ __noinline__ uint32_t dsq_redo_f32x4(uint4 v, uint32_t r, uint32_t m, double sd) {
  if (m & 0xFFFFu) r = (r & 0xFFFF0000u) | dsq_pair_exact<OUT>(__uint_as_float(v.x), __uint_as_float(v.y), sd);
  if (m >> 16) r = (r & 0xFFFFu) | (dsq_pair_exact<OUT>(__uint_as_float(v.z), __uint_as_float(v.w), sd) << 16);
  return r;
}
// Eight bf16 (four packed words) -> eight fp8 bytes.
template <int OUT, bool BOUNDED>
__device__ __forceinline__ uint2 dsq_convert_bf16x8(uint4 v, const DsqScale &s) {
  if (s.compensated) {
    return make_uint2(dsq_pair_compensated<OUT, BOUNDED>(bf16_lo(v.x), bf16_hi(v.x), s) |
                          (dsq_pair_compensated<OUT, BOUNDED>(bf16_lo(v.y), bf16_hi(v.y), s) << 16),
                      dsq_pair_compensated<OUT, BOUNDED>(bf16_lo(v.z), bf16_hi(v.z), s) |
                          (dsq_pair_compensated<OUT, BOUNDED>(bf16_lo(v.w), bf16_hi(v.w), s) << 16));
  }
  uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
  dsq_pair_bracket<OUT>(bf16_lo(v.x), bf16_hi(v.x), s, a0, b0);
  dsq_pair_bracket<OUT>(bf16_lo(v.y), bf16_hi(v.y), s, a1, b1);
  dsq_pair_bracket<OUT>(bf16_lo(v.z), bf16_hi(v.z), s, a2, b2);
  dsq_pair_bracket<OUT>(bf16_lo(v.w), bf16_hi(v.w), s, a3, b3);
  uint2 r = make_uint2(a0 | (a1 << 16), a2 | (a3 << 16));
  const uint2 m = make_uint2(r.x ^ (b0 | (b1 << 16)), r.y ^ (b2 | (b3 << 16)));
  if (__builtin_expect((m.x | m.y) != 0, 0)) r = dsq_redo_bf16x8<OUT>(v, r, m, s.sd);
  return r;
}
// Four fp32 -> four fp8 bytes.
template <int OUT>
__device__ __forceinline__ uint32_t dsq_convert_f32x4(uint4 v, const DsqScale &s) {
  uint32_t a0, a1, b0, b1;
  dsq_pair_bracket<OUT>(__uint_as_float(v.x), __uint_as_float(v.y), s, a0, b0);
  dsq_pair_bracket<OUT>(__uint_as_float(v.z), __uint_as_float(v.w), s, a1, b1);
  uint32_t r = a0 | (a1 << 16);
  const uint32_t m = r ^ (b0 | (b1 << 16));
  if (__builtin_expect(m != 0, 0)) r = dsq_redo_f32x4<OUT>(v, r, m, s.sd);
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
