// TEST INFRASTRUCTURE ONLY.  Thin extern "C" shims over the CUDA toolkit's
// host-callable number-format helpers (cuda_bf16.h / cuda_fp8.h have pure
// software host paths), the very functions the reference kernels call on the
// device (src/saturated_cast.cu:48-54,81,94-99; src/mx_cast.cu:36-41,153).
// The tests use them to pin the plain-C oracle's conversions exhaustively.
//
// Build: g++ -O2 -shared -fPIC -I/usr/local/cuda/include oracle/header_check.cpp
//            -o oracle/_build/libheader_check.so
#include <cstdint>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

static inline __nv_fp8_interpretation_t kind_of(int k) { return k == 0 ? __NV_E4M3 : __NV_E5M2; }

extern "C" {

uint8_t hdr_f32_to_fp8(float f, int kind) {
  return __nv_cvt_float_to_fp8(f, __NV_SATFINITE, kind_of(kind));
}

uint8_t hdr_bf16_to_fp8(uint16_t h, int kind) {
  __nv_bfloat16_raw r;
  r.x = h;
  return __nv_cvt_bfloat16raw_to_fp8(r, __NV_SATFINITE, kind_of(kind));
}

uint16_t hdr_f32_to_bf16(float f) {
  __nv_bfloat16 b = __float2bfloat16(f);
  uint16_t u;
  std::memcpy(&u, &b, 2);
  return u;
}

uint16_t hdr_bf16_mul(uint16_t a, uint16_t b) {
  __nv_bfloat16 x, y;
  std::memcpy(&x, &a, 2);
  std::memcpy(&y, &b, 2);
  __nv_bfloat16 p = __hmul(x, y);
  uint16_t u;
  std::memcpy(&u, &p, 2);
  return u;
}

uint8_t hdr_f32_to_fp4(float f) { return __nv_cvt_float_to_fp4(f, __NV_E2M1, cudaRoundNearest); }

uint8_t hdr_f32x2_to_fp4x2(float lo, float hi) {
  float2 v;
  v.x = lo;
  v.y = hi;
  return static_cast<uint8_t>(__nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest));
}

uint8_t hdr_f32_to_e8m0(float f) {
  return __nv_cvt_float_to_e8m0(f, __NV_SATFINITE, cudaRoundPosInf);
}

void hdr_f32_to_fp8_array(const float *in, uint8_t *out, int64_t n, int kind) {
  for (int64_t i = 0; i < n; ++i) out[i] = hdr_f32_to_fp8(in[i], kind);
}
void hdr_bf16_mul_array(const uint16_t *a, uint16_t b, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = hdr_bf16_mul(a[i], b);
}
void hdr_f32_to_bf16_array(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = hdr_f32_to_bf16(in[i]);
}
}
