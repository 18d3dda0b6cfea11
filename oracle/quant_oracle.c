/*
 * TEST INFRASTRUCTURE ONLY -- never linked into, imported by, or called from
 * the product path.  A plain-C CPU restatement of the arithmetic of the
 * reference's FP8 / MX quantization kernels, used as the checker by the tests,
 * by the smoke check, and (timed) as the CPU baseline of the benchmark.
 *
 * Parity status: pinned.  (1) The one known-answer vector in the reference's
 * tests (test/test_sat_cast.py:65-83) is checked on CPU.  (2) Golden fixtures
 * under tests/golden/ were produced by the unmodified reference CUDA kernels
 * on a B200 (tests/golden/make_golden.py) and are checked on CPU.  (3) The
 * number-format conversions are checked exhaustively against the CUDA
 * toolkit's host-callable header implementations (oracle/header_check.cpp).
 *
 * Every function cites the reference lines it restates.  Conversions are done
 * by value (scale to an integer grid, round half to even with rint() under the
 * default rounding mode), deliberately a different formulation from the
 * bit-twiddling in the toolkit headers so that the two can check each other.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC oracle/quant_oracle.c -o oracle/_build/libquant_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_BF16 0
#define ORACLE_F32 1
#define ORACLE_E4M3 0
#define ORACLE_E5M2 1

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* One rounding (nearest, ties to even) of a double to bfloat16, subnormals
 * kept, overflow to infinity, NaN to the canonical 0x7FFF that the device
 * multiply and conversion produce. */
static uint16_t f64_to_bf16_rne(double d) {
  if (isnan(d)) return 0x7FFF;
  uint16_t sign = signbit(d) ? 0x8000 : 0;
  double a = fabs(d);
  if (a == 0.0) return sign;
  if (isinf(a)) return sign | 0x7F80;
  int e;
  (void)frexp(a, &e); /* a = m * 2^e, m in [0.5, 1)  ->  floor(log2 a) = e - 1 */
  int fl = e - 1;
  if (fl < -126) fl = -126;      /* subnormal grid */
  double q = ldexp(1.0, fl - 7); /* spacing of bf16 values at this exponent */
  double v = rint(a / q) * q;    /* a / q is exact (power of two) */
  if (v >= ldexp(1.0, 128)) return sign | 0x7F80;
  float f = (float)v; /* exact: v has at most 8 significant bits */
  return sign | (uint16_t)(f32_bits(f) >> 16);
}

/* fp8 conversion with the semantics of cvt.rn.satfinite.{e4m3x2,e5m2x2}.f32:
 * nearest-even, magnitudes above the largest finite value (infinities too)
 * clamp to it, NaN -> 0x7F.  The reference reaches it through
 * __nv_cvt_float_to_fp8 / __nv_cvt_bfloat16raw_to_fp8 with __NV_SATFINITE
 * (src/saturated_cast.cu:49-54,94-99; src/dynamic_scaled_quant.cu:76-81;
 * src/mx_cast.cu:36-41). */
static uint8_t f32_to_fp8_sat(float x, int kind) {
  const int mbits = (kind == ORACLE_E4M3) ? 3 : 2;
  const int bias = (kind == ORACLE_E4M3) ? 7 : 15;
  const int emin = 1 - bias; /* exponent of the smallest normal */
  const double vmax = (kind == ORACLE_E4M3) ? 448.0 : 57344.0;
  const uint8_t cmax = (kind == ORACLE_E4M3) ? 0x7E : 0x7B;
  if (isnan(x)) return 0x7F;
  uint8_t sign = signbit(x) ? 0x80 : 0;
  double a = fabs((double)x);
  if (a > vmax) return sign | cmax;
  if (a == 0.0) return sign;
  int e;
  (void)frexp(a, &e);
  int fl = e - 1;
  if (fl < emin) fl = emin;
  double q = ldexp(1.0, fl - mbits);
  long n = (long)rint(a / q); /* in [0, 2^(mbits+1)] */
  if (n == (1L << (mbits + 1))) { n >>= 1; fl += 1; }
  uint8_t code;
  if (n < (1L << mbits)) code = (uint8_t)n; /* subnormal or zero (fl == emin) */
  else code = (uint8_t)(((fl + bias) << mbits) | (n - (1L << mbits)));
  return sign | code;
}

static inline float load_f32(const void *in, int in_dtype, int64_t i) {
  return in_dtype == ORACLE_BF16 ? bf16_to_f32(((const uint16_t *)in)[i]) : ((const float *)in)[i];
}

/* ---- saturated_cast: src/saturated_cast.cu:38-57 (one element per thread) and
 * :59-104 (packed pairs); both compute the same per-element value.
 * bf16 input: the fp32 scale is first rounded to bf16 (implicit conversion when
 * the packed scale is built, :66; __hmul's float argument, :48), the product is
 * a bf16 multiply (one rounding of the exact product to bf16, :48,81), then
 * bf16 -> fp32 -> fp8 (:49-50,94-96).  fp32 input: fp32 multiply, then fp8
 * (:52-54,84-85,98-99).  The op is elementwise over the flat storage. */
void oracle_saturated_cast(const void *in, int in_dtype, float scale, uint8_t *out, int64_t n,
                           int out_kind) {
  if (in_dtype == ORACLE_BF16) {
    const uint16_t *x = (const uint16_t *)in;
    double sb = (double)bf16_to_f32(f64_to_bf16_rne((double)scale));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      double prod = (double)bf16_to_f32(x[i]) * sb; /* exact in double */
      float p = bf16_to_f32(f64_to_bf16_rne(prod));
      out[i] = f32_to_fp8_sat(p, out_kind);
    }
  } else {
    const float *x = (const float *)in;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      volatile float p = x[i] * scale; /* one fp32 rounding, no contraction */
      out[i] = f32_to_fp8_sat(p, out_kind);
    }
  }
}

/* ---- amax: src/amax.cu:50-80.  max |x| as fp32, starting from -inf (:52 and the
 * -inf fill at :115); the comparisons drop NaNs (__hmax / max return the non-NaN
 * operand, :60-65).  Order independent, so any reduction order is exact. */
float oracle_amax(const void *in, int in_dtype, int64_t n) {
  float best = -INFINITY;
#pragma omp parallel
  {
    float mine = -INFINITY;
#pragma omp for schedule(static) nowait
    for (int64_t i = 0; i < n; ++i) {
      float a = fabsf(load_f32(in, in_dtype, i));
      if (a > mine) mine = a; /* false for NaN: dropped */
    }
#pragma omp critical
    { if (mine > best) best = mine; }
  }
  return best;
}

/* The cast phase of the fused op, src/dynamic_scaled_quant.cu:111-117: the scale
 * is a double because the literal 1e-12 is one (:111); the product is formed in
 * double, narrowed to fp32 on the way into __nv_cvt_float_to_fp8 (:76-81,115-116).
 * fp8 max is 448 / 57344 (:43-53). */
static inline double dsq_scale(float amax, int out_kind) {
  double fmax = (out_kind == ORACLE_E4M3) ? 448.0 : 57344.0;
  return fmax / ((double)amax + 1e-12);
}

void oracle_cast_with_amax(const void *in, int in_dtype, float amax, uint8_t *out, int64_t n,
                           int out_kind, float *scale_out) {
  if (!(amax > 0.0f)) amax = 0.0f; /* phase 1 starts from 0: never negative, never NaN */
  double sd = dsq_scale(amax, out_kind);
  if (scale_out) *scale_out = (float)sd;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float p = (float)(sd * (double)load_f32(in, in_dtype, i));
    out[i] = f32_to_fp8_sat(p, out_kind);
  }
}

/* ---- dynamic_scaled_quant: src/dynamic_scaled_quant.cu:83-118.  Phase 1 is
 * max |x| starting from 0 (:92,97-101; the scratch is zero-filled, :171); NaN
 * handling in the reference depends on thread order, here NaNs are dropped.
 * bf16 input is defined as the same arithmetic on float(x) (the reference
 * instantiates fp32 only, :130,147). */
void oracle_dynamic_scaled_quant(const void *in, int in_dtype, uint8_t *out, int64_t n, int out_kind,
                                 float *amax_out, float *scale_out) {
  float amax = oracle_amax(in, in_dtype, n);
  if (!(amax > 0.0f)) amax = 0.0f;
  if (amax_out) *amax_out = amax;
  oracle_cast_with_amax(in, in_dtype, amax, out, n, out_kind, scale_out);
}

/* Row-wise variant (no reference op): the arithmetic above applied to each row
 * with that row's amax; scale[r] is the double scale narrowed to fp32. */
void oracle_dynamic_scaled_quant_rowwise(const void *in, int in_dtype, uint8_t *out, int64_t rows,
                                         int64_t cols, int out_kind, float *amax_out,
                                         float *scale_out) {
  const size_t es = in_dtype == ORACLE_BF16 ? 2 : 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const char *row = (const char *)in + (size_t)r * cols * es;
    float amax = 0.0f;
    for (int64_t c = 0; c < cols; ++c) {
      float a = fabsf(load_f32(row, in_dtype, c));
      if (a > amax) amax = a;
    }
    double sd = dsq_scale(amax, out_kind);
    if (amax_out) amax_out[r] = amax;
    if (scale_out) scale_out[r] = (float)sd;
    for (int64_t c = 0; c < cols; ++c) {
      float p = (float)(sd * (double)load_f32(row, in_dtype, c));
      out[r * cols + c] = f32_to_fp8_sat(p, out_kind);
    }
  }
}

/* ---- mx_fp8_quantize: src/mx_cast.cu:44-86 (block scale) and :131-155 (payload,
 * scale byte).  Blocks are 32 consecutive elements of the flat bf16 array.
 * Per element e = ceil(log2 |x|) from the fp32 exponent field, +1 when the
 * mantissa is non-zero; zero -> -128, subnormal -> -126 (:50-65).  E = max e;
 * biased = clamp(E - 8 + 127, 0, 255); scale = fp32 with that exponent field and
 * zero mantissa (0.0 when biased == 0, +inf when 255) (:68-85).  The payload is
 * fp8_sat(x * rcp(scale), E4M3) whatever fp8 type was asked for (:146-148);
 * rcp(0) = +inf, so an all-zero or very small block yields 0*inf = NaN bytes and
 * +-448.  The scale byte is cvt.rp.satfinite.ue8m0(scale) = biased, with 255
 * clamped to 0xFE (:153). */
static inline int mx_ceil_log2(float a) {
  uint32_t b = f32_bits(a);
  int be = (int)((b >> 23) & 0xFF);
  if (be == 0) return (a == 0.0f) ? -128 : -126;
  return be - 127 + ((b & 0x7FFFFF) != 0);
}

void oracle_mx_fp8_quantize(const uint16_t *in, uint8_t *payload, uint8_t *scales, int64_t nblocks) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint16_t *x = in + b * 32;
    int E = -1000;
    for (int i = 0; i < 32; ++i) {
      int e = mx_ceil_log2(fabsf(bf16_to_f32(x[i])));
      if (e > E) E = e;
    }
    int biased = E - 8 + 127;
    if (biased < 0) biased = 0;
    if (biased > 255) biased = 255;
    float scale = bits_f32((uint32_t)biased << 23);
    /* rcp.rn of a power of two is exact, including the subnormal 2^-127 and the
     * limits rcp(0) = inf, rcp(inf) = 0. */
    float inv = (biased == 0) ? INFINITY : (biased == 255 ? 0.0f : (float)ldexp(1.0, 127 - biased));
    (void)scale;
    for (int i = 0; i < 32; ++i) {
      volatile float p = bf16_to_f32(x[i]) * inv;
      payload[b * 32 + i] = f32_to_fp8_sat(p, ORACLE_E4M3);
    }
    scales[b] = (uint8_t)(biased > 254 ? 254 : biased);
  }
}

/* ---- MX block-32 quantisation for the other element formats and input types.
 * The reference's scale rule (src/mx_cast.cu:44-86) with its constant 8 (the
 * exponent of e4m3's largest power of two, :72) replaced by the element
 * format's: 15 for e5m2, 2 for e2m1.  No reference kernel computes these (the
 * reference accepts the arguments and runs the bf16 -> e4m3 arithmetic,
 * :148,175-184,204), so no reference test pins them; the conversions are pinned
 * against the CUDA toolkit's header functions, and in_dtype bf16 / e4m3 must
 * reproduce oracle_mx_fp8_quantize. */
static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const int be = (h >> 10) & 0x1F;
  const uint32_t man = h & 0x3FFu;
  if (be == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
  if (be == 0) return (sign ? -1.0f : 1.0f) * (float)ldexp((double)man, -24);
  return bits_f32(sign | ((uint32_t)(be - 15 + 127) << 23) | (man << 13));
}

/* cvt.rn.satfinite.e2m1x2.f32 per element (what __nv_cvt_float_to_fp4 does): values
 * 0, 0.5, 1, 1.5, 2, 3, 4, 6 with a sign bit; nearest-even; above 6 (infinities too)
 * -> 6; NaN -> +6 (the format has no NaN). */
static uint8_t f32_to_e2m1_sat(float x) {
  if (isnan(x)) return 0x7;
  const uint8_t sign = signbit(x) ? 0x8 : 0;
  const double a = fabs((double)x);
  if (a > 6.0) return sign | 0x7;
  if (a == 0.0) return sign;
  int e;
  (void)frexp(a, &e);
  int fl = e - 1;
  if (fl < 0) fl = 0; /* smallest normal exponent: 2^0; below it the step is 0.5 */
  double q = ldexp(1.0, fl - 1);
  long n = (long)rint(a / q); /* in [0, 4] */
  if (n == 4) { n = 2; fl += 1; }
  uint8_t code = (n < 2) ? (uint8_t)n : (uint8_t)(((fl + 1) << 1) | (n - 2));
  return sign | code;
}
uint8_t oracle_f32_to_e2m1(float f) { return f32_to_e2m1_sat(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* in_dtype: 0 bf16, 1 fp32, 2 fp16.  fmt: 0 e4m3, 1 e5m2, 2 e2m1 (packed two per
 * byte, lower index in the low nibble). */
void oracle_mx_quantize(const void *in, int in_dtype, uint8_t *payload, uint8_t *scales, int64_t nblocks, int fmt) {
  const int emax = fmt == 0 ? 8 : (fmt == 1 ? 15 : 2);
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nblocks; ++b) {
    float x[32];
    int E = -1000;
    for (int i = 0; i < 32; ++i) {
      const int64_t j = b * 32 + i;
      x[i] = in_dtype == 0 ? bf16_to_f32(((const uint16_t *)in)[j])
           : in_dtype == 1 ? ((const float *)in)[j] : f16_to_f32(((const uint16_t *)in)[j]);
      int e = mx_ceil_log2(fabsf(x[i]));
      if (e > E) E = e;
    }
    int biased = E - emax + 127;
    if (biased < 0) biased = 0;
    if (biased > 255) biased = 255;
    const float inv = (biased == 0) ? INFINITY : (biased == 255 ? 0.0f : (float)ldexp(1.0, 127 - biased));
    for (int i = 0; i < 32; ++i) {
      volatile float p = x[i] * inv; /* one fp32 rounding (exact unless the product is subnormal) */
      if (fmt == 2) {
        const uint8_t nib = f32_to_e2m1_sat(p);
        uint8_t *dst = payload + (b * 32 + i) / 2;
        if (i & 1) *dst = (uint8_t)(*dst | (nib << 4)); else *dst = nib;
      } else {
        payload[b * 32 + i] = f32_to_fp8_sat(p, fmt);
      }
    }
    scales[b] = (uint8_t)(biased > 254 ? 254 : biased);
  }
}

/* Single-value entry points for exhaustive conversion checks. */
/* ---- MX block-scaled GEMM (the consumer of the MX casts).
 * D[m,n] = bf16( sum_k A[m,k] 2^(sa[m,k/32]-127) * B[n,k] 2^(sb[n,k/32]-127) ), the contraction the reference
 * hands to a CUTLASS block-scaled collective (src/mx_fp8_bf16.cu:42-163: e4m3 operands, ue8m0 scales of 32
 * elements, fp32 accumulation, bf16 output, alpha 1, beta 0; shapes and scale sizes :168-215).  A is [M,K]
 * row-major, B is [N,K] row-major (the reference's column-major [K,N] view), both scale arrays in the blocked
 * layout CUTLASS's Sm1xxBlockScaledConfig gives them (:100-110): 128-row x 4-block atoms of 512 bytes, atoms of
 * a 128-row band ordered along K, scale (r, c) of an atom at (r % 32) * 16 + (r / 32) * 4 + c.  The tensor core
 * accumulates in fp32 in an order this restatement does not model: the sum here is exact in double and rounded
 * once, so equality with the device is expected bit for bit only when every partial sum is exactly
 * representable in fp32 (small integers times powers of two); otherwise to within bf16 rounding of nearly equal
 * sums.  Element formats: fmt 0 = e4m3 (one byte per element), fmt 2 = e2m1 (two per byte, lower index in the
 * low nibble; K counts elements). */
static double e4m3_to_f64(uint8_t b) {
  const int sign = b >> 7, be = (b >> 3) & 0xF, man = b & 7;
  double v;
  if (be == 0xF && man == 7) return NAN;
  v = be == 0 ? ldexp((double)man, -9) : ldexp(1.0 + man / 8.0, be - 7);
  return sign ? -v : v;
}
static double e2m1_to_f64(uint8_t nib) {
  static const double mag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
  return (nib & 8) ? -mag[nib & 7] : mag[nib & 7];
}
static double e8m0_to_f64(uint8_t b) { return b == 0xFF ? NAN : ldexp(1.0, (int)b - 127); }
static inline int64_t blocked_scale_offset(int64_t r, int64_t c, int64_t katoms) {
  return ((r / 128) * katoms + c / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4;
}

void oracle_mx_gemm_bf16(const uint8_t *a, const uint8_t *b, const uint8_t *sa_blocked, const uint8_t *sb_blocked,
                         uint16_t *out, int64_t M, int64_t N, int64_t K, int fmt) {
  const int64_t kblocks = (K + 31) / 32, katoms = (kblocks + 3) / 4;
  const int64_t row_bytes = fmt == 2 ? K / 2 : K;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int64_t kb = 0; kb < kblocks; ++kb) {
        const double s = e8m0_to_f64(sa_blocked[blocked_scale_offset(m, kb, katoms)]) *
                         e8m0_to_f64(sb_blocked[blocked_scale_offset(n, kb, katoms)]);
        double part = 0.0;
        const int64_t k1 = (kb + 1) * 32 < K ? (kb + 1) * 32 : K;
        for (int64_t k = kb * 32; k < k1; ++k) {
          double x, y;
          if (fmt == 2) {
            const uint8_t xa = a[m * row_bytes + k / 2], xb = b[n * row_bytes + k / 2];
            x = e2m1_to_f64((k & 1) ? xa >> 4 : xa & 0xF);
            y = e2m1_to_f64((k & 1) ? xb >> 4 : xb & 0xF);
          } else {
            x = e4m3_to_f64(a[m * row_bytes + k]);
            y = e4m3_to_f64(b[n * row_bytes + k]);
          }
          part += x * y;
        }
        acc += part * s;
      }
      out[m * N + n] = f64_to_bf16_rne(acc);
    }
  }
}

/* ---- Row-wise scaled fp8 GEMM (the consumer of the row-wise quantisation scales).
 * out[m,n] = bf16( fp32( fp32(acc * xs[m]) * ws[n] ) + bias[n] ), acc = sum_k A[m,k] B[n,k] accumulated in fp32 on the
 * tensor cores: the epilogue tree of the reference's CUTLASS kernel, Cast(Add(Bias, Multiply(WScale, Multiply(XScale,
 * Acc)))) with fp32 compute (src/scaled_mm_kernels/f8f8bf16_rowwise_kernel.h:151-175), operands A e4m3 or e5m2, B e4m3
 * (src/sweep_mm.cu:20-21).  The sum is formed exactly in double and rounded to fp32 once: bit-exact with the device
 * when every partial sum is representable in fp32, as for the block-scaled GEMM above. */
static double e5m2_to_f64(uint8_t b) {
  const int sign = b >> 7, be = (b >> 2) & 0x1F, man = b & 3;
  double v;
  if (be == 0x1F) return man ? NAN : (sign ? -INFINITY : INFINITY);
  v = be == 0 ? ldexp((double)man, -16) : ldexp(1.0 + man / 4.0, be - 15);
  return sign ? -v : v;
}

void oracle_rowwise_gemm_bf16(const uint8_t *a, const uint8_t *b, const float *xs, const float *ws, const float *bias,
                              uint16_t *out, int64_t M, int64_t N, int64_t K, int a_kind) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k)
        acc += (a_kind == ORACLE_E5M2 ? e5m2_to_f64(a[m * K + k]) : e4m3_to_f64(a[m * K + k])) * e4m3_to_f64(b[n * K + k]);
      volatile float f = (float)acc;
      f = f * xs[m];
      f = f * ws[n];
      if (bias) f = f + bias[n];
      out[m * N + n] = f64_to_bf16_rne((double)f);
    }
  }
}

uint16_t oracle_f32_to_bf16(float f) { return f64_to_bf16_rne((double)f); }
uint16_t oracle_bf16_mul(uint16_t a, uint16_t b) {
  return f64_to_bf16_rne((double)bf16_to_f32(a) * (double)bf16_to_f32(b));
}
uint8_t oracle_f32_to_fp8(float f, int kind) { return f32_to_fp8_sat(f, kind); }

void oracle_f32_to_fp8_array(const float *in, uint8_t *out, int64_t n, int kind) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_fp8_sat(in[i], kind);
}
void oracle_bf16_mul_array(const uint16_t *a, uint16_t b, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_bf16_mul(a[i], b);
}
void oracle_f32_to_bf16_array(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_f32_to_bf16(in[i]);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
