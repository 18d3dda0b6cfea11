// Elementwise fp8 casts with the output transposed, or in both orientations from one read.
//
// The reference declares `transpose` on saturated_cast ("will transpose the input tensor during
// casting", driss_torch/__init__.py:24-38) but the Python wrapper asserts it off and the CUDA
// side only uses the flag to pick a kernel (src/saturated_cast.cu:168-181): a caller who needs the
// second orientation of an fp8 operand transposes and casts again.  Here, for a contiguous
// [rows, cols] input,
//   out_t [cols, rows] == cast(transpose(x))      (always written)
//   out   [rows, cols] == cast(x)                  (written when the pointer is given)
// where cast is dtq_saturated_cast (a device-resident scale; the reference's bf16 / fp32 product)
// or dtq_cast_with_amax (a device-resident amax; scale fp8_max / ((double)amax + 1e-12), product in
// double precision, src/dynamic_scaled_quant.cu:111-117), bit for bit.  The casts are elementwise,
// so out_t is the transpose of out: every element is converted ONCE.
//
// Fast path (rows % 16 == 0, 16-byte rows of input, aligned pointers): a CTA owns a tile of 128
// rows x 256 input bytes (128 bf16 or 64 fp32 columns).  Rows enter with 16-byte loads (a full
// 256-byte segment per row); each lane casts its chunk, stores the bytes to `out` if wanted, and
// parks them in shared memory (128 x 128 bytes; 4-word groups XOR-swizzled by the 16-row group, so
// both phases are free of bank conflicts).  Then a lane takes a word column (four byte columns) of
// 16 rows, transposes its 4 x 4 byte blocks with byte permutes, and stores 16 contiguous bytes to
// each of four rows of out_t; the eight lanes of a word column cover full 128-byte lines.
// Any other shape or alignment: a 32 x 32 byte-tile kernel, one element per thread.
#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {

// from amax.cu
int launch_amax(const void *in, float *out, int64_t numel, int in_dtype, Workspace *ws, const DeviceInfo &dev,
                cudaStream_t st);

namespace {

constexpr int kTileRows = 128;
constexpr int kTileWords = 32;  // 32-bit words of fp8 bytes per shared-memory row (fp32 input uses 16 of them)
constexpr int kThreadsT = 256;
constexpr int kRowPasses = kTileRows / 16;  // a pass of 8 warps covers 16 rows (2 per warp)

__device__ __forceinline__ void park(uint32_t *dst, uint2 b) { *reinterpret_cast<uint2 *>(dst) = b; }
__device__ __forceinline__ void park(uint32_t *dst, uint32_t b) { *dst = b; }

// ---- dtq_saturated_cast's arithmetic: a device-resident scale ----------------------------------------
template <int IN, int OUT>
struct Cast;

template <int OUT>
struct Cast<DTQ_BF16, OUT> {
  static constexpr int kChunkElems = 8;  // elements per 16-byte input chunk = fp8 bytes it produces
  using Bytes = uint2;
  using Scale = __nv_bfloat162;
  __device__ static Scale load_scale(const float *s) { return __float2bfloat162_rn(*s); }
  __device__ static float scale_value(const Scale &) { return 0.0f; }
  // two packed bf16 -> two fp8 bytes: one bf16 multiply each, then bf16 -> fp32 -> fp8
  __device__ static uint32_t pair(uint32_t w, Scale s) {
    const uint32_t p = as_u32(__hmul2(as_bf162(w), s));
    return cvt_fp8x2<OUT>(bf16_lo(p), bf16_hi(p));
  }
  __device__ static Bytes convert(uint4 v, const Scale &s) {
    return make_uint2(pair(v.x, s) | (pair(v.y, s) << 16), pair(v.z, s) | (pair(v.w, s) << 16));
  }
  __device__ static uint8_t one(const void *in, int64_t i, const Scale &s) {
    return cvt_fp8<OUT>(__bfloat162float(__hmul(static_cast<const __nv_bfloat16 *>(in)[i], s.x)));
  }
};

template <int OUT>
struct Cast<DTQ_F32, OUT> {
  static constexpr int kChunkElems = 4;
  using Bytes = uint32_t;
  using Scale = float;
  __device__ static Scale load_scale(const float *s) { return *s; }
  __device__ static float scale_value(const Scale &) { return 0.0f; }
  __device__ static Bytes convert(uint4 v, const Scale &s) {
    return cvt_fp8x4<OUT>(__fmul_rn(__uint_as_float(v.x), s), __fmul_rn(__uint_as_float(v.y), s),
                          __fmul_rn(__uint_as_float(v.z), s), __fmul_rn(__uint_as_float(v.w), s));
  }
  __device__ static uint8_t one(const void *in, int64_t i, const Scale &s) {
    return cvt_fp8<OUT>(__fmul_rn(static_cast<const float *>(in)[i], s));
  }
};

// ---- dtq_cast_with_amax's arithmetic: a device-resident amax instead of a scale ----------------------
template <int IN, int OUT>
struct DynCast;

template <int OUT>
struct DynCast<DTQ_BF16, OUT> {
  static constexpr int kChunkElems = 8;
  using Bytes = uint2;
  using Scale = DsqScale;
  __device__ static Scale load_scale(const float *amax) { return make_dsq_scale<OUT>(fmaxf(*amax, 0.0f)); }
  __device__ static float scale_value(const Scale &s) { return static_cast<float>(s.sd); }
  __device__ static Bytes convert(uint4 v, const Scale &s) { return dsq_convert_bf16x8<OUT, false>(v, s); }
  __device__ static uint8_t one(const void *in, int64_t i, const Scale &s) {
    return cvt_fp8<OUT>(dsq_mul(s.sd, __uint_as_float(uint32_t(static_cast<const uint16_t *>(in)[i]) << 16)));
  }
};

template <int OUT>
struct DynCast<DTQ_F32, OUT> {
  static constexpr int kChunkElems = 4;
  using Bytes = uint32_t;
  using Scale = DsqScale;
  __device__ static Scale load_scale(const float *amax) { return make_dsq_scale<OUT>(fmaxf(*amax, 0.0f)); }
  __device__ static float scale_value(const Scale &s) { return static_cast<float>(s.sd); }
  __device__ static Bytes convert(uint4 v, const Scale &s) { return dsq_convert_f32x4<OUT>(v, s); }
  __device__ static uint8_t one(const void *in, int64_t i, const Scale &s) {
    return cvt_fp8<OUT>(dsq_mul(s.sd, static_cast<const float *>(in)[i]));
  }
};

// FULL: the tile lies inside the matrix, no access is predicated.  BOTH: also write the row-major output.
template <typename C, bool BOTH, bool FULL>
__device__ __forceinline__ void transposed_tile(uint32_t (&tile)[kTileRows][kTileWords], const uint4 *__restrict__ in,
                                                uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                                                const typename C::Scale &s, int64_t rows, int64_t cols,
                                                int64_t row0, int64_t col0) {
  constexpr int kE = C::kChunkElems;      // columns per chunk
  constexpr int kChunkWords = kE / 4;     // words of fp8 bytes per chunk
  constexpr int kRowWords = 16 * kChunkWords;  // words of fp8 bytes per tile row: 32 (bf16) or 16 (fp32)
  // fp32 input fills only half of a shared-memory row: odd rows use the other half, so that the two rows a
  // warp parks at once fall on different banks
  constexpr int kSkew = kRowWords == 16 ? 16 : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row_chunks = cols / kE;

  // ---- rows: in pass p warp w owns tile rows 16p + 2w and + 1; lane l the 16-byte input chunk l & 15 of the row
  const int chunk = lane & 15;
  const int64_t c = col0 + chunk * kE;  // first column of the chunk; cols is a multiple of a chunk
  const bool col_live = FULL || c < cols;
  uint4 v[kRowPasses];
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int64_t r = row0 + p * 16 + warp * 2 + (lane >> 4);
    v[p] = (FULL || (col_live && r < rows)) ? ldg_stream(in + r * row_chunks + c / kE) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int rt = p * 16 + warp * 2 + (lane >> 4);  // rt >> 4 == p: the 16-row group of this row
    const typename C::Bytes b = C::convert(v[p], s);
    park(&tile[rt][(chunk * kChunkWords) ^ (p << 2) ^ ((rt & 1) * kSkew)], b);
    if (BOTH && (FULL || (col_live && row0 + rt < rows))) stg_stream(out + (row0 + rt) * cols + c, b);
  }
  __syncthreads();

  // ---- columns: lane = 8 * q + g: 16-row group g of the tile, word column 4 * warp + q (four byte columns)
  const int g = lane & 7, q = lane >> 3;
  const int word = warp * 4 + q;
  if (word >= kRowWords) return;  // fp32 input: half as many byte columns per tile
  const int64_t r_first = row0 + g * 16;
  const int64_t col = col0 + word * 4;
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = tile[g * 16 + i][word ^ (g << 2) ^ ((i & 1) * kSkew)];
  // 4 x 4 byte transposes: rows 4k .. 4k+3 of byte column j -> word k of column j's sixteen bytes
  uint32_t t[4][4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t a0 = __byte_perm(w[4 * k], w[4 * k + 1], 0x5140), a1 = __byte_perm(w[4 * k], w[4 * k + 1], 0x7362);
    const uint32_t b0 = __byte_perm(w[4 * k + 2], w[4 * k + 3], 0x5140), b1 = __byte_perm(w[4 * k + 2], w[4 * k + 3], 0x7362);
    t[0][k] = __byte_perm(a0, b0, 0x5410);
    t[1][k] = __byte_perm(a0, b0, 0x7632);
    t[2][k] = __byte_perm(a1, b1, 0x5410);
    t[3][k] = __byte_perm(a1, b1, 0x7632);
  }
  // rows % 16 == 0: a 16-row group is inside or outside as a whole; cols % 4 == 0 likewise for a word column
  if (FULL || (r_first < rows && col < cols)) {
    uint8_t *dst = out_t + col * rows + r_first;
#pragma unroll
    for (int j = 0; j < 4; ++j) stg_stream(dst + j * rows, make_uint4(t[j][0], t[j][1], t[j][2], t[j][3]));
  }
}

// `scale` points to the scale (Cast) or to the amax (DynCast); scale_out, if given, receives the fp32 scale
// a DynCast derived from the amax, amax_out the amax it used (the given one, clamped at zero).
constexpr int kTransposedMinBlocks = 4;
template <typename C, bool BOTH>
__global__ void __launch_bounds__(kThreadsT, kTransposedMinBlocks)
cast_transposed_kernel(const uint4 *__restrict__ in, uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                       const float *__restrict__ scale, float *__restrict__ scale_out, float *__restrict__ amax_out,
                       int64_t rows, int64_t cols, int64_t col_tiles) {
  __shared__ __align__(16) uint32_t tile[kTileRows][kTileWords];
  constexpr int kTileCols = 16 * C::kChunkElems;
  pdl_launch_dependents();
  pdl_wait();  // may have become resident under the tail of the kernel that delivers *scale
  const typename C::Scale s = C::load_scale(scale);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (scale_out) *scale_out = C::scale_value(s);
    if (amax_out) *amax_out = fmaxf(*scale, 0.0f);
  }
  // highest rows first: behind an amax (or any other pass over the input) the end of the tensor may still be in L2
  const int64_t t = int64_t(gridDim.x) - 1 - blockIdx.x;
  const int64_t row0 = (t / col_tiles) * kTileRows;
  const int64_t col0 = (t % col_tiles) * kTileCols;
  if (row0 + kTileRows <= rows && col0 + kTileCols <= cols)
    transposed_tile<C, BOTH, true>(tile, in, out, out_t, s, rows, cols, row0, col0);
  else
    transposed_tile<C, BOTH, false>(tile, in, out, out_t, s, rows, cols, row0, col0);
}

// Any shape and alignment: 32 x 32 tiles of fp8 bytes, block (32, 8), one element per thread per step.
template <typename C, bool BOTH>
__global__ void __launch_bounds__(256)
cast_transposed_generic(const void *__restrict__ in, uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                        const float *__restrict__ scale, float *__restrict__ scale_out, float *__restrict__ amax_out,
                        int64_t rows, int64_t cols, int64_t col_tiles) {
  __shared__ uint8_t tile[32][33];
  pdl_launch_dependents();
  pdl_wait();
  const typename C::Scale s = C::load_scale(scale);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (scale_out) *scale_out = C::scale_value(s);
    if (amax_out) *amax_out = fmaxf(*scale, 0.0f);
  }
  const int64_t row0 = (blockIdx.x / col_tiles) * 32, col0 = (blockIdx.x % col_tiles) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r = row0 + ty + 8 * j, c = col0 + tx;
    if (r < rows && c < cols) {
      const uint8_t b = C::one(in, r * cols + c, s);
      tile[ty + 8 * j][tx] = b;
      if (BOTH) out[r * cols + c] = b;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t c = col0 + ty + 8 * j, r = row0 + tx;
    if (r < rows && c < cols) out_t[c * rows + r] = tile[tx][ty + 8 * j];
  }
}

template <typename C, bool BOTH>
int launch_transposed(const void *in, void *out, void *out_t, const float *scale, float *scale_out, float *amax_out,
                      int64_t rows, int64_t cols, cudaStream_t st) {
  constexpr int kTileCols = 16 * C::kChunkElems;
  const bool fast = rows % 16 == 0 && cols % C::kChunkElems == 0 && aligned_to(in, 16) && aligned_to(out_t, 16) &&
                    (!BOTH || aligned_to(out, 8));
  if (fast) {
    const int64_t row_tiles = ceil_div64(rows, kTileRows), col_tiles = ceil_div64(cols, kTileCols);
    if (row_tiles > 0x7FFFFFFFLL / col_tiles) return DTQ_ERR_TOO_LARGE;
    return cuda_status(launch_after_dependency(cast_transposed_kernel<C, BOTH>, dim3(static_cast<unsigned>(row_tiles * col_tiles)),
                                               dim3(kThreadsT), 0, st, static_cast<const uint4 *>(in),
                                               static_cast<uint8_t *>(out), static_cast<uint8_t *>(out_t), scale, scale_out,
                                               amax_out, rows, cols, col_tiles));
  } else {
    const int64_t row_tiles = ceil_div64(rows, 32), col_tiles = ceil_div64(cols, 32);
    if (row_tiles > 0x7FFFFFFFLL / col_tiles) return DTQ_ERR_TOO_LARGE;
    return cuda_status(launch_after_dependency(cast_transposed_generic<C, BOTH>, dim3(static_cast<unsigned>(row_tiles * col_tiles)),
                                               dim3(256), 0, st, in, static_cast<uint8_t *>(out),
                                               static_cast<uint8_t *>(out_t), scale, scale_out, amax_out, rows, cols,
                                               col_tiles));
  }
}

template <typename C>
int launch_by_outputs(const void *in, void *out, void *out_t, const float *scale, float *scale_out, float *amax_out,
                      int64_t rows, int64_t cols, cudaStream_t st) {
  return out ? launch_transposed<C, true>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st)
             : launch_transposed<C, false>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st);
}

// CAST<IN, OUT> = Cast (static scale) or DynCast (amax)
template <template <int, int> class CAST>
int launch_by_dtypes(const void *in, void *out, void *out_t, const float *scale, float *scale_out, float *amax_out,
                     int64_t rows, int64_t cols, int in_dtype, int out_dtype, cudaStream_t st) {
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3 ? launch_by_outputs<CAST<DTQ_BF16, DTQ_E4M3>>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st)
                                 : launch_by_outputs<CAST<DTQ_BF16, DTQ_E5M2>>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st);
  return out_dtype == DTQ_E4M3 ? launch_by_outputs<CAST<DTQ_F32, DTQ_E4M3>>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st)
                               : launch_by_outputs<CAST<DTQ_F32, DTQ_E5M2>>(in, out, out_t, scale, scale_out, amax_out, rows, cols, st);
}

}  // namespace
}  // namespace dtq

namespace dtq {
namespace {
int check_transposed_args(const void *in, const void *out_t, const float *scale, int64_t rows, int64_t cols, int in_dtype,
                          int out_dtype, bool *nothing_to_do) {
  *nothing_to_do = false;
  if (rows < 0 || cols < 0 || !scale) return DTQ_ERR_INVALID_ARGUMENT;
  if ((in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) || (out_dtype != DTQ_E4M3 && out_dtype != DTQ_E5M2))
    return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (rows == 0 || cols == 0) {
    *nothing_to_do = true;
    return DTQ_OK;
  }
  if (!in || !out_t) return DTQ_ERR_INVALID_ARGUMENT;
  return DTQ_OK;
}
}  // namespace
}  // namespace dtq

extern "C" int dtq_saturated_cast_transposed(const void *in, void *out, void *out_t, const float *scale, int64_t rows,
                                             int64_t cols, int in_dtype, int out_dtype, void *stream) {
  using namespace dtq;
  bool nothing = false;
  if (int e = check_transposed_args(in, out_t, scale, rows, cols, in_dtype, out_dtype, &nothing)) return e;
  if (nothing) return DTQ_OK;
  return launch_by_dtypes<Cast>(in, out, out_t, scale, nullptr, nullptr, rows, cols, in_dtype, out_dtype,
                                static_cast<cudaStream_t>(stream));
}

extern "C" int dtq_cast_with_amax_transposed(const void *in, void *out, void *out_t, const float *amax, float *scale_out,
                                             int64_t rows, int64_t cols, int in_dtype, int out_dtype, void *stream) {
  using namespace dtq;
  bool nothing = false;
  if (int e = check_transposed_args(in, out_t, amax, rows, cols, in_dtype, out_dtype, &nothing)) return e;
  if (nothing) return DTQ_OK;  // like dtq_cast_with_amax on an empty input, scale_out is left alone
  return launch_by_dtypes<DynCast>(in, out, out_t, amax, scale_out, nullptr, rows, cols, in_dtype, out_dtype,
                                   static_cast<cudaStream_t>(stream));
}

extern "C" int dtq_dynamic_scaled_quant_dual(const void *in, void *out, void *out_t, float *amax_out, float *scale_out,
                                             int64_t rows, int64_t cols, int in_dtype, int out_dtype, void *workspace,
                                             size_t workspace_bytes, void *stream) {
  using namespace dtq;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  Workspace *ws = static_cast<Workspace *>(workspace);
  bool nothing = false;
  if (int e = check_transposed_args(in, out_t, &ws->amax, rows, cols, in_dtype, out_dtype, &nothing)) return e;
  if (nothing || !out) return nothing ? DTQ_OK : DTQ_ERR_INVALID_ARGUMENT;
  if (!aligned_to(in, in_dtype == DTQ_BF16 ? 2 : 4)) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the amax lands in the workspace; the cast is queued behind it so that it may become resident under its tail
  if (int e = launch_amax(in, &ws->amax, rows * cols, in_dtype, ws, dev, st)) return e;
  return launch_by_dtypes<DynCast>(in, out, out_t, &ws->amax, scale_out, amax_out, rows, cols, in_dtype, out_dtype, st);
}
