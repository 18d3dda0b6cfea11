// saturated_cast with the output transposed, or in both orientations from one read.
//
// The reference declares `transpose` on saturated_cast ("will transpose the input tensor during
// casting", driss_torch/__init__.py:24-38) but the Python wrapper asserts it off and the CUDA
// side only uses the flag to pick a kernel (src/saturated_cast.cu:168-181): a caller who needs the
// second orientation of an fp8 operand transposes and casts again.  Here, for a contiguous
// [rows, cols] input,
//   out_t [cols, rows] == saturated_cast(transpose(x))      (always written)
//   out   [rows, cols] == saturated_cast(x)                  (written when the pointer is given)
// with the arithmetic of dtq_saturated_cast, bit for bit (the op is elementwise, so out_t is the
// transpose of out).
//
// Fast path (rows % 16 == 0, 16-byte rows of input, aligned pointers): a CTA owns a tile of 128
// rows x 256 input bytes (128 bf16 or 64 fp32 columns).  Rows enter with 16-byte loads (a full
// 256-byte segment per row), are cast and stored from registers if `out` is wanted, and are
// parked unconverted in shared memory (32 KiB, 4-word groups XOR-swizzled by the 16-row group, so
// both phases are free of bank conflicts).  Then a lane walks 16 rows down one 32-bit word column
// (two bf16 columns or one fp32 column), casts, and stores 16 contiguous bytes of a row of out_t;
// the eight lanes of a word column cover a full 128-byte line.
// Any other shape or alignment: a 32 x 32 byte-tile kernel, one element per thread.
#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {
namespace {

constexpr int kTileRows = 128;
constexpr int kTileWords = 64;  // 32-bit words per tile row: 256 bytes
constexpr int kThreadsT = 256;
constexpr int kRowPasses = kTileRows / 16;  // a pass of 8 warps covers 16 rows (2 per warp)

template <int IN, int OUT>
struct Cast;

template <int OUT>
struct Cast<DTQ_BF16, OUT> {
  static constexpr int kColsPerWord = 2;
  using Scale = __nv_bfloat162;
  __device__ static Scale load_scale(const float *s) { return __float2bfloat162_rn(*s); }
  // two packed bf16 -> two fp8 bytes: one bf16 multiply each, then bf16 -> fp32 -> fp8
  __device__ static uint32_t pair(uint32_t w, Scale s) {
    const uint32_t p = as_u32(__hmul2(as_bf162(w), s));
    return cvt_fp8x2<OUT>(bf16_lo(p), bf16_hi(p));
  }
  // a 16-byte chunk of a row -> 8 fp8 bytes
  __device__ static void row_chunk(uint4 v, Scale s, uint8_t *dst) {
    stg_stream(dst, make_uint2(pair(v.x, s) | (pair(v.y, s) << 16), pair(v.z, s) | (pair(v.w, s) << 16)));
  }
  // sixteen rows of one word column -> 16 fp8 bytes for each of its two columns
  __device__ static void column(const uint32_t (&w)[16], Scale s, uint8_t *dst, int64_t next_col) {
    uint32_t a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = pair(__byte_perm(w[2 * i], w[2 * i + 1], 0x5410), s);
      b[i] = pair(__byte_perm(w[2 * i], w[2 * i + 1], 0x7632), s);
    }
    stg_stream(dst, make_uint4(a[0] | (a[1] << 16), a[2] | (a[3] << 16), a[4] | (a[5] << 16), a[6] | (a[7] << 16)));
    stg_stream(dst + next_col,
               make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16)));
  }
  __device__ static uint8_t one(const void *in, int64_t i, Scale s) {
    return cvt_fp8<OUT>(__bfloat162float(__hmul(static_cast<const __nv_bfloat16 *>(in)[i], s.x)));
  }
};

template <int OUT>
struct Cast<DTQ_F32, OUT> {
  static constexpr int kColsPerWord = 1;
  using Scale = float;
  __device__ static Scale load_scale(const float *s) { return *s; }
  __device__ static uint32_t quad(uint32_t a, uint32_t b, uint32_t c, uint32_t d, Scale s) {
    return cvt_fp8x4<OUT>(__fmul_rn(__uint_as_float(a), s), __fmul_rn(__uint_as_float(b), s),
                          __fmul_rn(__uint_as_float(c), s), __fmul_rn(__uint_as_float(d), s));
  }
  __device__ static void row_chunk(uint4 v, Scale s, uint8_t *dst) { stg_stream(dst, quad(v.x, v.y, v.z, v.w, s)); }
  __device__ static void column(const uint32_t (&w)[16], Scale s, uint8_t *dst, int64_t) {
    stg_stream(dst, make_uint4(quad(w[0], w[1], w[2], w[3], s), quad(w[4], w[5], w[6], w[7], s),
                               quad(w[8], w[9], w[10], w[11], s), quad(w[12], w[13], w[14], w[15], s)));
  }
  __device__ static uint8_t one(const void *in, int64_t i, Scale s) {
    return cvt_fp8<OUT>(__fmul_rn(static_cast<const float *>(in)[i], s));
  }
};

// FULL: the tile lies inside the matrix, no access is predicated.  BOTH: also write the row-major output.
template <int IN, int OUT, bool BOTH, bool FULL>
__device__ __forceinline__ void transposed_tile(uint32_t (&tile)[kTileRows][kTileWords], const uint32_t *__restrict__ in,
                                                uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                                                typename Cast<IN, OUT>::Scale s, int64_t rows, int64_t cols,
                                                int64_t row0, int64_t col0) {
  using C = Cast<IN, OUT>;
  constexpr int kCW = C::kColsPerWord;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row_words = cols / kCW;

  // ---- rows: in pass p warp w owns tile rows 16p + 2w and + 1; lane l the 16-byte chunk l & 15 of the row
  const int chunk = lane & 15;
  const int64_t c = col0 + chunk * 4 * kCW;  // first column of the chunk; cols is a multiple of a chunk
  const bool col_live = FULL || c < cols;
  uint4 v[kRowPasses];
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int64_t r = row0 + p * 16 + warp * 2 + (lane >> 4);
    v[p] = (FULL || (col_live && r < rows)) ? ldg_stream(in + r * row_words + c / kCW) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int rt = p * 16 + warp * 2 + (lane >> 4);  // rt >> 4 == p: the 16-row group of this row
    *reinterpret_cast<uint4 *>(&tile[rt][(chunk * 4) ^ (p << 2)]) = v[p];
    if (BOTH && (FULL || (col_live && row0 + rt < rows))) C::row_chunk(v[p], s, out + (row0 + rt) * cols + c);
  }
  __syncthreads();

  // ---- columns: lane = 8 * q + g: 16-row group g of the tile, word column 4 * warp + q (+ 32 in the second pass)
  const int g = lane & 7, q = lane >> 3;
  const int64_t r_first = row0 + g * 16;
  const bool rows_live = FULL || r_first < rows;  // rows % 16 == 0: a group is inside or outside as a whole
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int word = pass * 32 + warp * 4 + q;
    const int64_t col = col0 + word * kCW;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = tile[g * 16 + i][word ^ (g << 2)];
    if (FULL || (rows_live && col < cols)) C::column(w, s, out_t + col * rows + r_first, rows);
  }
}

template <int IN, int OUT, bool BOTH>
__global__ void __launch_bounds__(kThreadsT, 4)
saturated_cast_transposed_kernel(const uint32_t *__restrict__ in, uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                                 const float *__restrict__ scale, int64_t rows, int64_t cols, int64_t col_tiles) {
  __shared__ __align__(16) uint32_t tile[kTileRows][kTileWords];
  using C = Cast<IN, OUT>;
  constexpr int kTileCols = kTileWords * C::kColsPerWord;
  const typename C::Scale s = C::load_scale(scale);
  const int64_t row0 = (blockIdx.x / col_tiles) * kTileRows;
  const int64_t col0 = (blockIdx.x % col_tiles) * kTileCols;
  if (row0 + kTileRows <= rows && col0 + kTileCols <= cols)
    transposed_tile<IN, OUT, BOTH, true>(tile, in, out, out_t, s, rows, cols, row0, col0);
  else
    transposed_tile<IN, OUT, BOTH, false>(tile, in, out, out_t, s, rows, cols, row0, col0);
}

// Any shape and alignment: 32 x 32 tiles of fp8 bytes, block (32, 8), one element per thread per step.
template <int IN, int OUT, bool BOTH>
__global__ void __launch_bounds__(256)
saturated_cast_transposed_generic(const void *__restrict__ in, uint8_t *__restrict__ out, uint8_t *__restrict__ out_t,
                                  const float *__restrict__ scale, int64_t rows, int64_t cols, int64_t col_tiles) {
  __shared__ uint8_t tile[32][33];
  using C = Cast<IN, OUT>;
  const typename C::Scale s = C::load_scale(scale);
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

template <int IN, int OUT, bool BOTH>
int launch_transposed(const void *in, void *out, void *out_t, const float *scale, int64_t rows, int64_t cols,
                      cudaStream_t st) {
  using C = Cast<IN, OUT>;
  constexpr int kTileCols = kTileWords * C::kColsPerWord;
  const bool fast = rows % 16 == 0 && cols % (4 * C::kColsPerWord) == 0 && aligned_to(in, 16) && aligned_to(out_t, 16) &&
                    (!BOTH || aligned_to(out, 8));
  if (fast) {
    const int64_t row_tiles = ceil_div64(rows, kTileRows), col_tiles = ceil_div64(cols, kTileCols);
    if (row_tiles > 0x7FFFFFFFLL / col_tiles) return DTQ_ERR_TOO_LARGE;
    saturated_cast_transposed_kernel<IN, OUT, BOTH><<<static_cast<unsigned>(row_tiles * col_tiles), kThreadsT, 0, st>>>(
        static_cast<const uint32_t *>(in), static_cast<uint8_t *>(out), static_cast<uint8_t *>(out_t), scale, rows, cols,
        col_tiles);
  } else {
    const int64_t row_tiles = ceil_div64(rows, 32), col_tiles = ceil_div64(cols, 32);
    if (row_tiles > 0x7FFFFFFFLL / col_tiles) return DTQ_ERR_TOO_LARGE;
    saturated_cast_transposed_generic<IN, OUT, BOTH><<<static_cast<unsigned>(row_tiles * col_tiles), 256, 0, st>>>(
        in, static_cast<uint8_t *>(out), static_cast<uint8_t *>(out_t), scale, rows, cols, col_tiles);
  }
  return cuda_status(cudaGetLastError());
}

template <int IN, int OUT>
int launch_by_outputs(const void *in, void *out, void *out_t, const float *scale, int64_t rows, int64_t cols,
                      cudaStream_t st) {
  return out ? launch_transposed<IN, OUT, true>(in, out, out_t, scale, rows, cols, st)
             : launch_transposed<IN, OUT, false>(in, out, out_t, scale, rows, cols, st);
}

}  // namespace
}  // namespace dtq

extern "C" int dtq_saturated_cast_transposed(const void *in, void *out, void *out_t, const float *scale, int64_t rows,
                                             int64_t cols, int in_dtype, int out_dtype, void *stream) {
  using namespace dtq;
  if (rows < 0 || cols < 0 || !scale) return DTQ_ERR_INVALID_ARGUMENT;
  if ((in_dtype != DTQ_BF16 && in_dtype != DTQ_F32) || (out_dtype != DTQ_E4M3 && out_dtype != DTQ_E5M2))
    return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (rows == 0 || cols == 0) return DTQ_OK;
  if (!in || !out_t) return DTQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == DTQ_BF16)
    return out_dtype == DTQ_E4M3 ? launch_by_outputs<DTQ_BF16, DTQ_E4M3>(in, out, out_t, scale, rows, cols, st)
                                 : launch_by_outputs<DTQ_BF16, DTQ_E5M2>(in, out, out_t, scale, rows, cols, st);
  return out_dtype == DTQ_E4M3 ? launch_by_outputs<DTQ_F32, DTQ_E4M3>(in, out, out_t, scale, rows, cols, st)
                               : launch_by_outputs<DTQ_F32, DTQ_E5M2>(in, out, out_t, scale, rows, cols, st);
}
