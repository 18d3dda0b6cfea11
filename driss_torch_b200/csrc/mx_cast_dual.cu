// mx_fp8_quantize in both orientations from ONE read of the input.
//
// Training with MX operands needs a matrix quantised along its last dimension for one GEMM and
// its transpose quantised along ITS last dimension (blocks down the columns of the original) for
// the other.  The reference declares `axis` / `transpose` on mx_fp8_quantize but ignores them
// (src/mx_cast.cu:168-171), so a caller has to transpose and cast a second time: two more
// passes over the data.  This kernel produces, from a contiguous bf16 [M, N] input,
//   payload   [M, N], scales   [M * N/32]   == mx_fp8_quantize(x)                  and
//   payload_t [N, M], scales_t [N * M/32]   == mx_fp8_quantize(x.t().contiguous())
// byte for byte, reading x once: 2 + 2 * (1 + 1/32) bytes per element instead of 2 * (3 + 1/32)
// plus the transpose.
//
// A CTA owns a 128 x 128 tile, so every global access is at least a full 128-byte line in both
// orientations.  Row direction: as in the stream kernel -- each lane loads 16 bytes, four lanes
// share an MX block, results go out from registers; the chunk is also parked in shared memory
// (32 KiB, 4-word groups XOR-swizzled by the 16-row group so that both phases are free of bank
// conflicts).  Column direction: a lane owns two neighbouring columns x 16 rows (sixteen 32-bit
// shared loads), lanes l and l^1 together hold one MX block of each column; the eight lanes of a
// column pair write 128 contiguous bytes of a row of the transposed payload.
// CTAs are numbered so that eight row tiles of one column tile run back to back, then the next
// column tile: the 4-byte scale fragments that neighbouring tiles add to one 32-byte sector of
// either scale array arrive close together in time.
#include "dtq_host.h"
#include "mx_common.cuh"

namespace dtq {
namespace {

constexpr int kTile = 128;          // rows and columns of a CTA tile
constexpr int kTileWords = kTile / 2;  // 32-bit words (bf16 pairs) per tile row
constexpr int kThreadsDual = 256;
constexpr int kWarpsDual = kThreadsDual / 32;
constexpr int kPassRows = 2 * kWarpsDual;        // a row pass: every warp takes two rows
constexpr int kRowPasses = kTile / kPassRows;    // 8 (256 threads) or 4 (512)
constexpr int kColPasses = kTileWords / (4 * kWarpsDual);  // a column pass: every warp takes four word columns
static_assert(kRowPasses % 4 == 0 && kColPasses >= 1, "256 or 512 threads");
constexpr int kGroupRowTiles = 8;

// One tile.  FULL: the tile lies inside the matrix, no access is predicated.  ROW_OUT: the row-major payload
// and scales are wanted too (otherwise the row direction only loads the tile and parks it).
template <bool FULL, bool BLOCKED, bool ROW_OUT>
__device__ __forceinline__ void dual_tile(uint32_t (&tile)[kTile][kTileWords], const uint16_t *__restrict__ in,
                                          uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
                                          uint8_t *__restrict__ payload_t, uint8_t *__restrict__ scales_t, int64_t rows,
                                          int64_t cols, int64_t row0, int64_t col0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t kblocks = cols / 32, katoms = (kblocks + 3) / 4;          // scale grid of x: [rows, kblocks]
  const int64_t row_blocks = rows / 32, row_atoms = (row_blocks + 3) / 4;  // scale grid of x^T: [cols, row_blocks]

  // ---- row direction: in pass p warp w owns tile rows 16p + 2w and + 1; lane l the columns 8(l&15) .. +7
  const int chunk = lane & 15;
  const int64_t c = col0 + chunk * 8;
  const bool col_live = FULL || c < cols;  // cols % 32 == 0, so a quad of lanes is live or dead as a whole
  uint4 v[kRowPasses];
  int my_scale = 0;
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int64_t r = row0 + p * kPassRows + warp * 2 + (lane >> 4);
    v[p] = (FULL || (col_live && r < rows)) ? ldg_stream(in + r * cols + c) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int p = 0; p < kRowPasses; ++p) {
    const int rt = p * kPassRows + warp * 2 + (lane >> 4);
    const int64_t r = row0 + rt;
    *reinterpret_cast<uint4 *>(&tile[rt][(chunk * 4) ^ ((rt >> 4) << 2)]) = v[p];  // swizzled by the 16-row group
    if constexpr (!ROW_OUT) continue;
    uint32_t mag = chunk_absmax_bits(v[p]);
    mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 1));
    mag = max(mag, __shfl_xor_sync(0xFFFFFFFFu, mag, 2));
    const int biased = block_biased_exponent(mag);
    if (FULL || (col_live && r < rows)) stg_stream(payload + r * cols + c, mx_payload(v[p], inverse_scale(biased)));
    // All four lanes of a quad hold the block's scale; lane 4k + j keeps the one of pass 4h + j, so that
    // every lane has one byte to store after four passes instead of a quarter of the lanes after each.
    if ((lane & 3) == (p & 3)) my_scale = biased;
    if ((p & 3) == 3) {
      const int64_t sr = row0 + (p - 3 + (lane & 3)) * kPassRows + warp * 2 + (lane >> 4);
      if (FULL || (col_live && sr < rows)) scales[scale_offset<BLOCKED>(sr * kblocks + (c >> 5), kblocks, katoms)] = mx_scale_byte(my_scale);
    }
  }
  __syncthreads();

  // ---- column direction: lane = 8 * q + g: 16-row group g of the tile, column pair 4 * warp + q (+ 32 per pass)
  const int g = lane & 7, q = lane >> 3;
  const int64_t r_first = row0 + g * 16;
  const bool rows_live = FULL || r_first < rows;  // rows % 32 == 0: lanes g and g^1 are live or dead together
#pragma unroll
  for (int pass = 0; pass < kColPasses; ++pass) {
    const int word = pass * (4 * kWarpsDual) + warp * 4 + q;
    const int64_t col_a = col0 + word * 2;  // and col_a + 1; cols is even, so both or neither exist
    uint32_t w[16];
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      w[i] = tile[g * 16 + i][word ^ (g << 2)];
      m = packed_absmax_signed(m, w[i]);
    }
    m &= 0x7FFF7FFFu;
    m = packed_mag_max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    const int biased_a = block_biased_exponent(m & 0xFFFFu), biased_b = block_biased_exponent(m >> 16);
    const float inv_a = inverse_scale(biased_a), inv_b = inverse_scale(biased_b);
    uint32_t a[8], b[8];  // two consecutive rows of one column per word, as e4m3 byte pairs
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = mx_pair_f32(bf16_lo(w[2 * i]), bf16_lo(w[2 * i + 1]), inv_a);
      b[i] = mx_pair_f32(bf16_hi(w[2 * i]), bf16_hi(w[2 * i + 1]), inv_b);
    }
    if (FULL || (rows_live && col_a < cols)) {
      uint8_t *dst = payload_t + col_a * rows + r_first;  // 16 consecutive bytes of row col_a of the transpose
      stg_stream(dst, make_uint4(a[0] | (a[1] << 16), a[2] | (a[3] << 16), a[4] | (a[5] << 16), a[6] | (a[7] << 16)));
      stg_stream(dst + rows, make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16)));
      if ((g & 1) == 0) {
        const int64_t blk = col_a * row_blocks + (r_first >> 5);
        scales_t[scale_offset<BLOCKED>(blk, row_blocks, row_atoms)] = mx_scale_byte(biased_a);
        scales_t[scale_offset<BLOCKED>(blk + row_blocks, row_blocks, row_atoms)] = mx_scale_byte(biased_b);
      }
    }
  }
}

// 5 CTAs of 256 threads per SM (48 registers) measured 4 % faster than 4 (64 registers); 6 (40 registers) 12 % slower
constexpr int kDualMinBlocks = kThreadsDual == 256 ? 5 : 2;
template <bool BLOCKED, bool ROW_OUT>
__global__ void __launch_bounds__(kThreadsDual, BLOCKED ? kDualMinBlocks - 1 : kDualMinBlocks)  // the blocked offsets need the registers
mx_dual_kernel(const uint16_t *__restrict__ in, uint8_t *__restrict__ payload, uint8_t *__restrict__ scales,
               uint8_t *__restrict__ payload_t, uint8_t *__restrict__ scales_t, int64_t rows, int64_t cols,
               int64_t row_tiles, int64_t col_tiles) {
  __shared__ __align__(16) uint32_t tile[kTile][kTileWords];
  // programmatic dependent launch, both ways (see dtq_device.cuh): blocks may become resident under the tail of the
  // kernel before this one, and what is queued behind this one under its own tail
  pdl_launch_dependents();
  pdl_wait();
  // grouped numbering: groups of kGroupRowTiles row tiles; inside a group row tiles vary fastest
  const int64_t pid = blockIdx.x;
  const int64_t per_group = kGroupRowTiles * col_tiles;
  const int64_t first_row_tile = (pid / per_group) * kGroupRowTiles;
  const int64_t group_rows = min(row_tiles - first_row_tile, int64_t(kGroupRowTiles));
  const int64_t in_group = pid % per_group;
  const int64_t row0 = (first_row_tile + in_group % group_rows) * kTile;
  const int64_t col0 = (in_group / group_rows) * kTile;
  if (row0 + kTile <= rows && col0 + kTile <= cols)
    dual_tile<true, BLOCKED, ROW_OUT>(tile, in, payload, scales, payload_t, scales_t, rows, cols, row0, col0);
  else
    dual_tile<false, BLOCKED, ROW_OUT>(tile, in, payload, scales, payload_t, scales_t, rows, cols, row0, col0);
}

}  // namespace
}  // namespace dtq

namespace dtq {
namespace {
template <bool BLOCKED>
int launch_dual(const void *in_bf16, void *payload, void *scales_e8m0, void *payload_t, void *scales_t_e8m0, int64_t rows,
                int64_t cols, void *stream) {
  if (rows < 0 || cols < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (cols % 32 != 0 || rows % 32 != 0) return DTQ_ERR_SHAPE;
  if (rows == 0 || cols == 0) return DTQ_OK;
  // payload == NULL (then scales_e8m0 is ignored): only the transposed outputs are wanted
  const bool row_out = payload != nullptr;
  if (!in_bf16 || (row_out && !scales_e8m0) || !payload_t || !scales_t_e8m0) return DTQ_ERR_INVALID_ARGUMENT;
  // 16-byte loads of the input, 8-byte stores of the payload, 16-byte stores of the transposed payload
  if (!aligned_to(in_bf16, 16) || !aligned_to(payload, 8) || !aligned_to(payload_t, 16)) return DTQ_ERR_INVALID_ARGUMENT;
  const int64_t row_tiles = ceil_div64(rows, kTile), col_tiles = ceil_div64(cols, kTile);
  if (row_tiles > 0x7FFFFFFFLL / col_tiles) return DTQ_ERR_TOO_LARGE;  // grid.x
  auto kernel = row_out ? mx_dual_kernel<BLOCKED, true> : mx_dual_kernel<BLOCKED, false>;
  return cuda_status(launch_after_dependency(kernel, dim3(static_cast<unsigned>(row_tiles * col_tiles)), dim3(kThreadsDual), 0,
                                             static_cast<cudaStream_t>(stream), static_cast<const uint16_t *>(in_bf16),
                                             static_cast<uint8_t *>(payload), static_cast<uint8_t *>(scales_e8m0),
                                             static_cast<uint8_t *>(payload_t), static_cast<uint8_t *>(scales_t_e8m0), rows, cols,
                                             row_tiles, col_tiles));
}
}  // namespace
}  // namespace dtq

extern "C" int dtq_mx_fp8_quantize_dual(const void *in_bf16, void *payload, void *scales_e8m0, void *payload_t,
                                        void *scales_t_e8m0, int64_t rows, int64_t cols, void *stream) {
  return dtq::launch_dual<false>(in_bf16, payload, scales_e8m0, payload_t, scales_t_e8m0, rows, cols, stream);
}

extern "C" int dtq_mx_fp8_quantize_dual_blocked(const void *in_bf16, void *payload, void *scales_e8m0, void *payload_t,
                                                void *scales_t_e8m0, int64_t rows, int64_t cols, void *stream) {
  return dtq::launch_dual<true>(in_bf16, payload, scales_e8m0, payload_t, scales_t_e8m0, rows, cols, stream);
}
