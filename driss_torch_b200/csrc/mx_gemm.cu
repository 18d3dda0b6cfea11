// mx_fp8_bf16: D[M,N] (bf16) = sum_k  A[m,k] * 2^(sa[m,k/32]-127) * B[n,k] * 2^(sb[n,k/32]-127)
//
// The consumer of the MX casts: e4m3 operands with one E8M0 scale per 32 elements along K, both
// scale tensors in the blocked (128 x 4 atoms of 512 bytes) layout that mx_fp8_quantize_blocked
// emits.  Replaces driss_torch::mx_fp8_bf16 (src/mx_fp8_bf16.cu:42-163 run_gemm, :168-215 validate,
// :217-241), which instantiates a CUTLASS Sm100 block-scaled collective with 128x128x128 tiles; and, from
// the same source, mx_fp4_bf16 (:243-271) and the row-wise scaled GEMM behind sweep_mm (src/sweep_mm.cu,
// src/scaled_mm_kernels/f8f8bf16_rowwise_kernel.h:151-175), see Format below.
//
// Hand-written for sm_100a.  Three kernels from one source (chosen per call by a measured cost model, see
// launch_gemm): an SM pair on a 256 x 256 tile (tcgen05.mma.cta_group::2, further down), and one CTA per SM on a
// 128 x 256 or a 128 x 128 tile (this kernel).  Common to all:
//   * persistent CTAs of 320 threads walk the output tiles; K advances in stages of 128 bytes;
//   * warp 0 is the producer: per stage tiled TMA loads of the operands (boxes of 128 bytes of K, 128-byte
//     swizzle, rows and columns past the edges filled with zeros) and of the stage's scale atoms (a 3-D tensor
//     map over the blocked scale array, an atom past the end arrives as zeros), all counted on the stage's `full`
//     mbarrier;
//   * warp 1 issues the tensor-core work: tcgen05.cp moves the stage's scale atoms from shared memory into
//     tensor memory (32 rows x 16 bytes, replicated to the four lane quadrants, which is exactly one blocked
//     atom), then four tcgen05.mma (K = 32 bytes of every operand row each), the k-block picking its scale byte
//     through the descriptor's scale-factor id; tcgen05.commit releases the stage (`empty`) and finally hands
//     the accumulator (128 lanes x up to 256 fp32 columns of tensor memory) to the epilogue;
//   * both of those warps walk their loops as whole warps with one elected lane issuing (see elect_one);
//   * warps 2..9 are the epilogue: tcgen05.ld 2 x 32 columns at a time, fp32 -> bf16, 64-byte row segments
//     straight to global memory; the accumulator is released as soon as it is in registers, so the next tile's
//     MMAs overlap the stores.
// No load is shared between CTAs: every CTA loads its own operands (A and B of an 8192^3 problem both fit in
// L2).  Every wait is bounded: a wait that runs out records DTQ_ERR_TIMEOUT in the status word, raises the CTA's
// abort flag, the roles drain what they have in flight, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "dtq_device.cuh"
#include "dtq_host.h"

namespace dtq {
namespace {

constexpr int kBM = 128;        // tile rows (M)
constexpr int kBK = 128;        // K bytes per stage: one 128-byte swizzle span = 4 MX blocks of 32
constexpr int kGemmThreads = 320;  // producer warp, MMA warp, 8 epilogue warps
constexpr int kEpilogueWarps = 8;
constexpr int kSfaCol = 256;               // scales of A: 4 tensor-memory columns per atom (128 rows x 4 k-blocks)
constexpr int kSfbCol = 256 + 16;          // scales of B: 4 columns per atom, up to 2 (N) x 2 (K) atoms
// Element formats.  e4m3: one byte per element, a 128-byte stage is 128 elements = 4 MX blocks = one scale atom
// along K, tcgen05.mma kind::mxf8f6f4 (K = 32 per instruction, one scale byte each for A and B).  e2m1 (MXFP4): two
// elements per byte, a 128-byte stage is 256 elements = 8 MX blocks = two scale atoms along K, kind::mxf4 with
// block32 scaling (K = 64 per instruction, which uses two consecutive scale bytes).  Either way an instruction
// reads 32 bytes of every operand row, so the operand descriptors are the same.
//
// A third mode has no block scales at all: fp8 operands (e4m3, or e5m2 for A) through kind::f8f6f4, with one fp32
// scale per row of A and per row of B (and an optional bias per column) applied to the fp32 accumulator in the
// epilogue -- the row-wise scaled GEMM that consumes dtq_dynamic_scaled_quant_rowwise's scales.
constexpr int kMxFp8 = 0, kMxFp4 = 1, kRowwise = 2;
template <int MODE>
struct Format {
  static constexpr bool kScaled = MODE != kRowwise;            // block scales travel with the operands
  static constexpr int kKAtoms = MODE == kMxFp4 ? 2 : 1;      // scale atoms along K per stage (staging is sized for them)
  // k (0..3) = the instruction within a stage: which atom along K, and which byte (pair) of its 4-byte scale columns
  __device__ static constexpr uint32_t k_atom(uint32_t k) { return MODE == kMxFp4 ? k >> 1 : 0u; }
  __device__ static constexpr uint32_t sf_id(uint32_t k) { return MODE == kMxFp4 ? (k & 1u) * 2u : (MODE == kMxFp8 ? k : 0u); }
  // instruction-descriptor bits besides the shape: block-scaled kinds carry the scale format (bit 23 = E8M0) and for
  // kind::mxf4 the e2m1 operand format; kind::f8f6f4 carries the accumulator format (bits 4-5 = fp32), the operand
  // formats come with the call (e4m3 = 0 or e5m2 = 1 in bits 7-9 / 10-12)
  static constexpr uint32_t kFormatBits = MODE == kMxFp4 ? ((1u << 7) | (1u << 10) | (1u << 23)) : (MODE == kMxFp8 ? (1u << 23) : (1u << 4));
};
constexpr int kTmemCols = 512;             // allocation (power of two); columns 0..255 hold the accumulator(s)

// Two tile shapes.  Wide: 128 x 256, one accumulator of 256 columns, 4 stages -- least operand traffic per
// output (every byte of B serves 128 rows, every byte of A 256 columns), the shape for large problems.
// Narrow: 128 x 128, two accumulators of 128 columns (the epilogue of one tile runs under the MMAs of the
// next), 6 stages -- twice the tiles, for problems whose wide tiles would leave a large part of the last wave
// of SMs idle.
template <int BN_, int STAGES_, int ACC_>
struct GemmShape {
  static constexpr int BN = BN_, STAGES = STAGES_, ACC = ACC_;
  static_assert(BN == 128 || BN == 256, "N tile");
  static_assert(ACC * BN <= 256, "accumulators live in tensor-memory columns 0..255");
};
using WideShape = GemmShape<256, 4, 1>;
using NarrowShape = GemmShape<128, 6, 2>;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // a wait gives up after two seconds of wall time

template <typename SH, int MODE>
struct __align__(1024) GemmSmem {
  uint8_t a[SH::STAGES][kBM * kBK];        // 16 KB per stage, 1024-byte aligned (swizzle atom = 8 rows x 128 B)
  uint8_t b[SH::STAGES][SH::BN * kBK];     // 16 or 32 KB per stage
  uint8_t sfa[SH::STAGES][Format<MODE>::kKAtoms * 512];                  // blocked atoms of 128 rows x 4 k-blocks
  uint8_t sfb[SH::STAGES][SH::BN / 128 * Format<MODE>::kKAtoms * 512];  // [128 tile columns][atom along K]
  uint64_t full[SH::STAGES];
  uint64_t empty[SH::STAGES];
  uint64_t tmem_full[SH::ACC];
  uint64_t tmem_empty[SH::ACC];
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// One poll of the phase with the given parity; the thread may sleep up to about a microsecond inside it.
__device__ __forceinline__ bool mbar_poll(uint32_t addr, unsigned parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(addr), "r"(parity), "r"(1000u)
      : "memory");
  return done != 0;
}
// Bounded wait for the phase of the given parity: false if it has not completed after kWaitLimitNs of
// wall time, or if the CTA is aborting (`abort` may be null for a wait that must not be cut short).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, volatile int *abort) {
  const uint32_t addr = smem_addr(bar);
  if (mbar_poll(addr, parity)) return true;
  const unsigned long long start = global_ns();
  for (unsigned int spins = 1;; ++spins) {
    if (mbar_poll(addr, parity)) return true;
    if ((spins & 63u) == 0) {
      if (abort && *abort) return false;
      if (global_ns() - start > kWaitLimitNs) return false;
    }
  }
}
// The same wait by all lanes of a converged warp, with one answer for the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, unsigned parity, volatile int *abort) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort));
}
// True in one lane of a converged warp, the same lane every time.  The producer and the MMA issuer walk their
// loops as whole warps and let the elected lane issue the asynchronous instructions: everything those
// instructions take as operands (descriptors, coordinates, barrier addresses) is then the same in all lanes,
// which lets the compiler keep it in the warp's uniform registers, where TMA and tcgen05 instructions read
// their operands from.  A loop walked by a single lane instead pays a transfer into uniform registers for
// every operand of every instruction: measured here, 55 to 75 clocks per tcgen05 instruction, which made the
// issuing thread, not the tensor cores, the limit of the kernel.
__device__ __forceinline__ bool elect_one() {
  uint32_t elected;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
  return elected != 0;
}
// A value that is the same in every lane, in a form the compiler can see is.
__device__ __forceinline__ uint32_t warp_uniform(uint32_t v) { return __shfl_sync(0xFFFFFFFFu, v, 0); }

// Tiled TMA load of a box at (x = byte column, y = row) into this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_addr(dst)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                   smem_addr(dst)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes long and
// 128-byte swizzled (what the TMA loads above produce): start address, leading byte offset (unused
// for swizzled K-major tiles, encoded as 1), stride between 8-row groups = 1024 bytes, descriptor
// version 1, layout type 2 = 128-byte swizzle.  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  return uint64_t((saddr >> 4) & 0x3FFFu) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
// Descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle; 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t scale_desc(uint32_t saddr) {
  return uint64_t((saddr >> 4) & 0x3FFFu) | (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
}
// Instruction descriptor of tcgen05.mma kind::mxf8f6f4.block_scale: e4m3 x e4m3, both K-major, E8M0 scales,
// M = 128, N = `bn`; `k` (0..3) is the byte of the 4-byte scale column that this k-block uses, for A and B.
__device__ __forceinline__ uint32_t instr_desc(uint32_t sf_id, uint32_t bn, uint32_t m, uint32_t format_bits) {
  return (sf_id << 4) | format_bits | ((bn >> 3) << 17) | ((m >> 4) << 24) | (sf_id << 29);
}
// One MMA: D (tensor memory) (+)= A x B, block-scaled kinds with the scales found at the two tensor-memory addresses.
template <int MODE, bool PAIR>
__device__ __forceinline__ void issue_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem) {
#define DTQ_MMA(GROUP, KIND)                                                                                         \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                     \
               "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], %1, %2, %3, [%5], [%6], p;\n\t}"                \
               :                                                                                                     \
               : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)    \
               : "memory")
  if constexpr (MODE == kMxFp4 && PAIR) DTQ_MMA("2", "mxf4.block_scale.block32");
  else if constexpr (MODE == kMxFp4) DTQ_MMA("1", "mxf4.block_scale.block32");
  else if constexpr (MODE == kMxFp8 && PAIR) DTQ_MMA("2", "mxf8f6f4.block_scale");
  else if constexpr (MODE == kMxFp8) DTQ_MMA("1", "mxf8f6f4.block_scale");
  else if constexpr (PAIR)  // no block scales; the braces hold the (unused) mask of output lanes to leave alone
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 :
                 : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 :
                 : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
#undef DTQ_MMA
}
// One scale atom, shared memory -> 4 tensor-memory columns (32 rows x 16 bytes, replicated to the four lane quadrants).
template <bool PAIR>
__device__ __forceinline__ void copy_scale_atom(uint32_t tmem_col_addr, uint32_t smem_atom_addr) {
  if constexpr (PAIR)
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col_addr), "l"(scale_desc(smem_atom_addr)) : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col_addr), "l"(scale_desc(smem_atom_addr)) : "memory");
}

__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// fp32 pair -> packed bf16x2 (lo in the low half).
__device__ __forceinline__ uint32_t pack_bf16(uint32_t lo, uint32_t hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
  return r;
}

// Tile order: consecutive tile numbers (the tiles that the CTAs of one wave work on together) fill bands of
// kGroupM tile rows, n-tile by n-tile, so that a wave of 148 tiles touches about 16 x 9 tiles' worth of A
// and B (34 MB at K = 8192) instead of every row of A: what is re-read from L2 mostly stays there.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int *mt, int *nt) {
  const int per_group = kGroupM * n_tiles;
  const int g = tile / per_group, idx = tile - g * per_group;
  const int rows = min(kGroupM, m_tiles - g * kGroupM);
  *mt = g * kGroupM + idx % rows;
  *nt = idx / rows;
}

// The row-wise mode's epilogue: out = bf16(fp32(fp32(acc * row_scale[m]) * col_scale[n]) + bias[n]), every step rounded
// to fp32 (src/scaled_mm_kernels/f8f8bf16_rowwise_kernel.h:151-175: Multiply(WScale, Multiply(XScale, Acc)), Add(Bias), Cast).
struct RowwiseEpilogue {
  const float *row_scale;  // [M]
  const float *col_scale;  // [N]
  const void *bias;        // [N] fp32 or bf16, or null
  int bias_is_bf16;
  uint32_t operand_format_bits;  // a_format << 7 | b_format << 10 (e4m3 = 0, e5m2 = 1)
};
// What a thread of the epilogue needs of the scales for one tile, fetched BEFORE it waits for the accumulator (none of
// it depends on the MMAs): its row's scale, and for each 32-column chunk of its columns the scale and bias of column
// `lane` of the chunk; the value for column i of a chunk then comes from lane i by shuffle.  Columns past N get 0.
template <int CHUNKS>
struct RowwiseRegs {
  float xs;
  float cs[CHUNKS], bs[CHUNKS];
  bool has_bias;
};
template <int CHUNKS>
__device__ __forceinline__ void load_rowwise(RowwiseRegs<CHUNKS> &r, const RowwiseEpilogue &e, int64_t row, int64_t col0, int lane,
                                             int M, int N) {
  r.xs = row < M ? __ldg(e.row_scale + row) : 0.0f;
  r.has_bias = e.bias != nullptr;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int64_t col = col0 + c * 32 + lane;
    const bool live = col < N;
    r.cs[c] = live ? __ldg(e.col_scale + col) : 0.0f;
    r.bs[c] = 0.0f;
    if (live && r.has_bias)
      r.bs[c] = e.bias_is_bf16 ? __uint_as_float(uint32_t(__ldg(static_cast<const uint16_t *>(e.bias) + col)) << 16)
                               : __ldg(static_cast<const float *>(e.bias) + col);
  }
}
// 32 consecutive accumulator columns of one row (fp32 bit patterns) through the row-wise epilogue, in place:
// bf16((acc * x_scale[row]) * w_scale[col] + bias[col]), every step rounded to fp32 as the reference's epilogue tree does.
__device__ __forceinline__ void apply_rowwise(uint32_t (&v)[32], float xs, float cs, float bs, bool has_bias) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float f = __fmul_rn(__fmul_rn(__uint_as_float(v[i]), xs), __shfl_sync(0xFFFFFFFFu, cs, i));
    const float b = __shfl_sync(0xFFFFFFFFu, bs, i);
    if (has_bias) f = __fadd_rn(f, b);
    v[i] = __float_as_uint(f);
  }
}

// 32 accumulator columns of this thread's lane of tensor memory into registers (asynchronous: tmem_load_wait).
__device__ __forceinline__ void tmem_load_32(uint32_t (&v)[32], uint32_t taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct GemmParams {
  RowwiseEpilogue rowwise;
  uint16_t *out;  // bf16 [M, N]
  int M, N, K;
  int m_tiles, n_tiles, k_stages;
  int *status;
};

template <typename SH, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb, GemmParams p) {
  constexpr int kBN = SH::BN, kStagesG = SH::STAGES, kAcc = SH::ACC, kAtomsB = SH::BN / 128;
  constexpr int kKAtoms = Format<MODE>::kKAtoms;
  extern __shared__ unsigned char smem_raw[];
  GemmSmem<SH, MODE> &sm =
      *reinterpret_cast<GemmSmem<SH, MODE> *>(smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u));
  const int warp = int(warp_uniform(threadIdx.x >> 5)), lane = threadIdx.x & 31;
  volatile int *abort = &sm.abort;
  // Programmatic dependent launch, both ways: what is queued behind this kernel with that attribute may become
  // resident as this grid's CTAs leave, and this kernel's own set-up below (barriers, tensor memory, the tensor
  // maps in its parameters) may run under the tail of the kernel before it; nothing in global memory is touched
  // before pdl_wait.
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesG; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int i = 0; i < kAcc; ++i) {
      mbar_init(&sm.tmem_full[i], 1);
      mbar_init(&sm.tmem_empty[i], kEpilogueWarps);
    }
    sm.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the MMA warp owns tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  pdl_wait();  // the operands, the scales and the output buffer belong to this kernel from here on
  const uint32_t tmem = warp_uniform(sm.tmem_base);
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ---- producer: the warp walks the loop, the elected lane issues ------------------------------------
    uint32_t stage = 0, phase = 0;  // `phase`: parity of the current pass over the ring of stages
    bool first_pass = true, ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int mt, nt;
      tile_coords(tile, p.m_tiles, p.n_tiles, &mt, &nt);
      for (int ks = 0; ks < p.k_stages; ++ks) {
        // the MMAs that read this stage's previous contents (one pass ago) must have finished
        if (!first_pass && !mbar_wait_warp(&sm.empty[stage], phase ^ 1u, abort)) {
          ok = false;
          break;
        }
        if (elect_one()) {
          // a whole box always arrives: rows, columns and scale atoms past the end of the arrays come as zeros
          mbar_expect_tx(&sm.full[stage],
                         kBM * kBK + kBN * kBK + (Format<MODE>::kScaled ? (1 + kAtomsB) * kKAtoms * 512 : 0));
          tma_load_2d(sm.a[stage], &map_a, ks * kBK, mt * kBM, &sm.full[stage]);
          tma_load_2d(sm.b[stage], &map_b, ks * kBK, nt * kBN, &sm.full[stage]);
          if constexpr (Format<MODE>::kScaled) {  // one box each: A's atoms along K; B's for kAtomsB rows of atoms
            tma_load_3d(sm.sfa[stage], &map_sfa, 0, ks * kKAtoms, mt, &sm.full[stage]);
            tma_load_3d(sm.sfb[stage], &map_sfb, 0, ks * kKAtoms, nt * kAtomsB, &sm.full[stage]);
          }
        }
        __syncwarp();
        if (++stage == kStagesG) {
          stage = 0;
          phase ^= 1u;
          first_pass = false;
        }
      }
    }
    if (!ok && lane == 0) {
      // Give up, but not with copies on their way into this CTA's shared memory: wait (bounded) for the newest
      // copy of every stage (this pass's below `stage`, the previous pass's from there on); they complete
      // without anybody's help.
      atomicExch(p.status, DTQ_ERR_TIMEOUT);
      *abort = 1;
      for (uint32_t j = 0; j < uint32_t(kStagesG); ++j) {
        if (j < stage) mbar_wait(&sm.full[j], phase, nullptr);
        else if (!first_pass) mbar_wait(&sm.full[j], phase ^ 1u, nullptr);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the warp walks the loop, the elected lane issues ---------------------------------------
    uint32_t stage = 0, phase = 0;
    int local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
      // the epilogue must have taken this accumulator's previous tile out of tensor memory
      const int acc = local_tile % kAcc, use = local_tile / kAcc;
      if (use > 0 && !mbar_wait_warp(&sm.tmem_empty[acc], (use - 1) & 1u, abort)) {
        ok = false;
        break;
      }
      tmem_fence_after();
      const uint32_t d_tmem = tmem + uint32_t(acc * kBN);
      for (int ks = 0; ks < p.k_stages; ++ks) {
        if (!mbar_wait_warp(&sm.full[stage], phase, abort)) {
          ok = false;
          break;
        }
        tmem_fence_after();
        if (elect_one()) {
          // this stage's scales: shared memory -> tensor memory, ordered before the MMAs below.  Tensor-memory
          // columns: A's atom j along K at kSfaCol + 4 j; B's at kSfbCol + j * 4 kAtomsB + 4 h (h = 128 tile columns)
          if constexpr (Format<MODE>::kScaled) {
#pragma unroll
            for (int j = 0; j < kKAtoms; ++j) {
              copy_scale_atom<false>(tmem + kSfaCol + 4 * j, smem_addr(sm.sfa[stage] + j * 512));
#pragma unroll
              for (int h = 0; h < kAtomsB; ++h)
                copy_scale_atom<false>(tmem + kSfbCol + j * 4 * kAtomsB + 4 * h,
                                       smem_addr(sm.sfb[stage] + (h * kKAtoms + j) * 512));
            }
          }
          const uint32_t a_addr = smem_addr(sm.a[stage]), b_addr = smem_addr(sm.b[stage]);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {  // four instructions of 32 operand bytes inside the 128-byte swizzle span
            const uint32_t accumulate = (ks > 0 || k > 0) ? 1u : 0u;
            const uint32_t j = Format<MODE>::k_atom(k), id = Format<MODE>::sf_id(k);
            issue_mma<MODE, false>(d_tmem, operand_desc(a_addr + k * 32), operand_desc(b_addr + k * 32),
                                  instr_desc(id, kBN, kBM, Format<MODE>::kFormatBits | p.rowwise.operand_format_bits), accumulate,
                                  (tmem + kSfaCol + 4 * j) | (id << 30), (tmem + kSfbCol + j * 4 * kAtomsB) | (id << 30));
          }
          umma_commit(&sm.empty[stage]);  // the stage is free once these MMAs have read it
        }
        __syncwarp();
        if (++stage == kStagesG) {
          stage = 0;
          phase ^= 1u;
        }
      }
      // the accumulator is complete once all MMAs so far have finished
      if (ok && elect_one()) umma_commit(&sm.tmem_full[acc]);
      __syncwarp();
    }
    if (!ok && lane == 0) {
      atomicExch(p.status, DTQ_ERR_TIMEOUT);
      *abort = 1;
    }
  } else {
    // ---- epilogue: 8 warps; warp w reads lanes 32 (w % 4) .. + 31, column half (w - 2) / 4 -------------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    constexpr int kHalfCols = kBN / 2, kChunks = kHalfCols / 32;  // each warp takes half the tile's columns, 32 at a time
    int local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      int mt, nt;
      tile_coords(tile, p.m_tiles, p.n_tiles, &mt, &nt);
      const int acc = local_tile % kAcc, use = local_tile / kAcc;
      const int64_t row = int64_t(mt) * kBM + quad * 32 + lane;
      RowwiseRegs<kChunks> rw;
      if constexpr (MODE == kRowwise)
        load_rowwise<kChunks>(rw, p.rowwise, row, int64_t(nt) * kBN + half * kHalfCols, lane, p.M, p.N);
      if (!mbar_wait(&sm.tmem_full[acc], use & 1u, abort)) {
        if (lane == 0) {
          atomicExch(p.status, DTQ_ERR_TIMEOUT);
          *abort = 1;
        }
        break;
      }
      tmem_fence_after();
      uint32_t packed[kChunks][16];  // this thread's columns of one row as bf16 pairs
#pragma unroll
      for (int c = 0; c < kChunks; c += 2) {  // two loads in flight per wait: the accumulator is handed back sooner
        uint32_t v[2][32];
        const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(acc * kBN + half * kHalfCols + c * 32);
        tmem_load_32(v[0], taddr);
        tmem_load_32(v[1], taddr + 32);
        tmem_load_wait();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if constexpr (MODE == kRowwise) apply_rowwise(v[u], rw.xs, rw.cs[c + u], rw.bs[c + u], rw.has_bias);
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[c + u][i] = pack_bf16(v[u][2 * i], v[u][2 * i + 1]);
        }
      }
      // the accumulator is in registers: hand tensor memory back before storing
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.tmem_empty[acc]);
      if (row < p.M) {
        uint16_t *dst = p.out + row * p.N + int64_t(nt) * kBN + half * kHalfCols;
        const int64_t col0 = int64_t(nt) * kBN + half * kHalfCols;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // 8 columns = 16 bytes per store; N % 8 == 0
            if (col0 + c * 32 + q * 8 < p.N)
              stg_stream(dst + c * 32 + q * 8,  // streaming store: the output must not push the operands out of L2
                         make_uint4(packed[c][4 * q], packed[c][4 * q + 1], packed[c][4 * q + 2], packed[c][4 * q + 3]));
          }
        }
      }
    }
  }

  // ---- teardown: everybody meets, then the warp that allocated tensor memory frees it ----------------------
  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort && elect_one()) {  // the lane that issued the MMAs: a commit follows the issuing thread's own
      // MMAs may still be in flight: a commit that arrives on a barrier nobody else uses, and a bounded wait for it
      mbar_init(&sm.tmem_full[0], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      umma_commit(&sm.tmem_full[0]);
      mbar_wait(&sm.tmem_full[0], 0u, nullptr);
    }
    __syncwarp();
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- two SMs on one tile ----------------------------------------------------------------------------------
// The kernel above is bound by what one SM can pull out of L2 (about 64 bytes per clock): a 128 x 256 tile
// needs 48 KB of operands per 128 of K.  Here two CTAs of a cluster (an SM pair) share a 256 x 256 tile:
// tcgen05.mma.cta_group::2 multiplies M = 256 (each CTA supplies 128 rows of A and receives their 128 x 256
// accumulator in its own tensor memory) by N = 256 (each CTA supplies 128 of the 256 rows of B), so every CTA
// loads 16 + 16 KB per stage instead of 16 + 32: a third less traffic per flop, and room for 6 stages.
//   * both CTAs' producers load their own halves (TMA, .cta_group::2, each CTA for itself) and signal the LEADER
//     CTA's `full` barrier (the even CTA of the pair); the leader alone expects the bytes of both;
//   * the scale atoms come in through a 3-D tensor map over the blocked scale array ([atom row][atom column]
//     [512 bytes]), so that a missing atom is simply filled with zeros; every CTA needs its own A atom and
//     both B atoms (its accumulator spans all 256 columns);
//   * the leader's MMA thread copies the scales (tcgen05.cp.cta_group::2: each CTA's shared memory into that
//     CTA's tensor memory), issues the MMAs, and commits twice per barrier, once for each CTA's copy of it;
//   * the peer's epilogue warps arrive on the leader's `tmem_empty` barrier through the cluster address space.
// Every wait is bounded as above; an abort is forwarded to the other CTA, and both always meet at the cluster
// barrier before tensor memory is freed.
constexpr int kPairStages = 6;
constexpr int kPairBN = 256;  // tile columns; each CTA holds kPairBN / 2 rows of B

template <int MODE>
struct __align__(1024) PairSmem {
  uint8_t a[kPairStages][kBM * kBK];             // this CTA's 128 rows of A
  uint8_t b[kPairStages][kPairBN / 2 * kBK];     // this CTA's 128 of the tile's 256 rows of B
  uint8_t sfa[kPairStages][Format<MODE>::kKAtoms * 512];      // scales of this CTA's 128 rows of A
  uint8_t sfb[kPairStages][2 * Format<MODE>::kKAtoms * 512];  // scales of all 256 rows of B: [128 columns][atom along K]
  uint64_t full[kPairStages];                    // used in the leader CTA only
  uint64_t empty[kPairStages];
  uint64_t tmem_full;
  uint64_t tmem_empty;                           // used in the leader CTA only
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared address space, of `local` (an address of this CTA's shared memory) in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA loads of the pair kernel: destination in this CTA, completion counted on a barrier given by its cluster address.
__device__ __forceinline__ void tma_pair_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

struct PairParams {
  RowwiseEpilogue rowwise;
  uint16_t *out;  // bf16 [M, N]
  int M, N;
  int m_pairs, n_tiles, k_stages;  // 256-row tile rows, 256-column tile columns, 128-byte K stages
  int *status;
};

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb, PairParams p) {
  constexpr int kKAtoms = Format<MODE>::kKAtoms;
  extern __shared__ unsigned char smem_raw[];
  PairSmem<MODE> &sm = *reinterpret_cast<PairSmem<MODE> *>(smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u));
  const int warp = int(warp_uniform(threadIdx.x >> 5)), lane = threadIdx.x & 31;
  const uint32_t rank = warp_uniform(cluster_ctarank());  // 0 = leader
  const bool leader = rank == 0;
  const uint32_t peer = rank ^ 1u;
  volatile int *abort = &sm.abort;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int total_tiles = p.m_pairs * p.n_tiles;
  pdl_launch_dependents();  // as in the single-CTA kernel

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&sm.full[s], 1);   // the leader's producer arrives once, expecting both CTAs' bytes
      mbar_init(&sm.empty[s], 1);  // one commit of the leader's MMA thread per CTA
    }
    mbar_init(&sm.tmem_full, 1);
    mbar_init(&sm.tmem_empty, 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    sm.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // one warp of each CTA, together: 512 columns in both CTAs' tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals them
  tmem_fence_after();
  pdl_wait();
  const uint32_t tmem = warp_uniform(sm.tmem_base);

  if (warp == 0) {
    // ---- producer (in each CTA): the warp walks the loop, the elected lane issues ------------------------------
    uint32_t stage = 0, phase = 0;
    bool first_pass = true, ok = true;
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
      int mp, nt;
      tile_coords(tile, p.m_pairs, p.n_tiles, &mp, &nt);
      for (int ks = 0; ks < p.k_stages; ++ks) {
        if (!first_pass && !mbar_wait_warp(&sm.empty[stage], phase ^ 1u, abort)) {
          ok = false;
          break;
        }
        if (elect_one()) {
          const uint32_t bar = map_to_cta(smem_addr(&sm.full[stage]), 0);  // the leader's barrier
          if (leader)
            mbar_expect_tx(&sm.full[stage],
                           2 * (kBM * kBK + kPairBN / 2 * kBK + (Format<MODE>::kScaled ? 3 * kKAtoms * 512 : 0)));
          tma_pair_load_2d(sm.a[stage], &map_a, ks * kBK, mp * 256 + int(rank) * kBM, bar);
          tma_pair_load_2d(sm.b[stage], &map_b, ks * kBK, nt * kPairBN + int(rank) * (kPairBN / 2), bar);
          if constexpr (Format<MODE>::kScaled) {
            tma_pair_load_3d(sm.sfa[stage], &map_sfa, 0, ks * kKAtoms, mp * 2 + int(rank), bar);
            tma_pair_load_3d(sm.sfb[stage], &map_sfb, 0, ks * kKAtoms, nt * 2, bar);
          }
        }
        __syncwarp();
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1u;
          first_pass = false;
        }
      }
    }
    if (!ok && lane == 0) {
      atomicExch(p.status, DTQ_ERR_TIMEOUT);
      *abort = 1;
      st_cluster_u32(map_to_cta(smem_addr(&sm.abort), peer), 1u);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader's warp walks the loop, its elected lane drives both SMs' tensor cores ---------
    if (leader) {
      uint32_t stage = 0, phase = 0;
      int local_tile = 0;
      bool ok = true;
      const uint32_t peer_full = map_to_cta(smem_addr(&sm.tmem_full), 1);
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++local_tile) {
        if (local_tile > 0 && !mbar_wait_warp(&sm.tmem_empty, (local_tile - 1) & 1u, abort)) {
          ok = false;
          break;
        }
        tmem_fence_after();
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!mbar_wait_warp(&sm.full[stage], phase, abort)) {
            ok = false;
            break;
          }
          tmem_fence_after();
          if (elect_one()) {
            if constexpr (Format<MODE>::kScaled) {
#pragma unroll
              for (int j = 0; j < kKAtoms; ++j) {  // each CTA's shared memory -> that CTA's tensor memory, columns as above
                copy_scale_atom<true>(tmem + kSfaCol + 4 * j, smem_addr(sm.sfa[stage] + j * 512));
#pragma unroll
                for (int h = 0; h < 2; ++h)
                  copy_scale_atom<true>(tmem + kSfbCol + j * 8 + 4 * h, smem_addr(sm.sfb[stage] + (h * kKAtoms + j) * 512));
              }
            }
            const uint32_t a_addr = smem_addr(sm.a[stage]), b_addr = smem_addr(sm.b[stage]);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
              const uint32_t accumulate = (ks > 0 || k > 0) ? 1u : 0u;
              const uint32_t j = Format<MODE>::k_atom(k), id = Format<MODE>::sf_id(k);
              issue_mma<MODE, true>(tmem, operand_desc(a_addr + k * 32), operand_desc(b_addr + k * 32),
                                   instr_desc(id, kPairBN, 256, Format<MODE>::kFormatBits | p.rowwise.operand_format_bits),
                                   accumulate, (tmem + kSfaCol + 4 * j) | (id << 30), (tmem + kSfbCol + j * 8) | (id << 30));
            }
            // the stage is free in both CTAs once these MMAs have read it
            const uint32_t empty_bar = smem_addr(&sm.empty[stage]);
            umma_commit_pair(empty_bar);
            umma_commit_pair(map_to_cta(empty_bar, 1));
          }
          __syncwarp();
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && elect_one()) {  // both CTAs' halves of the accumulator are complete once all MMAs so far have finished
          umma_commit_pair(smem_addr(&sm.tmem_full));
          umma_commit_pair(peer_full);
        }
        __syncwarp();
      }
      if (!ok && lane == 0) {
        atomicExch(p.status, DTQ_ERR_TIMEOUT);
        *abort = 1;
        st_cluster_u32(map_to_cta(smem_addr(&sm.abort), peer), 1u);
      }
    }
  } else {
    // ---- epilogue: this CTA's 128 rows of the tile, 8 warps as in the single-CTA kernel --------------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const uint32_t leader_empty = map_to_cta(smem_addr(&sm.tmem_empty), 0);
    int local_tile = 0;
    for (int tile = cluster_id; tile < total_tiles; tile += n_clusters, ++local_tile) {
      int mp, nt;
      tile_coords(tile, p.m_pairs, p.n_tiles, &mp, &nt);
      const int64_t row = int64_t(mp) * 256 + int64_t(rank) * kBM + quad * 32 + lane;
      RowwiseRegs<4> rw;
      if constexpr (MODE == kRowwise) load_rowwise<4>(rw, p.rowwise, row, int64_t(nt) * kPairBN + half * 128, lane, p.M, p.N);
      if (!mbar_wait(&sm.tmem_full, local_tile & 1u, abort)) {
        if (lane == 0) {
          atomicExch(p.status, DTQ_ERR_TIMEOUT);
          *abort = 1;
          st_cluster_u32(map_to_cta(smem_addr(&sm.abort), peer), 1u);
        }
        break;
      }
      tmem_fence_after();
      uint32_t packed[4][16];
#pragma unroll
      for (int c = 0; c < 4; c += 2) {  // two loads in flight per wait
        uint32_t v[2][32];
        const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(half * 128 + c * 32);
        tmem_load_32(v[0], taddr);
        tmem_load_32(v[1], taddr + 32);
        tmem_load_wait();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if constexpr (MODE == kRowwise) apply_rowwise(v[u], rw.xs, rw.cs[c + u], rw.bs[c + u], rw.has_bias);
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[c + u][i] = pack_bf16(v[u][2 * i], v[u][2 * i + 1]);
        }
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_empty);
      if (row < p.M) {
        uint16_t *dst = p.out + row * p.N + int64_t(nt) * kPairBN + half * 128;
        const int64_t col0 = int64_t(nt) * kPairBN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col0 + c * 32 + q * 8 < p.N)
              stg_stream(dst + c * 32 + q * 8,
                         make_uint4(packed[c][4 * q], packed[c][4 * q + 1], packed[c][4 * q + 2], packed[c][4 * q + 3]));
          }
        }
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------------------
  // whoever gave up has already raised both CTAs' abort flags
  tmem_fence_before();
  __syncthreads();
  if (*abort) {
    // Copies and MMAs may still be in flight into or out of this CTA's memories.  Loads complete by themselves
    // within microseconds and the leader's MMAs within a tile's time; neither CTA leaves before the other
    // (cluster barrier below), and a short sleep here covers what was issued last.
    __nanosleep(200000);
  }
  cluster_sync_all();  // nobody's shared or tensor memory goes away while the other CTA may still touch it
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (no link against libcuda).
int encode_tiled_fn(EncodeTiledFn *fn) {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn f = cached.load(std::memory_order_acquire);
  if (!f) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    DTQ_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !sym) return DTQ_ERR_CUDA_BASE + static_cast<int>(cudaErrorNotSupported);
    f = reinterpret_cast<EncodeTiledFn>(sym);
    cached.store(f, std::memory_order_release);
  }
  *fn = f;
  return DTQ_OK;
}

// Map of a row-major [rows, k_bytes] byte matrix, boxes of box_rows x 128 bytes, 128-byte swizzle, zero fill.
int make_operand_map(CUtensorMap *map, const void *base, int64_t rows, int64_t k_bytes, int box_rows) {
  EncodeTiledFn encode = nullptr;
  if (int e = encode_tiled_fn(&encode)) return e;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DTQ_OK : DTQ_ERR_INVALID_ARGUMENT;
}

// Map of a blocked scale array as [atom rows][atoms along K][512 bytes]: boxes of `box_rows` x `box_katoms` atoms.
// Atoms past the end are delivered as zeros.
int make_scale_map(CUtensorMap *map, const void *base, int64_t atom_rows, int64_t katoms, int box_rows, int box_katoms) {
  EncodeTiledFn encode = nullptr;
  if (int e = encode_tiled_fn(&encode)) return e;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(katoms), static_cast<cuuint64_t>(atom_rows)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(512 * katoms)};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(box_katoms), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(base), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DTQ_OK : DTQ_ERR_INVALID_ARGUMENT;
}

constexpr int kMaxGemmDevices = 64;

// Clusters of two, launched as a programmatic dependent of what is before it on the stream (attr: room for two).
void cluster_launch_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int grid, size_t smem, cudaStream_t st) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(grid);
  cfg->blockDim = dim3(kGemmThreads);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 2;
}

// The SM-pair kernel: clusters of two CTAs, as many as the device can hold at once (at most one CTA per SM).
// *max_clusters (cached per device and format) is 0 where cluster launches of this kernel are not possible.
template <int MODE>
int pair_cluster_capacity(int dev_id, int *max_clusters) {
  static std::atomic<int> ready[kMaxGemmDevices];
  static int capacity[kMaxGemmDevices];
  if (dev_id < 0 || dev_id >= kMaxGemmDevices) return DTQ_ERR_INVALID_ARGUMENT;
  if (!ready[dev_id].load(std::memory_order_acquire)) {
    static std::mutex mutex;
    std::lock_guard<std::mutex> lock(mutex);
    if (!ready[dev_id].load(std::memory_order_relaxed)) {
      const int smem = static_cast<int>(sizeof(PairSmem<MODE>)) + 1024;
      int n = 0;
      if (cudaFuncSetAttribute(mx_gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        cluster_launch_config(&cfg, attr, 2, smem, nullptr);
        cfg.numAttrs = 1;  // the occupancy query wants the cluster shape only
        if (cudaOccupancyMaxActiveClusters(&n, mx_gemm_pair_kernel<MODE>, &cfg) != cudaSuccess) n = 0;
      }
      (void)cudaGetLastError();  // a device without cluster support is not an error of this call
      capacity[dev_id] = n;
      ready[dev_id].store(1, std::memory_order_release);
    }
  }
  *max_clusters = capacity[dev_id];
  return DTQ_OK;
}

// What every launcher needs: operand pointers, sizes (k_bytes = bytes per operand row), where the status word is.
struct GemmCall {
  RowwiseEpilogue rowwise;  // all zero for the block-scaled modes
  const void *a, *b, *sfa, *sfb;
  void *out;
  int64_t m, n, k_bytes, katoms;
  int *status;
  cudaStream_t st;
};

template <int MODE>
int launch_pair(const GemmCall &c, int max_clusters) {
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  constexpr int kKAtoms = Format<MODE>::kKAtoms;
  if (int e = make_operand_map(&map_a, c.a, c.m, c.k_bytes, kBM)) return e;
  if (int e = make_operand_map(&map_b, c.b, c.n, c.k_bytes, kPairBN / 2)) return e;
  if constexpr (Format<MODE>::kScaled) {
    if (int e = make_scale_map(&map_sfa, c.sfa, ceil_div64(c.m, 128), c.katoms, 1, kKAtoms)) return e;
    if (int e = make_scale_map(&map_sfb, c.sfb, ceil_div64(c.n, 128), c.katoms, 2, kKAtoms)) return e;
  } else {  // never dereferenced by the kernel
    map_sfa = map_a;
    map_sfb = map_a;
  }
  PairParams p;
  p.rowwise = c.rowwise;
  p.out = static_cast<uint16_t *>(c.out);
  p.M = static_cast<int>(c.m);
  p.N = static_cast<int>(c.n);
  p.m_pairs = static_cast<int>(ceil_div64(c.m, 256));
  p.n_tiles = static_cast<int>(ceil_div64(c.n, kPairBN));
  p.k_stages = static_cast<int>(ceil_div64(c.k_bytes, kBK));
  p.status = c.status;
  const int64_t tiles = int64_t(p.m_pairs) * p.n_tiles;
  const int clusters = static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  cluster_launch_config(&cfg, attr, 2 * clusters, sizeof(PairSmem<MODE>) + 1024, c.st);
  return cuda_status(cudaLaunchKernelEx(&cfg, mx_gemm_pair_kernel<MODE>, map_a, map_b, map_sfa, map_sfb, p));
}

// One CTA per tile, tile shape SH.
template <typename SH, int MODE>
int launch_shape(const GemmCall &c, const DeviceInfo &dev) {
  static std::atomic<int> configured[kMaxGemmDevices];
  int dev_id = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev_id));
  if (dev_id < 0 || dev_id >= kMaxGemmDevices) return DTQ_ERR_INVALID_ARGUMENT;
  const int smem = static_cast<int>(sizeof(GemmSmem<SH, MODE>)) + 1024;
  if (!configured[dev_id].load(std::memory_order_acquire)) {  // setting the attribute twice is harmless
    DTQ_CUDA_TRY(cudaFuncSetAttribute(mx_gemm_kernel<SH, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev_id].store(1, std::memory_order_release);
  }
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  if (int e = make_operand_map(&map_a, c.a, c.m, c.k_bytes, kBM)) return e;
  if (int e = make_operand_map(&map_b, c.b, c.n, c.k_bytes, SH::BN)) return e;
  if constexpr (Format<MODE>::kScaled) {
    if (int e = make_scale_map(&map_sfa, c.sfa, ceil_div64(c.m, 128), c.katoms, 1, Format<MODE>::kKAtoms)) return e;
    if (int e = make_scale_map(&map_sfb, c.sfb, ceil_div64(c.n, 128), c.katoms, SH::BN / 128, Format<MODE>::kKAtoms)) return e;
  } else {  // never dereferenced by the kernel
    map_sfa = map_a;
    map_sfb = map_a;
  }
  GemmParams p;
  p.rowwise = c.rowwise;
  p.out = static_cast<uint16_t *>(c.out);
  p.M = static_cast<int>(c.m);
  p.N = static_cast<int>(c.n);
  p.K = static_cast<int>(c.k_bytes);
  p.m_tiles = static_cast<int>(ceil_div64(c.m, kBM));
  p.n_tiles = static_cast<int>(ceil_div64(c.n, SH::BN));
  p.k_stages = static_cast<int>(ceil_div64(c.k_bytes, kBK));
  p.status = c.status;
  const int64_t tiles = int64_t(p.m_tiles) * p.n_tiles;
  const int grid = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
  return cuda_status(launch_after_dependency(mx_gemm_kernel<SH, MODE>, dim3(grid), dim3(kGemmThreads), size_t(smem), c.st, map_a,
                                             map_b, map_sfa, map_sfb, p));
}

template <int MODE>
int launch_gemm(const GemmCall &c, int kernel, const DeviceInfo &dev) {
  // Which kernel: estimated time = a fixed part (launch, set-up, filling the pipeline, the last epilogue) plus
  // rounds of tiles on the busiest SM x stages of 128 operand bytes along K x the time of such a stage, all in
  // microseconds as measured on a B200 (steady state, 1.3 to 1.5 GHz under the power cap): the SM pair's
  // 256 x 256 tile costs 0.36 per stage but 10 to start, a 128 x 256 tile 0.42 and 8, a 128 x 128 tile 0.30 and 6.
  // So large problems run on SM pairs, and problems of a tile or two per SM on the narrow kernel, whose
  // smaller tiles also spread a small output over more SMs.
  const int64_t m_tiles = ceil_div64(c.m, kBM);
  const double stages = static_cast<double>(ceil_div64(c.k_bytes, kBK));
  const double wide = 8.0 + static_cast<double>(ceil_div64(m_tiles * ceil_div64(c.n, 256), dev.sm_count)) * stages * 0.42;
  const double narrow = 6.0 + static_cast<double>(ceil_div64(m_tiles * ceil_div64(c.n, 128), dev.sm_count)) * stages * 0.30;
  int dev_id = 0, max_clusters = 0;
  DTQ_CUDA_TRY(cudaGetDevice(&dev_id));
  if (int e = pair_cluster_capacity<MODE>(dev_id, &max_clusters)) return e;
  const double pair =
      max_clusters > 0
          ? 10.0 + static_cast<double>(ceil_div64(ceil_div64(c.m, 256) * ceil_div64(c.n, 256), max_clusters)) * stages * 0.36
          : 1e30;
  if (kernel == DTQ_GEMM_PAIR && max_clusters <= 0) return DTQ_ERR_CUDA_BASE + static_cast<int>(cudaErrorNotSupported);
  if (kernel == DTQ_GEMM_AUTO)
    kernel = (pair <= wide && pair <= narrow) ? DTQ_GEMM_PAIR : (narrow < wide ? DTQ_GEMM_NARROW : DTQ_GEMM_WIDE);
  if (kernel == DTQ_GEMM_PAIR) return launch_pair<MODE>(c, max_clusters);
  if (kernel == DTQ_GEMM_NARROW) return launch_shape<NarrowShape, MODE>(c, dev);
  return launch_shape<WideShape, MODE>(c, dev);
}

}  // namespace
}  // namespace dtq

extern "C" size_t dtq_mx_gemm_scale_bytes(int64_t rows, int64_t k) {
  if (rows <= 0 || k <= 0) return 0;
  return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>(((k + 31) / 32 + 3) / 4) * 512;
}

extern "C" int dtq_mx_gemm_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                                void *out_bf16, int64_t m, int64_t n, int64_t k, int elem_format, int kernel, void *workspace,
                                size_t workspace_bytes, void *stream) {
  using namespace dtq;
  if (m < 0 || n < 0 || k < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (elem_format != DTQ_E4M3 && elem_format != DTQ_E2M1) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (kernel < DTQ_GEMM_AUTO || kernel > DTQ_GEMM_NARROW) return DTQ_ERR_INVALID_ARGUMENT;
  if (n % 8 != 0 || k % 32 != 0) return DTQ_ERR_SHAPE;  // 16-byte output vectors; whole MX blocks (also the TMA row pitch)
  if (m > 0x7FFFFFFF - 256 || n > 0x7FFFFFFF - 256 || k > 0x7FFFFFFF - 256) return DTQ_ERR_TOO_LARGE;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  if (m == 0 || n == 0) return DTQ_OK;
  if (!out_bf16 || !aligned_to(out_bf16, 16)) return DTQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k == 0) return cuda_status(cudaMemsetAsync(out_bf16, 0, static_cast<size_t>(m) * n * 2, st));
  if (!a || !b || !a_scales_blocked || !b_scales_blocked) return DTQ_ERR_INVALID_ARGUMENT;
  if (!aligned_to(a, 16) || !aligned_to(b, 16) || !aligned_to(a_scales_blocked, 16) || !aligned_to(b_scales_blocked, 16))
    return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  GemmCall c;
  c.rowwise = RowwiseEpilogue{};
  c.a = a;
  c.b = b;
  c.sfa = a_scales_blocked;
  c.sfb = b_scales_blocked;
  c.out = out_bf16;
  c.m = m;
  c.n = n;
  c.k_bytes = elem_format == DTQ_E2M1 ? k / 2 : k;
  c.katoms = ceil_div64(k / 32, 4);
  c.status = &static_cast<Workspace *>(workspace)->status;
  c.st = st;
  return elem_format == DTQ_E2M1 ? launch_gemm<kMxFp4>(c, kernel, dev) : launch_gemm<kMxFp8>(c, kernel, dev);
}

extern "C" int dtq_rowwise_fp8_bf16(const void *a, const void *b, const float *a_row_scale, const float *b_row_scale,
                                    const void *bias, int bias_dtype, void *out_bf16, int64_t m, int64_t n, int64_t k,
                                    int a_format, int kernel, void *workspace, size_t workspace_bytes, void *stream) {
  using namespace dtq;
  if (m < 0 || n < 0 || k < 0) return DTQ_ERR_INVALID_ARGUMENT;
  if (a_format != DTQ_E4M3 && a_format != DTQ_E5M2) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (bias && bias_dtype != DTQ_F32 && bias_dtype != DTQ_BF16) return DTQ_ERR_UNSUPPORTED_DTYPE;
  if (kernel < DTQ_GEMM_AUTO || kernel > DTQ_GEMM_NARROW) return DTQ_ERR_INVALID_ARGUMENT;
  if (n % 8 != 0 || k % 16 != 0) return DTQ_ERR_SHAPE;  // 16-byte output vectors; 16-byte operand row pitch (TMA)
  if (m > 0x7FFFFFFF - 256 || n > 0x7FFFFFFF - 256 || k > 0x7FFFFFFF - 256) return DTQ_ERR_TOO_LARGE;
  if (!workspace || workspace_bytes < sizeof(Workspace) || !aligned_to(workspace, 256)) return DTQ_ERR_WORKSPACE;
  if (m == 0 || n == 0) return DTQ_OK;
  if (!out_bf16 || !aligned_to(out_bf16, 16) || !a_row_scale || !b_row_scale) return DTQ_ERR_INVALID_ARGUMENT;
  if (k > 0 && (!a || !b || !aligned_to(a, 16) || !aligned_to(b, 16))) return DTQ_ERR_INVALID_ARGUMENT;
  DeviceInfo dev;
  if (int e = current_device_info(&dev)) return e;
  GemmCall c;
  c.rowwise.row_scale = a_row_scale;
  c.rowwise.col_scale = b_row_scale;
  c.rowwise.bias = bias;
  c.rowwise.bias_is_bf16 = bias_dtype == DTQ_BF16;
  c.rowwise.operand_format_bits = a_format == DTQ_E5M2 ? (1u << 7) : 0u;
  c.a = a;
  c.b = b;
  c.sfa = nullptr;
  c.sfb = nullptr;
  c.out = out_bf16;
  c.m = m;
  c.n = n;
  c.k_bytes = k;
  c.katoms = 0;
  c.status = &static_cast<Workspace *>(workspace)->status;
  c.st = static_cast<cudaStream_t>(stream);
  return launch_gemm<kRowwise>(c, kernel, dev);
}

extern "C" int dtq_mx_fp8_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                               void *out_bf16, int64_t m, int64_t n, int64_t k, void *workspace, size_t workspace_bytes,
                               void *stream) {
  return dtq_mx_gemm_bf16(a, b, a_scales_blocked, b_scales_blocked, out_bf16, m, n, k, DTQ_E4M3, DTQ_GEMM_AUTO, workspace,
                          workspace_bytes, stream);
}

extern "C" int dtq_mx_fp4_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                               void *out_bf16, int64_t m, int64_t n, int64_t k, void *workspace, size_t workspace_bytes,
                               void *stream) {
  return dtq_mx_gemm_bf16(a, b, a_scales_blocked, b_scales_blocked, out_bf16, m, n, k, DTQ_E2M1, DTQ_GEMM_AUTO, workspace,
                          workspace_bytes, stream);
}
