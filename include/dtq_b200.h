/*
 * dtq_b200 -- C ABI of the B200 (sm_100a) FP8 / MX quantization kernels.
 *
 * This is the boundary a host binding talks to.  It is what the reference's
 * C++ host functions `driss_torch::<op>(at::Tensor...)` do below their tensor
 * checks (validate, pick a launch shape, launch), with torch types replaced by
 * plain device pointers and sizes.  Every pointer is a DEVICE pointer unless a
 * name ends in `_host`.  Nothing here allocates, synchronises the host, or
 * throws: every call enqueues work on `stream` of the CURRENT device and
 * returns a status (0 = ok, see dtq_status_string).  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).
 *
 * Arithmetic is bit-exact with the reference CUDA kernels; the citations give
 * the reference function each entry point replaces (paths inside the
 * drisspg/driss_torch checkout).
 */
#ifndef DTQ_B200_H
#define DTQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define DTQ_BF16 0
#define DTQ_F32 1
#define DTQ_F16 2 /* dtq_mx_quantize only */
#define DTQ_E4M3 0 /* float8_e4m3fn */
#define DTQ_E5M2 1 /* float8_e5m2   */
#define DTQ_E2M1 2 /* float4_e2m1fn, two per byte, lower index in the low nibble; dtq_mx_quantize only */

/* status codes */
#define DTQ_OK 0
#define DTQ_ERR_INVALID_ARGUMENT 1
#define DTQ_ERR_UNSUPPORTED_DTYPE 2
#define DTQ_ERR_SHAPE 3
#define DTQ_ERR_WORKSPACE 4
#define DTQ_ERR_TIMEOUT 5 /* a bounded device-side wait gave up (see dtq_workspace_status) */
#define DTQ_ERR_TOO_LARGE 6
#define DTQ_ERR_CUDA_BASE 1000 /* 1000 + cudaError_t */

const char *dtq_status_string(int status);

/* Library version and the GPU architecture the kernels were built for ("sm_100a"). */
const char *dtq_version(void);

/*
 * Workspace.  amax and the fused ops finish their grid-wide reduction in the
 * same launch through a small scratch area (per-block partials, an arrival
 * counter, a barrier generation word and a status word).  The caller owns it:
 * allocate dtq_workspace_bytes() bytes of device memory (256-byte aligned),
 * call dtq_workspace_init once (a memset on `stream`), then pass it to any
 * number of calls.  Calls that may overlap on the GPU (different streams) need
 * different workspaces.  The kernels leave it ready for the next call.
 */
size_t dtq_workspace_bytes(void);
int dtq_workspace_init(void *workspace, size_t workspace_bytes, void *stream);
/* Copies the sticky device-side status word to the host (synchronises `stream`). */
int dtq_workspace_status(const void *workspace, int *status_host, void *stream);
/*
 * The same without synchronising: enqueues the 4-byte copy on `stream` and returns.  `status_host`
 * should be page-locked; it holds the status as of this point of the stream once the stream has
 * got there (a host that polls it before its next call learns of a timeout one call late, but
 * never blocks).
 */
int dtq_workspace_status_async(const void *workspace, int *status_host, void *stream);

/*
 * out[i] = fp8_satfinite(in[i] * scale), i < numel, over flat storage.
 * bf16 input: scale is rounded to bf16 and the product is a bf16 multiply
 * (one rounding), as in the reference; fp32 input: fp32 multiply.
 * `scale` points to one fp32 on the device (no host read).
 * Replaces driss_torch::saturated_cast / dispatch_best_kernel and its three
 * kernels: src/saturated_cast.cu:38-57, :59-104, :106-153, :168-252.
 */
int dtq_saturated_cast(const void *in, void *out, const float *scale, int64_t numel, int in_dtype,
                       int out_dtype, void *stream);

/*
 * The cast with the output transposed, or in both orientations from one read of a
 * contiguous [rows, cols] input:
 *   out_t [cols, rows] = dtq_saturated_cast(transpose(in))   always written
 *   out   [rows, cols] = dtq_saturated_cast(in)              written unless `out` is NULL
 * Same arithmetic as dtq_saturated_cast, bit for bit.  Any shape; the tiled fast path needs
 * rows % 16 == 0, cols % 8 == 0 (bf16) or % 4 == 0 (fp32), `in` and `out_t` 16-byte and `out`
 * 8-byte aligned.  The reference declares `transpose` on saturated_cast but its wrapper asserts
 * it off (driss_torch/__init__.py:24-38) and the CUDA side only uses the flag to choose a kernel
 * (src/saturated_cast.cu:168-181).
 */
int dtq_saturated_cast_transposed(const void *in, void *out, void *out_t, const float *scale, int64_t rows,
                                  int64_t cols, int in_dtype, int out_dtype, void *stream);

/*
 * dtq_cast_with_amax with the output transposed, or in both orientations from one read of a
 * contiguous [rows, cols] input (the two fp8 operands tensor-wise scaled training needs):
 *   out_t [cols, rows] = dtq_cast_with_amax(transpose(in))   always written
 *   out   [rows, cols] = dtq_cast_with_amax(in)              written unless `out` is NULL
 * Arithmetic of dtq_cast_with_amax / the reference's fused op (src/dynamic_scaled_quant.cu:111-117)
 * bit for bit; `amax` is a device float (dtq_amax's output, an all-reduced value, or the MX cast's
 * by-product), `scale_out` (nullable) receives the fp32 scale.  Shapes and alignment as for
 * dtq_saturated_cast_transposed.  No reference counterpart.
 */
int dtq_cast_with_amax_transposed(const void *in, void *out, void *out_t, const float *amax, float *scale_out,
                                  int64_t rows, int64_t cols, int in_dtype, int out_dtype, void *stream);

/*
 * Tensor-wise dynamic quantisation of a contiguous [rows, cols] input into both orientations:
 *   amax = max |in| (>= 0, NaNs dropped); out = dtq_cast_with_amax(in), out_t = dtq_cast_with_amax(transpose(in)),
 * i.e. dtq_dynamic_scaled_quant's payload for x and for x^T.  Two launches queued by this one call: the
 * amax kernel and, started under its tail (programmatic dependent launch), the kernel that converts
 * every element once and writes it in both orientations.  amax_out / scale_out: one fp32 each,
 * nullable.  `out` and `out_t` are both required.  Needs an initialised workspace.  No reference
 * counterpart (the reference's fused op, src/dynamic_scaled_quant.cu:83-176, has one orientation).
 */
int dtq_dynamic_scaled_quant_dual(const void *in, void *out, void *out_t, float *amax_out, float *scale_out,
                                  int64_t rows, int64_t cols, int in_dtype, int out_dtype, void *workspace,
                                  size_t workspace_bytes, void *stream);

/*
 * out[0] = max_i |in[i]| as fp32 (-inf for numel == 0; NaNs are dropped), one
 * launch, no pre-initialised output.
 * Replaces driss_torch::amax and amax_kernel: src/amax.cu:50-80, :82-119.
 */
int dtq_amax(const void *in, float *out, int64_t numel, int in_dtype, void *workspace,
             size_t workspace_bytes, void *stream);

/*
 * dtq_amax for callers that cannot allocate device memory -- a host whose own pool owns the
 * device heap and forbids cudaMalloc in plugins, or a latency-critical section that cannot
 * take the device-wide synchronisation of cudaMalloc / cudaFree.  Same result as dtq_amax,
 * but the reduction's scratch is a fixed array inside the library image (about 16.5 KB of
 * device memory on every GPU that loads the library, until the process exits), so there is
 * no workspace argument and the call allocates nothing.  Limits and rules:
 *   - inputs of at most DTQ_AMAX_STATIC_MAX_BYTES bytes (one partial slot of the array per
 *     64 KiB tile); larger inputs are rejected with DTQ_ERR_TOO_LARGE, nothing is launched;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins;
 *   - every call on a device uses the same array: calls that may overlap on the GPU
 *     (different streams, several host threads) race -- serialise them on one stream;
 *   - the arrival counter in the array is cleared on `stream` before each launch;
 *   - the looked-up address is cached per device for the life of the process: it belongs to the
 *     device's primary context, so do not call this entry point again after cudaDeviceReset.
 * No counterpart in the reference (its amax allocates its output and relies on a fill launch).
 */
#define DTQ_AMAX_STATIC_MAX_BYTES (268435456LL) /* 256 MiB: 4096 tiles x 64 KiB */
int dtq_amax_static_scratch(const void *in, float *out, int64_t numel, int in_dtype, void *stream);

/*
 * Fused tensor-wise dynamic quantisation in ONE launch (inputs above 320 MiB, where nothing
 * can stay on chip between the two looks at the data, are issued as an amax launch followed
 * by a cast launch on the same stream instead):
 *   amax = max |in| (>= 0);  scale_d = fp8_max / ((double)amax + 1e-12);
 *   out[i] = fp8_satfinite((float)(scale_d * (double)in[i])).
 * amax_out / scale_out (one fp32 each, nullable) receive amax and
 * (float)scale_d.  bf16 and fp32 inputs.
 * Replaces driss_torch::dynamic_scaled_quant and its cooperative kernel:
 * src/dynamic_scaled_quant.cu:83-118, :119-176.
 */
int dtq_dynamic_scaled_quant(const void *in, void *out, float *amax_out, float *scale_out,
                             int64_t numel, int in_dtype, int out_dtype, void *workspace,
                             size_t workspace_bytes, void *stream);

/*
 * dtq_dynamic_scaled_quant for a tensor that is row-sharded over the GPUs of one node, one
 * process per GPU, every rank making this same call on its shard: ONE launch per GPU whose
 * grid barrier also exchanges the per-GPU maxima through peer-addressable memory (plain
 * st.release.sys / ld.acquire.sys over NVLink; no collective library call, no second launch),
 * so every rank quantises with the global amax.  Output is bit-identical to the single-GPU
 * result on the concatenated tensor.
 *   peer_exchange[r] = rank r's exchange buffer (dtq_p2p_exchange_bytes() bytes, zero-filled
 *                      once, 8-byte aligned) as addressable from THIS device, r < world <= 16;
 *   epoch            = 1, 2, 3, ... : the same value on every rank for the same call;
 *   spin_limit       = polls before the wait for the peers gives up (0 = default, about 1 s);
 *                      a rank that never arrives makes the others return with
 *                      DTQ_ERR_TIMEOUT in the workspace status word instead of hanging: no
 *                      payload is written, amax_out / scale_out receive NaN
 *                      (re-initialise the workspace afterwards).
 * `in` must be 16-byte and `out` 8-byte (bf16) / 4-byte (fp32) aligned.  No reference counterpart
 * (the reference has no multi-GPU path); arithmetic as dtq_dynamic_scaled_quant.
 */
size_t dtq_p2p_exchange_bytes(void);
int dtq_dynamic_scaled_quant_p2p(const void *in, void *out, float *amax_out, float *scale_out,
                                 int64_t numel, int in_dtype, int out_dtype, void *workspace,
                                 size_t workspace_bytes, void *const *peer_exchange, int rank, int world,
                                 uint32_t epoch, uint32_t spin_limit, void *stream);

/*
 * Cast phase alone, for an amax that already exists on the device (a sharded
 * tensor after its max all-reduce): same arithmetic as the second half of
 * dtq_dynamic_scaled_quant (src/dynamic_scaled_quant.cu:111-117).
 * `amax` points to one fp32 on the device; scale_out is nullable.
 */
int dtq_cast_with_amax(const void *in, void *out, const float *amax, float *scale_out,
                       int64_t numel, int in_dtype, int out_dtype, void *stream);

/*
 * Row-wise dynamic quantisation of a contiguous [rows, cols] matrix: the
 * arithmetic of dtq_dynamic_scaled_quant applied to each row with that row's
 * amax.  amax_out / scale_out hold `rows` fp32 each (nullable).  Single pass:
 * a row is read from HBM once.  No counterpart op in the reference; the
 * arithmetic is src/dynamic_scaled_quant.cu:111-117 per row, the scales are
 * what its row-wise GEMM consumes (src/sweep_mm.cu:28-40).
 */
int dtq_dynamic_scaled_quant_rowwise(const void *in, void *out, float *amax_out, float *scale_out,
                                     int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                                     void *stream);

/*
 * MX block cast of a contiguous bf16 [rows, cols] matrix, cols % 32 == 0:
 * per 32 consecutive elements one E8M0 scale byte (row-major [rows, cols/32])
 * and 32 e4m3 payload bytes.
 * Replaces driss_torch::mx_fp8_quantize and mx_fp8_quantize_kernel:
 * src/mx_cast.cu:44-86, :96-161, :168-246.  Unlike the reference, rows need
 * not be a multiple of 128.
 */
int dtq_mx_fp8_quantize(const void *in_bf16, void *payload, void *scales_e8m0, int64_t rows,
                        int64_t cols, void *stream);

/*
 * dtq_mx_fp8_quantize that also returns the tensor's amax from the same read, for steps that
 * quantise one tensor both tensor-wise and MX: this call, then dtq_cast_with_amax, reads the
 * input twice instead of three times (amax, cast, MX cast).  payload / scales: exactly
 * dtq_mx_fp8_quantize's.  amax_out[0]: the largest non-NaN |x| as fp32, 0 if there is none -- the
 * running maximum of the reference's fused op (src/dynamic_scaled_quant.cu:83-110), i.e.
 * dtq_amax's result clamped at 0.  Needs an initialised workspace (as dtq_amax); `in` 16-byte
 * and `payload` 8-byte aligned.  No reference counterpart.
 */
int dtq_mx_fp8_quantize_amax(const void *in_bf16, void *payload, void *scales_e8m0, float *amax_out, int64_t rows,
                             int64_t cols, void *workspace, size_t workspace_bytes, void *stream);

/*
 * The same for a tensor that is row-sharded over the GPUs of one node (one process per GPU, every
 * rank making this call on its shard, empty shards included): the one-warp launch that finishes the
 * reduction on each GPU also exchanges the local maximum with all peers through peer-addressable
 * memory, so amax_out[0] is the maximum over the whole tensor on every rank and the cast can be
 * enqueued right behind it: no collective call.  peer_exchange, rank, world,
 * epoch, spin_limit: as for dtq_dynamic_scaled_quant_p2p (the two calls may share the exchange
 * buffers and the epoch sequence).  A peer that never arrives: DTQ_ERR_TIMEOUT in the workspace
 * status word, amax_out[0] = NaN (dtq_cast_with_amax passes a NaN amax on to its scale_out).
 */
int dtq_mx_fp8_quantize_amax_p2p(const void *in_bf16, void *payload, void *scales_e8m0, float *amax_out,
                                 int64_t rows, int64_t cols, void *workspace, size_t workspace_bytes,
                                 void *const *peer_exchange, int rank, int world, uint32_t epoch,
                                 uint32_t spin_limit, void *stream);

/*
 * MX block-32 quantisation for every input type and element format the reference's schema names:
 * in_dtype DTQ_BF16 / DTQ_F16 / DTQ_F32, elem_format DTQ_E4M3 / DTQ_E5M2 / DTQ_E2M1.
 * The reference accepts fp8_type = e5m2 and fp16 / fp32 inputs but computes bf16 -> e4m3 on the
 * bytes it was given (src/mx_cast.cu:148,175-184,204), and has no producer for the MXFP4 operands
 * of mx_fp4_bf16 (src/mx_fp8_bf16.cu:243-271).  Scale rule: the reference's (src/mx_cast.cu:44-86)
 * with its constant 8 replaced by the format's largest exponent (8 / 15 / 2):
 * biased = clamp(max_i ceil(log2|x_i|) - EMAX + 127, 0, 255), payload = cvt_satfinite(x * 2^(127-biased)),
 * scale byte = biased; blocks that are all zero or tiny give scale byte 0 and NaN (fp8) or +6 (e2m1)
 * payloads, as in the reference.  For DTQ_BF16 / DTQ_E4M3 the result equals dtq_mx_fp8_quantize's.
 * payload: rows*cols bytes (fp8) or rows*cols/2 bytes (e2m1); scales: rows*cols/32 bytes, row-major.
 * cols % 32 == 0; `in` 16-byte aligned, `payload` aligned to 8 bytes.
 */
int dtq_mx_quantize(const void *in, void *payload, void *scales_e8m0, int64_t rows, int64_t cols, int in_dtype,
                    int elem_format, void *stream);
/*
 * The same with the scales in the blocked layout of dtq_mx_fp8_quantize_blocked (dtq_mx_blocked_scale_bytes(rows,
 * cols) bytes; bytes of padding rows / blocks are not written: zero the buffer first if the shape is not a
 * multiple of (128, 128)): the operands of dtq_mx_fp4_bf16 straight from the cast.
 */
int dtq_mx_quantize_blocked(const void *in, void *payload, void *scales_blocked, int64_t rows, int64_t cols, int in_dtype,
                            int elem_format, void *stream);

/*
 * Both orientations from one read of a contiguous bf16 [rows, cols] matrix (rows % 32 == 0,
 * cols % 32 == 0):
 *   payload   [rows, cols], scales   [rows * cols/32]  = dtq_mx_fp8_quantize(x)
 *   payload_t [cols, rows], scales_t [cols * rows/32]  = dtq_mx_fp8_quantize(transpose(x))
 * byte for byte.  The reference declares `axis` and `transpose` on its op but ignores them
 * (src/mx_cast.cu:168-171); getting the second operand there takes a transpose and a second
 * cast.  `in` 16-byte, `payload` 8-byte, `payload_t` 16-byte aligned.
 * `payload` may be NULL (`scales_e8m0` is then ignored): only the transposed pair is written, which
 * is what the schema's own `transpose` / `axis = 0` arguments ask for.
 */
int dtq_mx_fp8_quantize_dual(const void *in_bf16, void *payload, void *scales_e8m0, void *payload_t,
                             void *scales_t_e8m0, int64_t rows, int64_t cols, void *stream);

/*
 * The same with both scale arrays in the blocked layout of dtq_mx_fp8_quantize_blocked: `scales`
 * for the [rows, cols/32] grid (dtq_mx_blocked_scale_bytes(rows, cols) bytes), `scales_t` for the
 * [cols, rows/32] grid (dtq_mx_blocked_scale_bytes(cols, rows) bytes); padding bytes are not
 * written (zero-fill the arrays when rows or cols is not a multiple of 128).  Both operands of the
 * reference's mx_fp8_bf16 (src/mx_fp8_bf16.cu:197-205) for x and for x^T from one read, with no
 * transpose, second cast or to_blocked pass.
 */
int dtq_mx_fp8_quantize_dual_blocked(const void *in_bf16, void *payload, void *scales_e8m0, void *payload_t,
                                     void *scales_t_e8m0, int64_t rows, int64_t cols, void *stream);

/*
 * dtq_mx_fp8_quantize through shared memory: same outputs, but the input is staged by the bulk
 * asynchronous copy engine (TMA, cp.async.bulk + mbarrier ring) for a persistent grid of
 * producer/consumer CTAs instead of being loaded straight into registers.  Kept as a measured
 * alternative (the register path is the default because it is faster on B200 at every size
 * measured).  Needs 16-byte aligned input, 8-byte aligned payload, and `status_dev`, one int in
 * device memory (zero it once): a bounded wait that gives up stores DTQ_ERR_TIMEOUT there.
 * Replaces the same reference code as dtq_mx_fp8_quantize (src/mx_cast.cu:96-161), whose kernel
 * also stages its tile in shared memory.
 */
int dtq_mx_fp8_quantize_tma(const void *in_bf16, void *payload, void *scales_e8m0, int64_t rows,
                            int64_t cols, int *status_dev, void *stream);

/*
 * As dtq_mx_fp8_quantize, but the scales are written directly in the blocked layout that the
 * reference's MX GEMM (mx_fp8_bf16, src/mx_fp8_bf16.cu:97-110,197-205) hands to CUTLASS
 * (Sm1xxBlockScaledConfig::tile_atom_to_shape_SFA): 128-row x 4-block atoms of 512 bytes,
 * k-major atom order; row r, block c of an atom at (r % 32) * 16 + (r / 32) * 4 + c.  The
 * reference reaches that layout with a separate re-layout pass over the row-major scales
 * (`to_blocked`, test/test_mx.py:28-32); emitting it here saves that pass.
 * `scales_blocked` holds dtq_mx_blocked_scale_bytes(rows, cols) bytes; bytes that belong to
 * padding rows / blocks (rows % 128, (cols/32) % 4) are not written: zero the buffer first if
 * the shape is not a multiple of (128, 128).
 */
size_t dtq_mx_blocked_scale_bytes(int64_t rows, int64_t cols);
int dtq_mx_fp8_quantize_blocked(const void *in_bf16, void *payload, void *scales_blocked, int64_t rows,
                                int64_t cols, void *stream);

/*
 * MX block-scaled GEMM, the consumer of the MX casts above:
 *   out[m, n] = bf16( sum_k a[m, k] * 2^(sa[m, k/32] - 127) * b[n, k] * 2^(sb[n, k/32] - 127) ),  fp32 accumulation
 *   a  [m, k] e4m3 bytes, row-major;
 *   b  [n, k] e4m3 bytes, row-major -- the memory of the reference's column-major [k, n] operand;
 *   a_scales_blocked / b_scales_blocked: E8M0 bytes in the blocked layout of dtq_mx_fp8_quantize_blocked,
 *       dtq_mx_gemm_scale_bytes(m, k) and dtq_mx_gemm_scale_bytes(n, k) bytes (bytes that belong to padding
 *       rows or k-blocks must not be 0xFF; the quantisers here write zeros there);
 *   out [m, n] bf16, row-major, 16-byte aligned.
 * n % 8 == 0 and k % 32 == 0; m, n, k need not be multiples of the 128 x 256 x 128 tile (out-of-range
 * rows and columns are loaded as zeros and not stored).  a, b and the scale arrays 16-byte aligned.
 * tcgen05 tensor-core kernel with the accumulator in tensor memory, operands staged by TMA; it occupies
 * each SM exclusively while it runs.  Needs an initialised workspace: a bounded device-side wait that
 * gives up leaves DTQ_ERR_TIMEOUT in its status word (dtq_workspace_status).
 * Replaces driss_torch::mx_fp8_bf16: src/mx_fp8_bf16.cu:42-163 (run_gemm), :168-215 (validate), :217-241.
 */
size_t dtq_mx_gemm_scale_bytes(int64_t rows, int64_t k);
int dtq_mx_fp8_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                    void *out_bf16, int64_t m, int64_t n, int64_t k, void *workspace, size_t workspace_bytes,
                    void *stream);
/*
 * The MXFP4 GEMM: as dtq_mx_fp8_bf16 with e2m1 operands packed two per byte (lower index in the low nibble,
 * what dtq_mx_quantize writes for DTQ_E2M1): a [m, k/2] bytes, b [n, k/2] bytes; k counts elements, k % 32 == 0.
 * tcgen05.mma kind::mxf4 with one scale per 32 elements.
 * Replaces driss_torch::mx_fp4_bf16: src/mx_fp8_bf16.cu:243-271.
 */
int dtq_mx_fp4_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                    void *out_bf16, int64_t m, int64_t n, int64_t k, void *workspace, size_t workspace_bytes,
                    void *stream);

/*
 * Both GEMMs with the element format (DTQ_E4M3 or DTQ_E2M1) and the kernel named instead of chosen from the
 * problem size (for benchmarks, and for tests that run every kernel on every size; the results of the kernels are
 * bit-identical):
 *   DTQ_GEMM_PAIR    two CTAs of a cluster (an SM pair) per 256 x 256 tile, tcgen05.mma.cta_group::2: least
 *                    operand traffic per SM, what large problems use;
 *   DTQ_GEMM_WIDE    one CTA per 128 x 256 tile;
 *   DTQ_GEMM_NARROW  one CTA per 128 x 128 tile, two accumulators (epilogue under the next tile's MMAs).
 * No reference counterpart (the reference fixes one CUTLASS tile shape, src/mx_fp8_bf16.cu:231-233).
 */
#define DTQ_GEMM_AUTO 0
#define DTQ_GEMM_PAIR 1
#define DTQ_GEMM_WIDE 2
#define DTQ_GEMM_NARROW 3
int dtq_mx_gemm_bf16(const void *a, const void *b, const void *a_scales_blocked, const void *b_scales_blocked,
                     void *out_bf16, int64_t m, int64_t n, int64_t k, int elem_format, int kernel, void *workspace,
                     size_t workspace_bytes, void *stream);

/*
 * Row-wise scaled fp8 GEMM, the consumer of dtq_dynamic_scaled_quant_rowwise's scales:
 *   out[m, n] = bf16( fp32( fp32(acc[m, n] * a_row_scale[m]) * b_row_scale[n] ) + bias[n] ),
 *   acc[m, n] = sum_k a[m, k] * b[n, k] in fp32 on the tensor cores (tcgen05.mma kind::f8f6f4, no block scales);
 *   a [m, k] e4m3 or e5m2 bytes (a_format), row-major; b [n, k] e4m3 bytes, row-major -- the memory of the
 *   reference's column-major [k, n] operand; a_row_scale [m], b_row_scale [n] fp32 (the DEQUANTISATION scales:
 *   reciprocals of the quantisation scales); bias [n] fp32 or bf16 (bias_dtype DTQ_F32 / DTQ_BF16) or NULL;
 *   n % 8 == 0, k % 16 == 0; `kernel` as for dtq_mx_gemm_bf16.
 * Replaces driss_torch::sweep_mm (src/sweep_mm.cu:11-88) and its CUTLASS Sm90 kernels
 * (src/scaled_mm_kernels/f8f8bf16_rowwise_kernel.h:101-280, epilogue :151-175), which exist for Hopper only; their
 * tuning arguments (fast accumulation, cluster shape, transposition, swizzle) have no counterpart here.
 */
int dtq_rowwise_fp8_bf16(const void *a, const void *b, const float *a_row_scale, const float *b_row_scale, const void *bias,
                         int bias_dtype, void *out_bf16, int64_t m, int64_t n, int64_t k, int a_format, int kernel,
                         void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DTQ_B200_H */
