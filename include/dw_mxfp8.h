/*
 * dw_mxfp8.h — C ABI of the B200 (sm_100a) MXFP8 linear path.
 *
 * MX quantisation of bf16 matrices (E4M3 payload, one E8M0 power-of-two scale per
 * 32 elements, row-wise or column-wise) and the block-scaled tcgen05 GEMM that
 * consumes those operands.  Plain pointers and sizes only; every pointer is a
 * DEVICE pointer unless stated; `stream` is a cudaStream_t passed as void*.
 * All calls are asynchronous on `stream`, allocate nothing, and borrow the caller's
 * buffers.  State is kept per device (one process may drive several GPUs; the device that is
 * current at the call is the one used) and every launching call returns DW_ERR_ARCH on a
 * device that is not compute capability 10.x.  Return value: DW_OK or a negative DW_ERR_* code (the convention of the
 * reference's only C ABI, dw_fmha_bf16_forward, csrc/fmha_bridge_min/fmha_bridge_min.cu:39-46).
 *
 * Stream order is kept: every kernel launched here behaves as if it started after the work before it on `stream`
 * had finished.  (The GEMM and the quantisers are launched with programmatic stream serialisation: their thread blocks
 * may become resident while the preceding kernel is finishing, but they wait for that kernel to complete before they
 * read or write any memory.  The one exception is asked for explicitly: DW_QUANT_OVERLAP_PREVIOUS.)
 *
 * Each entry point names the reference interface it replaces (path:line inside the
 * reference project).
 */
#ifndef DW_MXFP8_H_
#define DW_MXFP8_H_

#include <stddef.h>
#include <stdint.h>

/* symbol visibility: the library is built with -fvisibility=hidden */
#if defined(DW_BUILDING_LIB) && defined(__GNUC__)
#define DW_API __attribute__((visibility("default")))
#else
#define DW_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define DW_OK                 0
#define DW_ERR_BAD_ARG       (-1)  /* null pointer, bad shape, misaligned pointer, bad enum */
#define DW_ERR_ARCH          (-2)  /* current device is not compute capability 10.x */
#define DW_ERR_LAUNCH        (-3)  /* CUDA runtime / driver error at launch or descriptor encode */
#define DW_ERR_DEVICE_STATUS (-4)  /* a kernel recorded a non-zero status word (bounded wait expired) */
#define DW_ERR_TOO_LARGE     (-5)  /* problem exceeds a fixed capacity of the entry point */

/* direction of the 32-element scaling blocks for a row-major [rows, cols] input */
#define DW_DIR_ROW    0  /* blocks along cols; codes [rows, cols]; scales for [rows, cols/32]           */
#define DW_DIR_COL_T  1  /* blocks along rows; codes TRANSPOSED [cols, rows]; scales for [cols, rows/32] */
#define DW_DIR_COL    2  /* blocks along rows; codes in the input's layout [rows, cols]; scales as COL_T */

#define DW_RULE_OCP_FLOOR 0  /* scale = 2^(floor(log2 amax) - 8)                                     */
#define DW_RULE_REF_CEIL  1  /* scale = 2^ceil(log2(amax/448)), csrc/mxfp8_quantization.cu:109-114, bit for bit
                                as the reference's kernel gives it when built with its own flags (--use_fast_math)
                                for sm_100a: amax below 448 * 2^-126 -> scale 1; amax = 1.75 * 2^k <= 224 -> one
                                step higher than the formula                                              */

#define DW_SF_FLAT   0  /* scales[r * ceil(K/32) + kb], one byte each                                 */
#define DW_SF_TILED  1  /* 512-byte tiles of 128 rows x 4 k-blocks, the tcgen05 scale-factor layout:
                           tile (r/128, kb/4) at ((r/128)*ceil(KB/4) + kb/4)*512, inside it
                           (r%32)*16 + ((r/32)%4)*4 + kb%4.  Padding bytes are written as 127.       */

/* Library / device probes. */
int         dw_mxfp8_abi_version(void);
int         dw_mxfp8_device_supported(int device);      /* 1 if compute capability 10.x */
const char *dw_mxfp8_error_string(int code);

/* Pitched device-to-device copy on `stream`: row r (r < height) of width_bytes bytes from src + r * src_pitch to
 * dst + r * dst_pitch.  Either side may be another GPU's memory mapped into this process (symmetric memory): the copy is
 * executed by a copy engine, so it proceeds while kernels occupy every SM.  Used to place a rank's column shard
 * Y[:, n0:n1] (contiguous [M, n_local] as the GEMM writes it) into columns [n0, n1) of the row-major [M, N] result on every
 * rank.  The reference has no multi-GPU code (src/deepwell/__init__.py:45-83 is a placeholder). */
int dw_mxfp8_copy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t height,
                     void *stream);

/* Bytes of the scale buffer for an operand with `rows` rows and `k` elements along its
 * scaled dimension.  Replaces get_mxfp8_scale_layout_info, csrc/mxfp8_quantization.cu:287-298. */
size_t dw_mxfp8_scale_bytes(int64_t rows, int64_t k, int scale_layout);

/* MX quantisation of a row-major bf16 [rows, cols] matrix.
 * Replaces quantize_to_mxfp8_bf16 (csrc/mxfp8_quantization.cu:229-246; row_major=true is
 * DW_DIR_ROW, row_major=false is DW_DIR_COL) and gives transpose_quantize_to_mxfp8_kernel
 * (:216-226, an empty body in the reference) its function as DW_DIR_COL_T.
 * codes: uint8 E4M3 (fn); scales: uint8 E8M0.  x and codes 16-byte aligned. */
int dw_mxfp8_quantize(const void *x_bf16, void *codes, void *scales, int64_t rows, int64_t cols,
                      int direction, int scale_rule, int scale_layout, void *stream);

/* dw_mxfp8_quantize with launch flags.  DW_QUANT_OVERLAP_PREVIOUS: the launch need not wait for the kernel issued just
 * before it on the same stream to finish (programmatic dependent launch): it starts as soon as that kernel lets its
 * dependents go, which dw_mxfp8_gemm's kernel does once all its thread blocks are resident.  The pattern it serves:
 *     dw_mxfp8_gemm(layer i)  ->  dw_mxfp8_quantize_ex(operands of layer i + 1, DW_QUANT_OVERLAP_PREVIOUS)  ->  dw_mxfp8_gemm(layer i + 1)
 * on one stream.  The GEMM, issued first, takes the SMs it needs (it uses the smallest number that keeps its number
 * of rounds of tiles); the quantiser's short-lived thread blocks run on the SMs that leaves free, and on all of them
 * once the GEMM's blocks retire.  (Launched the other way round, or on a second stream, the quantiser fills every SM
 * first and the GEMM waits for it: nothing is scheduled beside a GEMM thread block on its own SM.)  Only for x, codes
 * and scales that the preceding kernel neither reads nor writes; the next ordinary launch on the stream still waits
 * for both kernels.  The flag takes effect on the large-input row-wise path and is ignored elsewhere.
 * The reference has one launch shape and no overlap (csrc/mxfp8_quantization.cu:232-240). */
#define DW_QUANT_OVERLAP_PREVIOUS 1
int dw_mxfp8_quantize_ex(const void *x_bf16, void *codes, void *scales, int64_t rows, int64_t cols,
                         int direction, int scale_rule, int scale_layout, int flags, void *stream);

/* Up to DW_QUANT_BATCH_MAX row-wise quantisations in ONE launch: matrix i is x_bf16[i] [rows[i], cols[i]] -> codes[i], scales[i],
 * all with the same scale rule and scale layout.  For steps made of several small operands (on N GPUs a rank quantises its
 * 1/N row slices of the activations and its 1/N weight shards), where every separate launch pays its own ramp and tail.
 * Each matrix needs cols % 32 == 0 and 16-byte aligned x and codes; with DW_SF_TILED also rows % 128 == 0 and
 * cols % 128 == 0 (whole scale tiles: this entry point writes no padding bytes); anything else is DW_ERR_BAD_ARG and the
 * caller uses dw_mxfp8_quantize per matrix.  Empty matrices are skipped.  `flags` as for dw_mxfp8_quantize_ex.  Results are
 * byte-identical to dw_mxfp8_quantize on each matrix.  The pointer arrays are host arrays read during the call.
 * No counterpart in the reference (quantize_to_mxfp8_bf16, csrc/mxfp8_quantization.cu:232-240, takes one tensor). */
#define DW_QUANT_BATCH_MAX 8
int dw_mxfp8_quantize_rows_batch(int count, const void *const *x_bf16, void *const *codes, void *const *scales,
                                 const int64_t *rows, const int64_t *cols, int scale_rule, int scale_layout, int flags,
                                 void *stream);

/* Tuning switch of the column-wise (transposed-payload) kernel, process-wide.  Bits [0,2): 0 or 2 = the transposed payload is
 * written through a shared-memory staging buffer, whole 128-byte row segments per store (the default); 1 = straight from
 * registers, 32 bytes per thread and output row (as fast or slightly faster on some GPUs while the output rows are less than
 * 1 MiB apart, half the rate beyond).  Bit 2 set: the fused both-forms kernel always runs its row and column pass one after
 * the other in 256 threads instead of side by side in two groups of 256 on large inputs; bit 3 set: always side by side;
 * bit 4 set: the column-wise kernel always with two tile buffers per thread block (three are used up to 2^28 elements).
 * Same bytes in every setting.  For
 * measurements; the reference has no column-wise kernel (csrc/mxfp8_quantization.cu:216-226 is empty). */
int dw_mxfp8_quantize_set_tuning(int word);

/* One read of x, both operand forms: row-wise (codes_row [rows, cols]) and column-wise
 * transposed (codes_col_t [cols, rows]).  Either output pair may be NULL.
 * Counterpart of MicroscaleManager::transpose_mxfp8 (csrc/cutlass_kernels.cpp:412-424, empty). */
int dw_mxfp8_quantize_both(const void *x_bf16, void *codes_row, void *scales_row, void *codes_col_t,
                           void *scales_col, int64_t rows, int64_t cols, int scale_rule,
                           int scale_layout, void *stream);

/* dw_mxfp8_quantize_both plus the sum of every column of x, from the same read: for an output
 * gradient dY [tokens, out_features] the column sums are the bias gradient, which otherwise costs
 * one more pass over dY.  colsum_out: [cols], fp32 (colsum_is_bf16 == 0) or bf16 (== 1, rounded once
 * from the fp32 sum).  The sums are accumulated in fp32 in a fixed order, so repeated calls give
 * identical bits.
 * workspace: dw_mxfp8_colsum_workspace(rows, cols) bytes, 4-byte aligned.
 * Needs rows % 32 == 0, cols % 32 == 0 and 16-byte aligned x, payload and (tiled) scale pointers
 * (DW_ERR_BAD_ARG otherwise); all four outputs are required.
 * The reference's linear replacement has a forward only (OptimizedLinear,
 * src/deepwell/kernels/production_kernels.py:145-194); this is the backward companion of
 * dw_mxfp8_quantize_both. */
size_t dw_mxfp8_colsum_workspace(int64_t rows, int64_t cols);
int dw_mxfp8_quantize_both_colsum(const void *x_bf16, void *codes_row, void *scales_row,
                                  void *codes_col_t, void *scales_col, int64_t rows, int64_t cols,
                                  int scale_rule, int scale_layout, void *colsum_out,
                                  int colsum_is_bf16, void *workspace, size_t workspace_bytes,
                                  void *stream);

/* codes [rows, cols] (row-wise blocks) + scales -> bf16 [rows, cols].
 * Replaces dequantize_from_mxfp8_bf16, csrc/mxfp8_quantization.cu:267-284. */
int dw_mxfp8_dequantize(const void *codes, const void *scales, void *out_bf16, int64_t rows,
                        int64_t cols, int scale_layout, void *stream);

/* Rolling history of a tensor's absolute maximum: amax_history[i] <- amax_history[i - 1] for i = len-1 .. 1,
 * amax_history[0] <- max |x| over num_elements bf16 values (NaN ignored; 0 for an empty tensor).  amax_history is a
 * device array of history_len floats.  Gives a body to MicroscaleManager::update_amax_history
 * (csrc/cutlass_kernels.cpp:426-434, empty in the reference).  MX block scaling itself needs no history; the call
 * serves per-tensor scaling policies (src/deepwell/precision/policy.py:50, amax_history_len). */
int dw_mxfp8_update_amax_history(const void *x_bf16, float *amax_history, int history_len,
                                 int64_t num_elements, void *stream);

/* D[M,N] = bf16(alpha * A[M,K] . B[N,K]^T + beta * D + bias[N]).
 * A and B are E4M3 codes, both K-major (contraction dim contiguous), with DW_SF_TILED scales;
 * bias (bf16 [N]) may be NULL; with beta == 0 the previous content of D is not read.
 * Replaces launch_blackwell_mxfp8_gemm (csrc/blackwell_gemm_kernel.cu:103-156) and the MXFP8
 * branch of BlackwellGemmKernel::gemm (csrc/cutlass_kernels.cpp:173-204), which allocated and
 * freed two scale buffers per call and ran a bf16 cuBLAS GEMM.
 * K % 32 == 0; a_codes, b_codes, d 16-byte aligned.
 * workspace: dw_mxfp8_gemm_workspace(M, N, K) bytes, 16-byte aligned.  It is non-zero when the
 * output has too few tiles to fill the GPU and K is long (weight-gradient shapes): the GEMM then
 * splits K, leaves fp32 partial sums in the workspace and reduces them in a second kernel.  With
 * NULL or too small a workspace the GEMM runs unsplit (same result within rounding).
 * status_word: optional device int32, set non-zero by the kernel if a bounded wait expires
 * (then read it with dw_mxfp8_check_status). */
int dw_mxfp8_gemm(const void *a_codes, const void *a_sf, const void *b_codes, const void *b_sf,
                  void *d_bf16, const void *bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                  float beta, void *workspace, size_t workspace_bytes, void *status_word, void *stream);

/* GEMM with a fused epilogue: D = act(alpha * A.B^T + beta * D + bias), act applied in fp32 before the
 * bf16 rounding, and - when out_codes / out_scales are given - the bf16 result quantised row-wise
 * (32-element blocks along N, DW_SF_TILED scales for an [M, N/32] operand) in the same pass, so the
 * next layer's GEMM can consume it without the activation travelling through HBM in bf16 and back.
 * The codes are exactly what dw_mxfp8_quantize(DW_DIR_ROW) gives on the bf16 D of the same call.
 * d_bf16 may be NULL when only the quantised form is wanted (beta must be 0 then).  N % 32 == 0 for
 * the quantised output.  Gives a body to EpilogueConfig::Op::{BiasReLU, BiasGELU, BiasSwish}
 * (csrc/cutlass_kernels.h:65-77; accepted and ignored at csrc/cutlass_kernels.cpp:223-226) and to
 * FusedLinearGELU (src/deepwell/kernels/blackwell_production.py:487-527). */
#define DW_ACT_NONE 0
#define DW_ACT_RELU 1
#define DW_ACT_GELU 2   /* exact: 0.5 x (1 + erf(x / sqrt 2)) */
#define DW_ACT_SILU 3
/* DW_ACT_SWIGLU: the gated unit of a Llama-style MLP in the epilogue of the fused gate+up projection.  B holds the
 * gate and the up weight with their rows interleaved in groups of 32: rows [64 j, 64 j + 32) are gate rows
 * [32 j, 32 j + 32), rows [64 j + 32, 64 j + 64) are the up rows of the same outputs (bias, if any, interleaved the
 * same way).  N is the fused width (a multiple of 64); the outputs have N / 2 columns:
 *     h[m, f] = silu(alpha * gate[m, f] + bias_g[f]) * (alpha * up[m, f] + bias_u[f])      (fp32, rounded to bf16 once)
 * d_bf16 is [M, N/2] (may be NULL), out_codes [M, N/2] and out_scales the DW_SF_TILED scales of an [M, (N/2)/32]
 * operand: exactly dw_mxfp8_quantize(DW_DIR_ROW) of h, i.e. the down projection's A operand.  The 2 x [M, N/2] bf16
 * gate and up activations never exist in memory.  beta must be 0.  Body of EpilogueConfig::Op::BiasSwish
 * (csrc/cutlass_kernels.h:65-77) in the gated form the Llama shapes of the target need. */
#define DW_ACT_SWIGLU 4
int dw_mxfp8_gemm_fused(const void *a_codes, const void *a_sf, const void *b_codes, const void *b_sf,
                        void *d_bf16, const void *bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                        float beta, int activation, void *out_codes, void *out_scales, int scale_rule,
                        void *status_word, void *stream);

/* Grouped GEMM, one launch for all experts of an MoE layer:  D[rows of group g] = alpha * A[rows of group g] . B_g^T.
 * a_codes [M_total, K] is the row-wise concatenation of the groups' activations (quantised as one matrix,
 * DW_SF_TILED scales), every group padded with zero rows to a multiple of rows_per_tile (128 or 256);
 * tile_group[M_total / rows_per_tile] (device int32) names the group of each row tile; b_codes
 * [num_groups * N, K] stacks the groups' weights ([N, K] each, quantised as one matrix), N % 128 == 0.
 * d_bf16 [M_total, N].  rows_per_tile = 256 runs the CTA-pair kernel, 128 the single-CTA one (less padding
 * for small groups).  Out-of-range group ids are clamped.
 * Replaces BlackwellGroupedGemmKernel::grouped_gemm (csrc/cutlass_kernels.cpp:310-341: a loop of fp16
 * cublasHgemm calls, one per group), bound at csrc/python_bindings.cpp:116-194. */
int dw_mxfp8_gemm_grouped(const void *a_codes, const void *a_sf, const void *b_codes, const void *b_sf,
                          void *d_bf16, const int *tile_group, int64_t M_total, int64_t N, int64_t K,
                          int num_groups, int rows_per_tile, float alpha, void *status_word, void *stream);

/* Replaces BlackwellGemmKernel::get_workspace_size, csrc/cutlass_kernels.cpp:229-231. */
size_t dw_mxfp8_gemm_workspace(int64_t M, int64_t N, int64_t K);

/* dw_mxfp8_gemm with the launch choices of THIS call in `plan` instead of the process default
 * (dw_mxfp8_gemm_set_variant): bits [0,8) kernel variant (0 = chosen per problem; 1: one CTA, 128-wide
 * column tiles; 2: one CTA, 256-wide; 3: CTA pair on a 256 x 256 tile; 4: CTA pair, 128-wide; 5: CTA pair,
 * 192-wide), bits [8,16) row tiles per raster band, bits [16,24) split-K count, bit 24 per-thread stores
 * instead of TMA stores; 0 = everything automatic.  Two host threads (or two kernel objects) can thus run
 * different variants at the same time; nothing the call reads is process state.
 * This is where BlackwellGemmKernel::set_cluster_shape / enable_tmem_residency (csrc/cutlass_kernels.cpp:265-272,
 * per-object flags the reference stores and ignores) take effect: the Python class keeps its own plan word.
 * dw_mxfp8_gemm_workspace_planned is the matching workspace query. */
int dw_mxfp8_gemm_planned(const void *a_codes, const void *a_sf, const void *b_codes, const void *b_sf,
                          void *d_bf16, const void *bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                          float beta, void *workspace, size_t workspace_bytes, int plan, void *status_word,
                          void *stream);
size_t dw_mxfp8_gemm_workspace_planned(int64_t M, int64_t N, int64_t K, int plan);

/* Split-K GEMM that allocates nothing and needs no workspace from the caller.  No counterpart in
 * the reference.
 *
 * Some callers of this library may not (or cannot) obtain device memory at the moment they need a
 * GEMM: an operator running inside a serving engine that has already handed all free HBM to its
 * own pool and forbids cudaMalloc after warm-up, a plugin called under a lock the allocator also
 * takes, a host language binding with no access to the framework's caching allocator.  dw_mxfp8_gemm
 * asks such a caller for a workspace when it splits K; this entry point instead keeps the fp32
 * partial sums in an array that is part of the library itself: DW_GEMM_STATIC_SCRATCH_BYTES of
 * device memory on every GPU that loads the library, held until the process exits.
 *
 * Same arithmetic and operands as dw_mxfp8_gemm, with K divided among `splits` (2..255; never more
 * than ceil(K/128)) groups of thread blocks and a second kernel summing the partial results.
 * Limits and rules:
 *   - min(splits, ceil(K/128)) * M * N * 4 bytes must fit in the array, else DW_ERR_TOO_LARGE and
 *     nothing is launched;
 *   - the first call on each device looks up the array's device address (with that device current)
 *     and caches it, so make that first call outside any stream capture;
 *   - all calls on a device share the one array and it keeps whatever the last call left there.
 *     Nothing in it has to start at zero (every element the reduction reads is written by the
 *     same call first), but two calls that overlap on the GPU (different streams, or different
 *     host threads without ordering) race on it: serialise them;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine. */
#define DW_GEMM_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int dw_mxfp8_gemm_splitk_static(const void *a_codes, const void *a_sf, const void *b_codes, const void *b_sf,
                                void *d_bf16, const void *bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                                float beta, int splits, void *status_word, void *stream);

/* Synchronises `stream`, reads the status word; DW_OK or DW_ERR_DEVICE_STATUS.
 * The kernels only SET the word (once, first failure wins: low byte = which wait gave up, upper bits = CTA);
 * nothing in the library reads it back on its own, so a caller that passes a status word polls it here at a
 * point where it synchronises anyway (once per optimizer step, say) and clears it after a failure.
 * The reference reports kernel trouble with printf only (csrc/blackwell_gemm_kernel.cu:76-98). */
int dw_mxfp8_check_status(const void *status_word, void *stream);

/* Test aid for that error path: launches one tiny kernel whose single thread waits, for at most
 * `limit_cycles` SM cycles (<= DW_SELFTEST_MAX_WAIT_CYCLES, about a millisecond), on a barrier nothing
 * arrives at, with no copy and no tensor-core operation in flight.  The wait runs out, the kernel records
 * code 5 in the status word exactly as the GEMM's roles do, and returns; the context stays usable.
 * No counterpart in the reference. */
#define DW_SELFTEST_MAX_WAIT_CYCLES 2000000ll
int dw_mxfp8_selftest_bounded_wait(long long limit_cycles, void *status_word, void *stream);

/* Test aids.  dw_mxfp8_debug_fake_device: every later call of this process takes the current device to have
 * compute capability `cc_major`.x and `sms` SMs instead of asking the runtime (cc_major < 0 switches it off);
 * with cc_major != 10 every launching entry point returns DW_ERR_ARCH before it touches the device, which is
 * how that path is tested on machines without a GPU.  dw_mxfp8_debug_counter(0): tensor maps encoded so far
 * (the rest were served from the per-thread table).  No counterpart in the reference. */
int dw_mxfp8_debug_fake_device(int cc_major, int sms);
long long dw_mxfp8_debug_counter(int which);

/* Tuning aid: per-CTA counters of the SM cycles the GEMM's producer, MMA-issuer and epilogue
 * roles spent waiting, written by every later dw_mxfp8_gemm launch of this process into
 * `device_buffer` (8 int64 per CTA: [0] free stage, [1] accumulator drained, [2] shared accumulator
 * columns drained, [3] operand data, [4] accumulator finished, [7] kernel cycles).  NULL switches
 * them off.  No counterpart in the reference (its profile_kernel returns constants,
 * csrc/python_bindings.cpp:244-255). */
#define DW_GEMM_TIMING_BYTES (296 * 8 * 8)
int dw_mxfp8_gemm_set_timing_buffer(void *device_buffer, size_t bytes);

/* Process default of the plan word (see dw_mxfp8_gemm_planned) for the entry points that take none:
 * dw_mxfp8_gemm, dw_mxfp8_gemm_fused, dw_mxfp8_gemm_grouped (store mode only) and
 * dw_mxfp8_gemm_splitk_static (variant only).  A tuning and test switch; library users pass the plan per call.
 * Counterpart of the process-wide defaults in KernelSelector (csrc/cutlass_kernels.h:227-241). */
int dw_mxfp8_gemm_set_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif /* DW_MXFP8_H_ */
