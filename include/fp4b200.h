/* libfp4b200 — C ABI of the B200 (sm_100a) FP4 training hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream), enqueues its kernels on
 * that stream and returns without synchronising.  Return value: 0 on success, -1 on a
 * rejected argument or a CUDA launch error, with a message available from
 * fp4b200_last_error() (thread-local).  Outputs are caller-allocated; no entry point
 * allocates device memory unless its comment says so.
 *
 * Reference paths are relative to the reference repository root.
 *
 * Layouts (identical to the reference extensions):
 *   packed codes   uint8 [rows, cols/2], element 2j in the low nibble of byte j
 *   NVFP4 scales   E4M3 bytes, tiles of 128 rows x 4 blocks = 512 bytes,
 *                  [rows/128, cols/64, 512], offset (r%32)*16 + ((r%128)/32)*4 + (kb%4)
 *   MXFP4 scales   E8M0 bytes, same 512-byte tile, [rows/128, cols/128, 32, 16]
 *   amax_sg        float[2]: [0] tensor amax, [1] sg = amax / 2688 (GEMM-side tensor scale)
 */
#ifndef FP4B200_H_
#define FP4B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- housekeeping --------------------------------------------------------------------- */

/* Message of the last failed call on this thread ("" if none). */
const char* fp4b200_last_error(void);
/* ABI revision of this header. */
int fp4b200_abi_version(void);
/* Synchronises the current device, returns and clears the device status word: 0, or the code
 * of a kernel that gave up a bounded wait (1 quantiser TMA, 2..5 GEMM pipeline stages).
 * The reference has no counterpart: its kernels spin without a limit
 * (fp4_runtime/TK_quantisation/nvfp4_v5/fused_amax_quantize.cuh:198-206). */
int fp4b200_device_status(void);

/* ---- NVFP4 producers ------------------------------------------------------------------ */

/* Tensor amax of a bf16 buffer and sg = amax/2688.
 * Replaces pipelined_amax::fused_amax_pipelined_kernel
 * (fp4_runtime/TK_quantisation/nvfp4_v5/amax_pipelined.cuh:26-48,504-512). */
int fp4b200_nvfp4_amax(const void* x_bf16, int64_t n_elems, float* amax_sg, void* stream);

/* Row-wise (and, when col_* are non-NULL, column-wise) NVFP4 quantisation of bf16 [M,K]
 * from given device-resident tensor amaxes (amax_col NULL = same as amax_row).  M, K
 * multiples of 128.  sg_out (optional) receives amax_row/2688.
 * Replaces tk_quantize_transpose / quantize_transpose_nvfp4_tuned_1D_kernel, RTN path
 * (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:3807-3926,
 *  quantize_transpose_tuned.cuh:530-1007). */
int fp4b200_nvfp4_quantize(const void* x_bf16, int64_t M, int64_t K, const float* amax_row,
                           const float* amax_col, int encode_centric, void* row_fp4, void* row_sc,
                           void* col_fp4, void* col_sc, float* sg_out, void* stream);

/* amax + quantise in one call: tk_quantize_for_gemm(input, return_transpose, encode_centric)
 * (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:2208-2412). */
int fp4b200_nvfp4_quantize_for_gemm(const void* x_bf16, int64_t M, int64_t K, int return_transpose,
                                    int encode_centric, void* row_fp4, void* row_sc, void* col_fp4,
                                    void* col_sc, float* amax_sg, void* stream);

/* One launch of the stochastic-rounding / Hadamard variant of the quantiser, the counterpart of
 * tk_quantize_transpose(input, amax_row, amax_col, return_transpose, stochastic_rounding, encode_centric,
 * scale_sr=false, row_rht, col_rht, return_row, rng_state) (tk_quantize.cu:3807-3926; kernel
 * quantize_transpose_tuned.cuh:256-528).  data_sr: Philox4x32-10 stochastic rounding of the codes,
 * key rng_seed, counter offset rng_offset (= the reference's rng_state[1]), sequence and draw order
 * those of the reference kernel, so equal (seed, offset) give equal bytes: 1 = on every pass of this
 * launch; 2 = row pass only, the bytes of the reference's row-only launch at rng_offset (its stream
 * has 8 words per stage), with the column pass rounded to nearest in the same launch; 3 = column pass
 * only, at rng_offset_col (the offset of the reference's separate column launch); 4 = both passes, the row pass
 * as with 2 and the column pass as with 3.  With 2, 3 and 4 the callers that the reference serves with two
 * launches (one axis stochastic, or a sign-masked transform) read the input once.
 * rht_row / rht_col: per-16 Hadamard transform (x0.25, rounded to bf16) along K for the row operand /
 * along M for the column operand, optionally after a sign flip hashed from (sign_seed, sign_subseq,
 * coordinate) (tk_quantize.cu:483-488,620-627).  gamma/inv_rms non-NULL fuse RMSNorm.  return_row = 0
 * writes no row-wise output but keeps its words in the random stream.  scale_sr: the E4M3 scale byte of
 * every block is rounded stochastically by one more word of the same stream, drawn before the block's data
 * words (quantize_transpose_tuned.cuh:205-254); with data_sr 2 / 3 the row pass follows the row-only launch
 * at rng_offset and the column pass the column launch at rng_offset_col, as above.  The reference draws no
 * scale word for an encode-centric block whose maximum is <= 1e-9 (quantize_transpose_tuned.cuh:244-254), which
 * moves every later draw of the reference thread that owns the block: with ec_zero_scratch (device memory,
 * M*K/32 bytes, 2-byte aligned; used only when encode_centric and scale_sr) a first kernel maps those blocks and
 * the draws follow the reference's; with NULL every block is taken to draw a scale word.  scale_sr needs 16-byte
 * aligned outputs.
 * rng_state: NULL, or two 64-bit device words {key, base} (8-byte aligned) that fp4b200_sr_prepare_state wrote
 * earlier on the stream: the kernel then takes its key from rng_state[0] (rng_seed is ignored) and adds
 * rng_state[1] to rng_offset and rng_offset_col, which become the launch's place among the launches that were
 * reserved together (0, 2^32, ...).  This is the reference's rng_state tensor (tk_quantize.cu:3807-3926 reads it in
 * the kernel), and what makes the call safe to capture in a CUDA graph. */
int fp4b200_nvfp4_quantize_opt(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                               const float* amax_row, const float* amax_col, int encode_centric, int data_sr,
                               int rht_row, int rht_col, int with_sign, uint64_t sign_seed, uint64_t sign_subseq,
                               int return_row, uint64_t rng_seed, uint64_t rng_offset, uint64_t rng_offset_col,
                               const uint64_t* rng_state, int scale_sr,
                               void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* ec_zero_scratch, void* stream);

/* Numbering of stochastic launches on the device (tk_quantize.cu:443-481: tk_sr_invocation_offset,
 * tk_prepare_advancing_rng_state_kernel).  The library keeps one 64-bit counter per device.
 * fp4b200_sr_prepare_state launches one thread that adds launches * 2^32 to the counter and writes
 * rng_state[0] = rng_seed, rng_state[1] = rng_subsequence + (the counter before the addition); rng_state is device
 * memory for two 64-bit words.  Because the addition happens on the device, a replayed CUDA graph that holds this
 * launch reserves new numbers on every replay.  fp4b200_sr_set_invocation_offset stores a value into the counter
 * (stream-ordered; checkpoint resume and tests: the reference's counter cannot be set) and
 * fp4b200_sr_get_invocation_offset copies it into out_dev (device memory, stream-ordered). */
int fp4b200_sr_prepare_state(uint64_t* rng_state, uint64_t rng_seed, uint64_t rng_subsequence, uint64_t launches,
                             void* stream);
int fp4b200_sr_set_invocation_offset(uint64_t value, void* stream);
int fp4b200_sr_get_invocation_offset(uint64_t* out_dev, void* stream);
/* The per-producer numbering (low_bits_training/quantization/localcta_sr_state.py:1-11: one persistent int64[2]
 * {seed, next subsequence} per producer, advanced by the extension on the producer's stream right before its
 * quantiser).  One thread copies producer_state[0..1] into rng_state[0..1] and adds launches * 2^32 to
 * producer_state[1]; rng_state then serves fp4b200_nvfp4_quantize_opt exactly as after fp4b200_sr_prepare_state.
 * Both are device memory, 8-byte aligned.  The library's per-device counter is not touched. */
int fp4b200_sr_reserve_from_state(int64_t* producer_state, uint64_t* rng_state, uint64_t launches, void* stream);

/* As fp4b200_nvfp4_quantize_opt, with the row-wise codes written into a column slice of a wider matrix:
 * row_pitch_bytes is that matrix's row pitch (0: K/2, a dense [M, K/2]); 16-byte aligned outputs only.  Serves the
 * stochastic-rounding route of tk_group_quantize_dim1_split3_for_gemm (nvfp4_v5/tk_quantize.cu:6485-6548: one
 * launch of the tuned kernel per gradient stream into slices of one row-wise and one column-wise code matrix). */
int fp4b200_nvfp4_quantize_opt_into(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                                    const float* amax_row, const float* amax_col, int encode_centric, int data_sr,
                                    int rht_row, int rht_col, int with_sign, uint64_t sign_seed, uint64_t sign_subseq,
                                    int return_row, uint64_t rng_seed, uint64_t rng_offset, uint64_t rng_offset_col,
                                    const uint64_t* rng_state, int scale_sr, void* row_fp4, int64_t row_pitch_bytes, void* row_sc, void* col_fp4,
                                    void* col_sc, void* ec_zero_scratch, void* stream);

/* Tensor amax (and sg) of the per-16 Hadamard transform of x along K (along_k != 0) or along M,
 * measured on the fp32 transform output: rht16_bf16_amax_kernel (tk_quantize.cu:574-664).  gamma/inv_rms
 * non-NULL (along K only) transform bf16(x*inv_rms*gamma): rmsnorm_rht16_amax_with_orig_kernel (:1113-1172).
 * plain_amax_sg (NULL or two floats; scan along M only): the tensor amax and sg of x itself from the same read — the
 * row operand's scale when only the column operand is transformed (the reference runs a second scan for it). */
int fp4b200_nvfp4_rht16_amax(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                             int along_k, int with_sign, uint64_t sign_seed, uint64_t sign_subseq, float* amax_sg,
                             float* plain_amax_sg, void* stream);

/* tk_quantize_weight_2d(input) (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:2445-2555): one
 * decode-centric scale per 16x16 tile shared by both orientations, so that the column-wise codes
 * are the exact transpose of the row-wise codes. */
int fp4b200_nvfp4_quantize_weight_2d(const void* w_bf16, int64_t N, int64_t K, void* row_fp4, void* row_sc,
                                     void* col_fp4, void* col_sc, float* amax_sg, void* stream);

/* The same 16x16-tile quantisation with the tensor amax given (a device scalar) instead of computed: a row shard of a
 * weight quantised with the amax of the whole weight gives the whole weight's bytes for its rows, which is what a
 * packed all-gather of 2-D quantised weight shards needs.  No counterpart in the reference, which quantises the
 * gathered weight. */
int fp4b200_nvfp4_quantize_weight_2d_with_amax(const void* w_bf16, int64_t N, int64_t K, const float* amax, void* row_fp4,
                                               void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* RMSNorm statistics: inv_rms[M] = rsqrt(mean(x^2)+eps) (computed when compute_inv_rms != 0,
 * else read) and amax of bf16(x*inv_rms*gamma); amax_sg may be NULL when only inv_rms is wanted (the MXFP4
 * producers: no tensor scale), which skips the second sweep over each row.
 * Replaces rmsnorm_bf16_amax_kernel (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:1025-1111). */
int fp4b200_nvfp4_rmsnorm_stats(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                float* inv_rms, int compute_inv_rms, float* amax_sg, void* stream);

/* Fused RMSNorm + NVFP4 quantisation: tk_fused_norm_quantize (barrier-free branch) and
 * tk_fused_norm_quantize_from_inv_rms (compute_inv_rms = 0)
 * (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:8003-8243,8250-8259).  The reference
 * hard-wires encode_centric = 1 on this path. */
int fp4b200_nvfp4_fused_norm_quantize(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M,
                                      int64_t K, float* inv_rms, int compute_inv_rms, int encode_centric,
                                      void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                      float* amax_sg, void* stream);

/* Second pass of the fused producer on its own: quantise bf16(x*inv_rms*gamma) given inv_rms[M]
 * and the device-resident tensor amax (as written by fp4b200_nvfp4_rmsnorm_stats).
 * Replaces launch_v2_rmsnorm_kernel / quantize_transpose_nvfp4_tuned_1D_kernel<APPLY_RMSNORM>
 * (fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:1512-1582, quantize_transpose_tuned.cuh:761-779). */
int fp4b200_nvfp4_quantize_normed(const void* x_bf16, const void* gamma_bf16, const float* inv_rms,
                                  const float* amax, int64_t M, int64_t K, int encode_centric, void* row_fp4,
                                  void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* Fused RMSNorm + NVFP4 quantisation (encode-centric, as fp4b200_nvfp4_fused_norm_quantize with
 * compute_inv_rms = 1) for callers that cannot allocate device memory: code running under a memory pool
 * that is already full by design, or in a host thread that is not allowed to touch the allocator.
 * It has no counterpart in the reference, whose producers
 * always allocate their scratch through torch.  The caller passes inputs and outputs only (sg_out
 * receives amax/2688); the per-row inverse RMS and the first pass's per-CTA partial maxima live
 * in a fixed array inside the library (264 KiB per device, held until the process exits), so M is
 * limited to 65536 rows and larger calls are rejected with an error.  The first call on a device
 * looks up the array's device address (cached afterwards; host threads may race to cache the same value).  All calls
 * share the array, which keeps the previous call's contents (every call overwrites the part it
 * reads): two calls that overlap on the GPU, e.g. on different streams, race. */
int fp4b200_nvfp4_fused_norm_quantize_noalloc(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M,
                                              int64_t K, void* row_fp4, void* row_sc, void* col_fp4,
                                              void* col_sc, float* sg_out, void* stream);

/* ---- MXFP4 producers ------------------------------------------------------------------- */

/* Row (+column when col_* non-NULL) MXFP4 quantisation of bf16 [M,K]: 32-element blocks, E8M0
 * scale = exponent of the block amax rounded by mode (0 RTE, 1 ceil, 2 floor), codes =
 * e2m1(x * 6 * 2^(127-e)).  Replaces mxfp4_quantize_row_and_col / mxfp4_quantize_for_gemm
 * (fp4_runtime/TK_quantisation/mxfp4_v4/tk_quantize.cu:1883-2060; kernels mxfp4_v3_quantize.cuh:1540-1790) and, with
 * row_fp4 = row_sc = NULL, mxfp4_quantize_col_only (tk_quantize.cu:2404-2470): the column operand alone. */
int fp4b200_mxfp4_quantize(const void* x_bf16, int64_t M, int64_t K, int mode, void* row_fp4, void* row_sc,
                           void* col_fp4, void* col_sc, void* stream);

/* Same on bf16(x * inv_rms[row] * gamma[col]): second half of
 * mxfp4_fused_rmsnorm_quantize_row_and_col (mxfp4_v4/tk_quantize.cu:6947-6964); inv_rms comes from
 * fp4b200_nvfp4_rmsnorm_stats. */
int fp4b200_mxfp4_quantize_normed(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M,
                                  int64_t K, int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                  void* stream);
/* inv_rms[r] = rsqrtf(sum_k x[r,k]^2 / K + eps) in the summation order of the reference's MXFP4 producer
 * (mxfp4_v4/mxfp4_v3_quantize.cuh:109-172, compute_inv_rms_kernel: 256 threads, thread t takes the 8-element vectors
 * t, t + 256, ... in sequence, xor butterflies inside and across its warps), which differs from the NVFP4 producer's
 * tree in the last bit of some rows.  gamma (16-byte aligned, [K]) is only staged, not used.  Feeds
 * fp4b200_mxfp4_quantize_normed for mxfp4_fused_rmsnorm_quantize_row_and_col. */
int fp4b200_mxfp4_rmsnorm_inv_rms(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                  float* inv_rms, void* stream);
/* The same in the order of the inverse-RMS kernel that runs in front of tk_fused_norm_quantize_opt's stochastic forms
 * (nvfp4_v5/fused_norm_quantize.cuh:391-434: 256 threads, thread t takes the single elements t, t + 256, ...; xor
 * butterflies inside the warps, then over the eight warp sums) — a third tree, again different in the last bit of
 * some rows from the one tk_fused_norm_quantize uses. */
int fp4b200_nvfp4_rmsnorm_inv_rms_opt(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                      float* inv_rms, void* stream);

/* ---- SwiGLU producers ------------------------------------------------------------------ */

/* h = bf16(silu(h1) * h3) element-wise and its tensor amax / sg; n_elems multiple of 8.
 * Replaces tk_silu_split::silu_mul_split_kernel
 * (fp4_runtime/TK_quantisation/nvfp4_v5/silu_split_bf16.cuh:62-140). */
int fp4b200_silu_mul_bf16(const void* h1, const void* h3, int64_t n_elems, void* h_out, float* amax_sg,
                          void* stream);

/* tk_silu_quantize_split_for_gemm(h1_raw, h3) (tk_quantize.cu:8985-9123): h as above (materialised
 * in h_bf16 [M,H]) then row (+column) NVFP4 quantisation of h with its own tensor amax. */
int fp4b200_nvfp4_silu_quantize(const void* h1, const void* h3, int64_t M, int64_t H, void* h_bf16,
                                int encode_centric, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                float* amax_sg, void* stream);

/* dh1 = bf16(dh*h3*silu'(h1)), dh3 = bf16(dh*silu(h1)) and their amax/sg pairs.
 * Replaces tk_silu_split::silu_deriv_dual_split_kernel (silu_split_bf16.cuh:181-300); the
 * quantisation of dh1/dh3 (tk_silu_deriv_quantize_split_for_gemm[_opt], tk_quantize.cu:9418-9640,
 * 10063-10255) is two calls of fp4b200_nvfp4_quantize with these amaxes. */
int fp4b200_silu_deriv_bf16(const void* dh, const void* h3, const void* h1, int64_t n_elems, void* dh1_out,
                            void* dh3_out, float* amax_sg1, float* amax_sg3, void* stream);

/* ---- block-scaled FP4 GEMMs ------------------------------------------------------------ */
/* Shapes: M % 128 == 0, N % 128 == 0, K % 256 == 0 (NVFP4) or K % 128 == 0 (MXFP4).  A [M,K/2] and
 * B [N,K/2] packed codes, scales in the 512-byte tile layout above, D row-major [M,N] written in place.
 * out_fp32 = 0: D is bf16, = 1: D is fp32 (the accumulator times the tensor scales, unrounded).
 * residual_bf16 (optional, bf16 [M,N]): D = bf16(bf16(acc*scale) + R).
 * The kernels are launched as programmatic dependents of the previous kernel in the stream (their set-up
 * overlaps its tail; they touch no global memory before its writes are visible). */

/* The first-pass kernels of the quantisers (tensor maximum, RMSNorm statistics) are launched as programmatic
 * dependents too.  By default they read nothing before the previous kernel on the stream has ended, because their
 * input is usually what that kernel produced.  enabled = 1 is the caller's promise that no input of a call (x, gamma)
 * is written by the kernel launched immediately before it on the same stream — true of back-to-back calls on
 * independent inputs — and lets those kernels fill their shared-memory rings while the previous kernel drains
 * (-5 us per fused call at [16384 x 4096]).  Process-wide; returns the previous setting; FP4B200_PDL_EARLY_READS=1
 * sets it at load.  No counterpart in the reference. */
int fp4b200_set_pdl_early_reads(int enabled);

/* No counterpart in the reference.  Launches a one-warp kernel that waits, with the same bounded wait every kernel
 * of this library uses, on a barrier nothing will arrive on: after limit_cycles (1 .. 1e8) clock cycles it gives
 * up, stores status code 6 and returns.  fp4b200_device_status() then reports 6 once and 0 afterwards.  For tests of
 * the failure-reporting path; no copy is in flight and nothing is left waiting. */
int fp4b200_selftest_bounded_wait(int64_t limit_cycles, void* stream);
/* Self-test of the SwiGLU producers' division: for every bf16 pattern x with |x| < 64 compares, on the device, the
 * short sequence they use for x / d and 1 / d (d = 1 + __expf(-x): reciprocal estimate, one Newton step, one corrected
 * product) with the general IEEE division; mismatches_dev[0], [1] receive the number of patterns that differ (0, 0
 * on a correct build).  No counterpart in the reference, whose element kernels use the general division. */
int fp4b200_selftest_silu_division(uint32_t* mismatches_dev, void* stream);

/* Switches that launch attribute for the GEMM calls of the calling thread (1 = on, the default; 0 = ordinary
 * launches) and returns the previous setting: what the reference's *_nopdl entry points select
 * (nvfp4_b200_gemm.cu:1702-1735; kernel nvfp4_gemm.cuh:577,596,1002).  FP4B200_GEMM_PDL=0 in the environment
 * switches it off for the whole process. */
int fp4b200_set_gemm_pdl(int enabled);

/* D = bf16((A.B^T) * A_sg * B_sg): nvfp4_gemm / nvfp4_gemm_config / nvfp4_gemm_nopdl /
 * nvfp4_gemm_residual (fp4_runtime/ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:648-761,
 * 1702-1735, 1899-1920; kernel nvfp4_gemm.cuh:490-1012).  A_sg, B_sg: device scalars. */
int fp4b200_nvfp4_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                       const float* B_sg, void* D, int out_fp32, const void* residual_bf16, int64_t M, int64_t N,
                       int64_t K, void* stream);

/* One term of nvfp4_batched_accum_gemm (nvfp4_b200_gemm.cu:2567-2635; kernel nvfp4_batched_accum_gemm.cuh):
 * D = round(fma(acc, A_sg * B_sg, partial_f32)), partial_f32 a caller buffer [M,N] holding the fp32 sum of the
 * earlier terms (written by this entry point or by fp4b200_nvfp4_gemm with out_fp32 = 1).  One rounding per term
 * after the first, as the reference's kernel does (nvfp4_batched_accum_gemm.cuh:293-310: its multiply and add are
 * compiled to a fused multiply-add).  D may alias partial_f32 when out_fp32 = 1. */
int fp4b200_nvfp4_gemm_accum(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                             const float* B_sg, const float* partial_f32, void* D, int out_fp32, int64_t M, int64_t N,
                             int64_t K, void* stream);

/* nvfp4_batched_accum_gemm in one launch (nvfp4_b200_gemm.cu:2567-2635; kernel nvfp4_batched_accum_gemm.cuh):
 * D = bf16(sum_i (A_i . B_i^T) * A_sg_i * B_sg_i) for 1 to 4 terms, each with its own operands, scale tensors,
 * tensor scales and reduction width K[i].  The terms' accumulators are handed to the epilogue one after the other
 * and summed there in fp32 registers in the reference's order (term 0 multiplied, every later term by one fused
 * multiply-add), one rounding to bf16, one store.  A term's A may be a column slice of a wider matrix, which is what
 * nvfp4_split_dgrad_sum (nvfp4_b200_gemm.cu:2424-2565) needs: A_pitch_bytes[i] is then the row pitch of its codes
 * (NULL or 0: K[i]/2) and A_sc_row_tiles[i] the number of 512-byte scale tiles between consecutive 128-row blocks of
 * its scale tensor (NULL or 0: K[i]/64).  round_each_term = 1 gives nvfp4_split_dgrad_sum's arithmetic instead of
 * nvfp4_batched_accum_gemm's: the reference runs a batched GEMM into one bf16 matrix per split and adds those with
 * Tensor.add_ (nvfp4_b200_gemm.cu:2466-2487), so every term is rounded to bf16 and the running sum is rounded to bf16
 * after every addition, left to right.  Needs M % 256 == 0 (two-CTA kernel); otherwise chain fp4b200_nvfp4_gemm
 * (fp32 output) and fp4b200_nvfp4_gemm_accum. */
int fp4b200_nvfp4_batched_accum_gemm(int n_terms, const void* const* A, const void* const* A_sc, const float* const* A_sg,
                                     const void* const* B, const void* const* B_sc, const float* const* B_sg,
                                     const int64_t* K, const int64_t* A_pitch_bytes, const int64_t* A_sc_row_tiles, void* D,
                                     int64_t M, int64_t N, int round_each_term, void* stream);

/* nvfp4_grouped_gemm (nvfp4_b200_gemm.cu:764-841): B is the row concatenation of n_out weights,
 * B_sg_per_tile holds one tensor scale per 256 rows of B, output i receives D_cols[i] columns
 * (each a multiple of 256, adding up to N) into its own bf16 [M, D_cols[i]] buffer. */
int fp4b200_nvfp4_grouped_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                               const float* B_sg_per_tile, int n_out, void* const* D, const int64_t* D_cols,
                               int64_t M, int64_t N, int64_t K, void* stream);

/* D = bf16((A.B^T) / 36) with E8M0 scales per 32 elements: mxfp4_gemm / mxfp4_gemm_config /
 * mxfp4_gemm_residual (fp4_runtime/ThunderKittens/kernels/gemm/mxfp4_gb200/mxfp4_gb200_gemm.cu:2704-2950;
 * kernel mxfp4_gemm.cuh, 1/36 at :557-558). */
int fp4b200_mxfp4_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int out_fp32,
                       const void* residual_bf16, int64_t M, int64_t N, int64_t K, void* stream);

/* mxfp4_gemm_rope_live64[_config] / mxfp4_gemm_rope_live[_config](A, A_sc, B, B_sc, D, rope_cs, rope_seq_len)
 * (mxfp4_gb200/mxfp4_gb200_gemm.cu:1777-1812; epilogue mxfp4_rope_epilogue.cuh:263-308): D = bf16(rotate((A.B^T) / 36)),
 * every neighbouring column pair (2i, 2i+1) of token row r rotated by rope_cs[r mod rope_seq_len, i mod
 * (rope_head_dim / 2)] = (cos, sin) in fp32 before the one rounding.  rope_cs fp32 [rope_seq_len, rope_head_dim/2, 2];
 * rope_seq_len and rope_head_dim powers of two.  Same kernels as the NVFP4 rotary forms (two-CTA kernel with eight
 * epilogue warps when M is a multiple of 256). */
int fp4b200_mxfp4_gemm_rope(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, const float* rope_cs,
                            int64_t rope_seq_len, int64_t rope_head_dim, int64_t M, int64_t N, int64_t K, void* stream);

/* mxfp4_split2_dgrad_strided_onepass_gemm(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list,
 * D_out, config_idx) (mxfp4_gb200/mxfp4_gb200_gemm.cu:2572-2596; kernel mxfp4_split2_accum_gemm.cuh):
 * D = bf16((sum_s A_full[:, off_s : off_s + w_s] * B_s^T) / 36) with all terms accumulated in tensor memory
 * before the one rounding.  A_full's codes are [M, a_width/2]; segment s has its own scale tiles
 * A_sc_list[s] [M/128, w_s/128, 512], operand B_list[s] [N, w_s/2] and B_sc_list[s] [N/128, w_s/128, 512].
 * Up to 4 segments, each a multiple of 256 elements wide. */
int fp4b200_mxfp4_gemm_ksplit(const void* A_full, int64_t a_width, int n_seg, const int64_t* a_col_offsets,
                              const int64_t* a_col_widths, const void* const* A_sc_list, const void* const* B_list,
                              const void* const* B_sc_list, void* D, int out_fp32, int64_t M, int64_t N, void* stream);

/* The same with A_sc_list[s] a column slice of a wider scale tensor, as the reference's caller passes it
 * (row_sc.narrow(1, ...) of the combined producer's [M/128, 2H/128, 512] tensor, mxfp4_fused_linear.py:10803-10829):
 * a_sc_row_tiles[s] = 512-byte tiles from one 128-row block of that tensor to the next (0 or a null array: w_s/128). */
int fp4b200_mxfp4_gemm_ksplit_strided(const void* A_full, int64_t a_width, int n_seg, const int64_t* a_col_offsets,
                                      const int64_t* a_col_widths, const void* const* A_sc_list,
                                      const int64_t* a_sc_row_tiles, const void* const* B_list,
                                      const void* const* B_sc_list, void* D, int out_fp32, int64_t M, int64_t N, void* stream);

/* ---- helpers around the hot path -------------------------------------------------------- */

/* mxfp4_quantize_weight_2d(input) (mxfp4_v4/tk_quantize.cu:2734-2737; kernel mx_weight_2d_quantize,
 * mxfp4_v3_quantize.cuh:1797-1960): one E8M0 scale per 32x32 tile shared by both orientations = the
 * ceil exponent of the tile amax, lowered by one when amax * 2^-(e-127) < 0.87; column codes are the
 * transposed row codes. */
int fp4b200_mxfp4_quantize_weight_2d(const void* w_bf16, int64_t N, int64_t K, void* row_fp4, void* row_sc,
                                     void* col_fp4, void* col_sc, void* stream);

/* mxfp4_quantize_nhsd_wo_row_and_col(input, mode) (mxfp4_v4/tk_quantize.cu:2739-2830): the attention output in its
 * native [B, H, S, D] layout (D a multiple of 64, S of 128) quantised as the matrix [M = B*S, K = H*D] the output
 * projection consumes (element (b*S + s, h*D + d) = input[b, h, s, d]) without a transposing copy; outputs as
 * fp4b200_mxfp4_quantize. */
int fp4b200_mxfp4_quantize_nhsd_wo(const void* x_bf16, int64_t B, int64_t H, int64_t S, int64_t D, int mode, void* row_fp4,
                                   void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* mxfp4_quantize_split2_row_and_col(input0, input1, mode) / mxfp4_quantize_split3_row_and_col(input0, input1, input2,
 * mode) and their _launch_inplace twins (mxfp4_v4/tk_quantize.cu:5375-5470, 6254-6440): the operands of the column
 * concatenation [M, sum widths] of n = 2 or 3 bf16 matrices with the same row count (the gradients of a fused
 * projection's outputs) without concatenating them: row_fp4 [M, K/2], row_sc [M/128, K/128, 512], col_fp4 [K, M/2],
 * col_sc [K/128, M/128, 512], K = sum of widths. */
int fp4b200_mxfp4_quantize_split(const void* const* xs, const int64_t* widths, int n, int64_t M, int mode, void* row_fp4,
                                 void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* mxfp4_quantize_split3_row_and_col_inverse_rope_live64(input0, input1, input2, rope_cs, rope_seq_len, mode)
 * (mxfp4_v4/tk_quantize.cu:6551-6644; kernel mxfp4_v3_quantize.cuh:6165, rotation :251-285): the three-input split
 * quantiser with the inverse rotary embedding of dQ and dK folded into the load (heads of 64, neighbouring columns
 * (2i, 2i+1) of token row r rotated back by rope_cs[r mod rope_seq_len, i mod 32] = (cos, sin), rounded to bf16, then
 * quantised); dV is quantised as it is.  rope_cs fp32 [rope_seq_len, 32, 2], rope_seq_len a power of two. */
int fp4b200_mxfp4_quantize_split3_inverse_rope(const void* dq, const void* dk, const void* dv, int64_t M, int64_t kq,
                                               int64_t kk, int64_t kv, const float* rope_cs, int64_t rope_seq_len, int mode,
                                               void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* mxfp4_fused_silu_mul_quantize_row_and_col_strided(h13, H, h3_offset, mode) (mxfp4_v4/tk_quantize.cu:4105-4132): the
 * SwiGLU producer reading h1 and h3 out of one packed gate|up activation h13 [M, h13_stride] (h1 in columns [0, H), h3
 * in [h3_offset, h3_offset + H)); outputs as fp4b200_mxfp4_silu_mul_quantize. */
int fp4b200_mxfp4_silu_mul_quantize_strided(const void* h13, int64_t h13_stride, int64_t h3_offset, int64_t M, int64_t H,
                                            int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* One-pass MXFP4 SwiGLU producers: the activation is computed on the chunk in shared memory and only codes and
 * scales are written (no tensor-level scale exists, so nothing has to be known about the whole tensor first).
 * fp4b200_mxfp4_silu_mul_quantize: operands of bf16(silu(h1_raw) * h3)
 * (mxfp4_fused_silu_mul_quantize_row_and_col[_launch_inplace], mxfp4_v4/tk_quantize.cu:3231-3310).
 * fp4b200_mxfp4_silu_deriv_quantize_split2: operands of dh1 = bf16(dh * h3 * silu'(h1_raw)) and dh3 =
 * bf16(dh * silu(h1_raw)), dh3's stacked behind dh1's in every output array: row_fp4 [2, M, H/2], row_sc
 * [2, M/128, H/128, 512], col_fp4 [2, H, M/2], col_sc [2, H/128, M/128, 512]
 * (mxfp4_fused_silu_deriv_quantize_split2_row_and_col[_launch_inplace], mxfp4_v4/tk_quantize.cu:4513-4700).
 * Same bytes as the element kernels (fp4b200_silu_mul_bf16 / fp4b200_silu_deriv_bf16) followed by
 * fp4b200_mxfp4_quantize.  M % 128 == 0, H % 128 == 0, 16-byte aligned inputs; all outputs required. */
int fp4b200_mxfp4_silu_mul_quantize(const void* h1_raw, const void* h3, int64_t M, int64_t H, int mode, void* row_fp4,
                                    void* row_sc, void* col_fp4, void* col_sc, void* stream);
int fp4b200_mxfp4_silu_deriv_quantize_split2(const void* dh, const void* h3, const void* h1_raw, int64_t M, int64_t H,
                                             int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                             void* stream);

/* mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined(dh, h13, H, h3_offset, mode)
 * (mxfp4_v4/tk_quantize.cu:5015-5099; kernel mxfp4_v3_quantize.cuh:8559): the same two gradients from dh [M, dh_stride]
 * and a packed gate|up activation h13 [M, h13_stride] (h1 in columns [0, H), h3 in [h3_offset, h3_offset + H)), laid
 * out for the one-pass split dgrad GEMM: row_fp4 [M, H] bytes = dh1's codes | dh3's codes, row_sc
 * [M/128, 2H/128, 512] = dh1's scale tiles | dh3's per row block, col_fp4 [2H, M/2] and col_sc [2H/128, M/128, 512]
 * = dh1's over dh3's. */
int fp4b200_mxfp4_silu_deriv_quantize_split2_combined(const void* dh, int64_t dh_stride, const void* h13, int64_t h13_stride,
                                                      int64_t h3_offset, int64_t M, int64_t H, int mode, void* row_fp4,
                                                      void* row_sc, void* col_fp4, void* col_sc, void* stream);

/* mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols[_launch_inplace](dh, h3, h1_raw, ...)
 * (mxfp4_v4/tk_quantize.cu:4708-4905), the producer the reference's default gate/up backward feeds its one-pass split
 * dgrad GEMM from (mxfp4_fused_linear.py:10415-10431): the row-wise operand in the combined layout above (row_fp4
 * [M, H] bytes, row_sc [M/128, 2H/128, 512]), the column-wise operands of dh1 and dh3 in tensors of their own
 * (col*_fp4 [H, M/2], col*_sc [H/128, M/128, 512]). */
int fp4b200_mxfp4_silu_deriv_quantize_split2_splitcols(const void* dh, const void* h3, const void* h1_raw, int64_t M,
                                                       int64_t H, int mode, void* row_fp4, void* row_sc, void* col0_fp4,
                                                       void* col0_sc, void* col1_fp4, void* col1_sc, void* stream);

/* mxfp4_quantize_for_gemm_opt(input, mode, data_stochastic_rounding, scale_stochastic_rounding, rng_seed,
 * rng_subsequence) (mxfp4_v4/tk_quantize.cu:1796-1881; kernel mxfp4_v3_fused_kernel_opt / mx_rowwise_quantize_opt,
 * mxfp4_v3_quantize.cuh:1618-1790, 5270-5345): row operand only.  data_sr rounds the codes stochastically
 * (cvt.rs.satfinite.e2m1x4.f32 with the words of the owning reference thread's Philox stream: subsequence
 * rng_subsequence + ((chunk * 4 + tile) * 128 + thread), offset 0); scale_sr rounds the E8M0 byte up with
 * probability mantissa / 2^23 (and replaces the mode's rule).  Each 16-element half of a 32-block rounds the
 * scale with its own word: the stored byte is the first half's, the second half's codes use its own, as the
 * reference does.  rht_block 16 or 32 (mxfp4_quantize_for_gemm_opt_rht, tk_quantize.cu:1883-2060): a Hadamard
 * transform of that many consecutive elements of a row in front of the quantisation (fp32 butterflies, block
 * maximum of the fp32 output, codes from its bf16 rounding), behind the reference's fixed sign diagonal when
 * rht_sign is set; with a transform both SR flags may be 0.  M, K multiples of 128; row_fp4 [M, K/2],
 * row_sc [M/128, K/128, 512]. */
int fp4b200_mxfp4_quantize_row_sr(const void* x_bf16, int64_t M, int64_t K, int mode, int data_sr, int scale_sr,
                                  int rht_block, int rht_sign, uint64_t rng_seed, uint64_t rng_subsequence, void* row_fp4,
                                  void* row_sc, void* stream);

/* mxfp4_quantize_row_and_col_opt(input, mode, data_stochastic_rounding, scale_stochastic_rounding, rng_seed,
 * rng_subsequence) without a Hadamard transform (mxfp4_v4/tk_quantize.cu:2820-2953; kernel
 * mxfp4_v4_rowcol_fused_kernel_opt, mxfp4_v3_quantize.cuh:5443-5560).  rng_subsequence here is the base the launch
 * ends up with: the caller's value plus the reference's per-call offset (2^40 times the number of earlier SR
 * calls; the Python mirror keeps that counter).  data_sr is the reference's "correlated" rounding: the row and the
 * column view round element (i, j) with the same 16-bit integer, derived from (rng_seed, base, chunk, i, j) by a
 * GF(2^16) construction instead of the Philox stream; scale_sr draws from the reference threads' Philox streams
 * as in fp4b200_mxfp4_quantize_row_sr (column view: its own subsequences).  row_rht / col_rht with rht_block 16 or
 * 32 (mxfp4_quantize_row_and_col_opt_rht: column view only, _rht_both, _rht_row_only; tk_quantize.cu:2955-3146)
 * transform the row view along K and / or the column view along M; data_sr then draws from the Philox streams in
 * both views instead of the correlated construction, as the reference does. */
int fp4b200_mxfp4_quantize_row_and_col_sr(const void* x_bf16, int64_t M, int64_t K, int mode, int data_sr, int scale_sr,
                                          int rht_block, int rht_sign, int row_rht, int col_rht, uint64_t rng_seed,
                                          uint64_t rng_subsequence, void* row_fp4, void* row_sc, void* col_fp4,
                                          void* col_sc, void* stream);

/* nvfp4_row_rms_reduce(row_rms_partial, coeff, hidden_size, eps) (nvfp4_b200_gemm.cu:1792-1803; kernel
 * common/c1_rms_reduce.cuh:11-38), also the first step of tk_fused_norm_quantize_from_row_rms_partial
 * (nvfp4_v5/tk_quantize.cu:8266-8308) and of mxfp4_fused_rmsnorm_quantize_row_and_col_from_row_rms_partial
 * (mxfp4_v4/tk_quantize.cu:6960-7052): inv_rms[r] = rsqrtf(sum_c partial[r, c] / hidden_size + eps), the
 * sum taken per lane over columns l, l+32, ... and then by a shuffle-down tree, as the reference. */
int fp4b200_row_rms_reduce(const float* row_rms_partial, int64_t M, int64_t partial_cols, int64_t hidden_size,
                           float eps, float* inv_rms, void* stream);

/* One group of tk_group_quantize_dim1_split3_for_gemm(input0, input1, input2, ...) (nvfp4_v5/tk_quantize.cu:6425-6835):
 * amax + quantisation of one [M, K] input whose row-wise codes go into a column slice of a wider code matrix
 * (row_fp4 points at the slice's first byte, row_pitch_bytes is the wide matrix's pitch); its column-wise codes are a
 * contiguous row block of the transposed matrix.  Per-group tensor amax, as the reference. */
int fp4b200_nvfp4_quantize_for_gemm_into(const void* x_bf16, int64_t M, int64_t K, int return_transpose, int encode_centric,
                                         void* row_fp4, int64_t row_pitch_bytes, void* row_sc, void* col_fp4, void* col_sc,
                                         float* amax_sg, void* stream);

/* tk_group_quantize_dim1_split3_for_gemm(input0, input1, input2) with round-to-nearest codes
 * (nvfp4_v5/tk_quantize.cu:6425-6835) in two launches: the three tensor maxima, then all three [M, n_g] inputs
 * quantised (encode-centric, each with its own amax) into the column slices of row_fp4_full [M, N/2] and the row blocks
 * of col_fp4_full [N, M/2], N = n0 + n1 + n2.  Row-wise scales go to one swizzled tensor per input
 * ([M/128, n_g/64, 512]); column-wise scales to the row blocks of col_sc_cat [N/128, M/64, 512], which is their
 * concatenation.  amax3[g] = tensor amax of input g, sg3[g] = amax3[g] / 2688.  Same bytes as one
 * fp4b200_nvfp4_quantize_for_gemm_into call per input. */
int fp4b200_nvfp4_quantize_split3_into(const void* x0, const void* x1, const void* x2, int64_t M, int64_t n0, int64_t n1,
                                       int64_t n2, void* row_fp4_full, void* row_sc0, void* row_sc1, void* row_sc2,
                                       void* col_fp4_full, void* col_sc_cat, float* amax3, float* sg3, void* stream);

/* tk_quantize_nhsd_wo_for_gemm(input, return_transpose, encode_centric) (nvfp4_v5/tk_quantize.cu:3006-3134):
 * the attention output in its native [B, H, S, D = 64] layout, quantised as the matrix [M = B*S, K = H*D] the
 * output projection consumes (element (b*S + s, h*64 + d) = input[b, h, s, d]) without a transposing copy.
 * Same bytes as fp4b200_nvfp4_quantize_for_gemm on the permuted tensor.  S % 128 == 0; outputs 16-byte aligned. */
int fp4b200_nvfp4_quantize_nhsd_wo(const void* x_bf16, int64_t B, int64_t H, int64_t S, int64_t D, int return_transpose,
                                   int encode_centric, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                   float* amax_sg, void* stream);

/* nvfp4_grouped_gemm_rope_live64 / _rope_packed_cat / _rope_packed_split (nvfp4_b200_gemm.cu:1338-1441; epilogue
 * nvfp4_rope_epilogue.cuh:104-161): the grouped GEMM of the fused QKV projection with the rotary embedding applied in
 * the epilogue to the output columns [0, rope_cols) (Q and K): after the accumulator has been multiplied by the tensor
 * scales (and, with round_input_bf16, rounded to bf16), neighbouring columns (2i, 2i+1) of token row r are rotated by
 * rope_cs[r mod rope_seq_len, (col mod rope_head_dim) / 2] = (cos, sin), then rounded to bf16.  Outputs as in
 * fp4b200_nvfp4_grouped_gemm (1 to 3 bf16 matrices split by column range, each a multiple of 256 wide);
 * rope_seq_len and rope_head_dim powers of two, rope_cs fp32 [rope_seq_len, rope_head_dim/2, 2].
 * silu_dim > 0 (the silu_dim argument of nvfp4_grouped_gemm and nvfp4_grouped_gemm_rope_live64, nvfp4_gemm.cuh:210-225):
 * x / (1 + __expf(-x)) on the scaled accumulator of the columns [0, silu_dim) before any rotation; rope_cs may then be
 * null (SiLU only). */
int fp4b200_nvfp4_grouped_gemm_rope(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                                    const float* B_sg_per_tile, int n_out, void* const* D, const int64_t* D_cols,
                                    const float* rope_cs, int64_t rope_seq_len, int64_t rope_head_dim, int64_t rope_cols,
                                    int round_input_bf16, int64_t silu_dim, int64_t M, int64_t N, int64_t K, void* stream);

/* nvfp4_forward_rope_packed_qk / nvfp4_inverse_rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out)
 * (nvfp4_b200_gemm.cu:1083-1218): rotary embedding (inverse != 0: its inverse, the backward of the attention side) of
 * contiguous bf16 Q [rows, q_dim] and K [rows, k_dim] in one launch; rope_cs fp32 [rope_seq_len, rope_head_dim/2, 2]. */
int fp4b200_rope_packed_qk(const void* q, const void* k, const float* rope_cs, int64_t rope_seq_len, int64_t rope_head_dim,
                           void* q_out, void* k_out, int64_t rows, int64_t q_dim, int64_t k_dim, int inverse, void* stream);

/* ---- RMSNorm backward behind the dgrad GEMMs ----------------------------------------------- */

/* sum3_rmsnorm_bwd_out(d0, d1, d2, input, norm_weight, inv_rms, d_sum, grad_input, dgamma_partials, dgamma)
 * (nvfp4_b200_gemm.cu:432-562; kernels :196-323 and :382-430): all matrices [M, K] bf16 row-major.
 *   d_sum      = bf16(bf16(d0 + d1) + d2)
 *   grad_input = bf16(inv * (d_sum*gamma - x*inv*mean)),  mean = sum_c(d_sum * (x*inv*gamma)) / K per row, summed in
 *                the order of the reference's 512-thread block (thread t: columns t, t+512, ...; cub block sum)
 *   dgamma_partials [ceil(M/256), K] fp32: per 256-row tile, rows accumulated in turn; dgamma [K] (fp32, or bf16
 *                when dgamma_is_bf16) = the tiles added in turn.  Deterministic: no atomics.
 * K a multiple of 256, at most 8192 (the reference takes any K).  Outputs must not overlap inputs or each other. */
int fp4b200_sum3_rmsnorm_bwd(const void* d0, const void* d1, const void* d2, const void* input, const void* norm_weight,
                             const float* inv_rms, void* d_sum, void* grad_input, float* dgamma_partials, void* dgamma,
                             int dgamma_is_bf16, int64_t M, int64_t K, void* stream);

/* rmsnorm_bwd_residual_out(d_normed, input, norm_weight, inv_rms, residual_grad, grad_input, dgamma)
 * (nvfp4_b200_gemm.cu:564-646; kernel :325-380): K = 4096 only, as the reference.
 *   grad_input = bf16(bf16(dx) + residual_grad), dx as above with the reference's 256-thread block order.
 *   dgamma [K] fp32 = sum over rows of d_normed * (x*inv).  The reference adds these with atomics in no fixed
 *                order; here they go through the same 256-row tiles as above, which needs the scratch
 *                dgamma_partials [ceil(M/256), K] fp32 from the caller and makes the result reproducible. */
int fp4b200_rmsnorm_bwd_residual(const void* d_normed, const void* input, const void* norm_weight, const float* inv_rms,
                                 const void* residual_grad, void* grad_input, float* dgamma_partials, float* dgamma,
                                 int64_t M, int64_t K, void* stream);

/* fp32_to_fp4x2(A_fp32) / fp4x2_to_fp32(A_fp4x2) of the reference GEMM module (nvfp4_b200_gemm.cu:1480-1510;
 * kernels nvfp4_quantize.cuh:293-308): element 2i in the low nibble, RN-even, saturating. */
int fp4b200_fp32_to_fp4x2(const float* in_f32, int64_t n_pairs, void* out_fp4x2, void* stream);
int fp4b200_fp4x2_to_fp32(const void* in_fp4x2, int64_t n_bytes, float* out_f32, void* stream);

/* nvfp4_quantize(A_bf16, A_fp4x2, A_sc, A_sc_global, scale_2d) of the reference GEMM module
 * (nvfp4_b200_gemm.cu:1443-1478; kernels nvfp4_quantize.cuh:57-255): A_sc_global = amax / (6*448);
 * block scale e4m3(b / 6 * (1 / max(A_sc_global, 1e-12))); codes e2m1(x / max(float(scale) * A_sc_global, 1e-12));
 * scale_2d shares one scale per 16x16 tile.  Scale tiles [M/128, N/64, 512]. */
int fp4b200_tk_nvfp4_quantize(const void* A_bf16, int64_t M, int64_t N, void* A_fp4x2, void* A_sc,
                              float* A_sc_global, int scale_2d, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FP4B200_H_ */
