/* Plain-C entry points for the parts of the reference API that exist only as
 * C++ (namespace cumpsgemm, include/cumpsgemm/cumpsgemm.hpp:45-129, and
 * namespace cumpsgemm::hijack_control, include/cumpsgemm/hijack_control.hpp:7-34),
 * so that ctypes / cgo / JNI style bindings can reach them without C++ name
 * mangling.  Suffix _s = float, _c = cuComplex.  Every function forwards to
 * the C++ function named in its comment; argument meaning is identical.
 *
 * The last section adds what a multi-GPU caller needs to make the AUTO /
 * FP16TCEC_SCALING decisions global across ranks; it has no counterpart in
 * the reference, which is single-GPU.
 */
#ifndef CUMPSGEMM_B200_CUMPSGEMM_EXT_H
#define CUMPSGEMM_B200_CUMPSGEMM_EXT_H
#include "cumpsgemm.h"
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- exponent statistics ------------------------------------------------ */
/* cumpsgemm::exp_stats_ext<T>  (reference: src/exp_stats.cu:502-525) */
unsigned cuMpSGEMM_exp_stats_ext_s(cuMpSGEMM_handle_t handle, unsigned m, unsigned n,
                                   const float *ptr, unsigned ld, unsigned batch_size,
                                   unsigned stride);
unsigned cuMpSGEMM_exp_stats_ext_c(cuMpSGEMM_handle_t handle, unsigned m, unsigned n,
                                   const cuComplex *ptr, unsigned ld, unsigned batch_size,
                                   unsigned stride);
/* cumpsgemm::exp_max_ext<T>  (reference: src/exp_stats.cu:534-557) */
unsigned cuMpSGEMM_exp_max_ext_s(cuMpSGEMM_handle_t handle, unsigned m, unsigned n,
                                 const float *ptr, unsigned ld, unsigned batch_size,
                                 unsigned stride);
unsigned cuMpSGEMM_exp_max_ext_c(cuMpSGEMM_handle_t handle, unsigned m, unsigned n,
                                 const cuComplex *ptr, unsigned ld, unsigned batch_size,
                                 unsigned stride);
/* cumpsgemm::get_exp_stats  (reference: src/exp_stats.cu:615-629).  Synchronises. */
void cuMpSGEMM_get_exp_stats(cuMpSGEMM_handle_t handle, unsigned buffer_id,
                             size_t *underflow_count, size_t *total_count);
/* cumpsgemm::get_current_exp_stats_buffer_id / reset_exp_stats_buffer_id */
unsigned cuMpSGEMM_get_current_exp_stats_buffer_id(cuMpSGEMM_handle_t handle);
void cuMpSGEMM_reset_exp_stats_buffer_id(cuMpSGEMM_handle_t handle);
/* cumpsgemm::set_exp_stats_params  (reference: src/exp_stats.cu:631-638) */
void cuMpSGEMM_set_exp_stats_params(cuMpSGEMM_handle_t handle, float ignore_threshold,
                                    float underflow_threshold, float underflow_ratio_tolerance);
/* cumpsgemm::enable_exp_stats / disable_exp_stats */
void cuMpSGEMM_enable_exp_stats(cuMpSGEMM_handle_t handle);
void cuMpSGEMM_disable_exp_stats(cuMpSGEMM_handle_t handle);
/* cumpsgemm::get_max_exp  (reference: src/dynamic_scaling.cu:352-361).  Synchronises. */
float cuMpSGEMM_get_max_exp(cuMpSGEMM_handle_t handle, unsigned buffer_id);
/* cumpsgemm::get_exp_stats_compute_mode_level  (reference: src/exp_stats.cu:675-683) */
int cuMpSGEMM_get_exp_stats_compute_mode_level(cuMpSGEMM_handle_t handle, unsigned buffer_id);

/* ---- dynamic scaling (reference: src/dynamic_scaling.cu:227-350) --------- */
void cuMpSGEMM_scale_A_s(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                         unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                         float *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_scale_A_c(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                         unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                         cuComplex *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_scale_B_s(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                         unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                         float *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_scale_B_c(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                         unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                         cuComplex *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_scale_C_s(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_A_id,
                         unsigned exp_stats_buffer_B_id, unsigned dynamic_launch_flag_buffer_id,
                         unsigned m, unsigned n, float *ptr, unsigned ld, unsigned batch_size,
                         unsigned stride);
void cuMpSGEMM_scale_C_c(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_A_id,
                         unsigned exp_stats_buffer_B_id, unsigned dynamic_launch_flag_buffer_id,
                         unsigned m, unsigned n, cuComplex *ptr, unsigned ld, unsigned batch_size,
                         unsigned stride);
void cuMpSGEMM_reset_scale_A_s(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                               unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                               float *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_reset_scale_A_c(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                               unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                               cuComplex *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_reset_scale_B_s(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                               unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                               float *ptr, unsigned ld, unsigned batch_size, unsigned stride);
void cuMpSGEMM_reset_scale_B_c(cuMpSGEMM_handle_t handle, unsigned exp_stats_buffer_id,
                               unsigned dynamic_launch_flag_buffer_id, unsigned m, unsigned n,
                               cuComplex *ptr, unsigned ld, unsigned batch_size, unsigned stride);

/* ---- dynamic launch (reference: src/dynamic_launch.cu:36-70,
 *      src/cumpsgemm.cu:776-812) ------------------------------------------ */
unsigned cuMpSGEMM_get_current_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle);
unsigned cuMpSGEMM_get_next_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle);
int cuMpSGEMM_get_dynamic_launch_gemm_compute_mode(cuMpSGEMM_handle_t handle, unsigned buffer_id);
void cuMpSGEMM_get_dynamic_launch_scaling_mode_AB(cuMpSGEMM_handle_t handle, unsigned buffer_id,
                                                  int *scale_A, int *scale_B);
void cuMpSGEMM_set_dynamic_launch_buffer_by_exp_stats(cuMpSGEMM_handle_t handle,
                                                      unsigned dynamic_launch_buffer_id,
                                                      unsigned A_exp_stats_buffer_id,
                                                      unsigned B_exp_stats_buffer_id);
/* cumpsgemm::dynamic_launch::set_/unset_dynamic_launch_flag_buffer_id
 * (reference: src/dynamic_launch.cu:60-70): selects the flag slot a following
 * gemm(..., CUMPSGEMM_AUTO) call is gated by. */
void cuMpSGEMM_set_dynamic_launch_flag_buffer_id(cuMpSGEMM_handle_t handle, unsigned id);
void cuMpSGEMM_unset_dynamic_launch_flag_buffer_id(cuMpSGEMM_handle_t handle);

/* ---- timers (reference: src/cumpsgemm.cu:814-849) ------------------------ */
void cuMpSGEMM_enable_exp_stats_profiling(cuMpSGEMM_handle_t handle);
void cuMpSGEMM_disable_exp_stats_profiling(cuMpSGEMM_handle_t handle);
void cuMpSGEMM_reset_exp_stats_profiling(cuMpSGEMM_handle_t handle);
void cuMpSGEMM_print_exp_stats_profiling(cuMpSGEMM_handle_t handle, unsigned csv);
/* cumpsgemm::debug::get_exp_stats_profiling_result for one timer name; returns 0 when the
 * timer never ran. */
int cuMpSGEMM_get_exp_stats_profiling_result(cuMpSGEMM_handle_t handle, const char *name,
                                             double *time_sum_s, unsigned long long *n);

/* ---- gemm variants reporting the tile configuration used ----------------- */
/* cumpsgemm::gemm<T> / gemm_stridedBatch<T> with their used_kernel_module_id out-parameter
 * (reference: include/cumpsgemm/cumpsgemm.hpp:18-43). */
cublasStatus_t cuMpSGEMM_sgemm_module(
    cuMpSGEMM_handle_t handle, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m,
    uint64_t n, uint64_t k, const float *alpha, const float *a, uint64_t lda, const float *b,
    uint64_t ldb, const float *beta, float *c, uint64_t ldc, cuMpSGEMM_compute_mode_t mode,
    unsigned *used_kernel_module_id);

/* ---- kernel status -------------------------------------------------------- */
/* Every wait inside the GEMM kernel is bounded; a wait that gives up records a non-zero
 * code in a device word.  This call synchronises the handle's stream, returns the word and
 * clears it.  0 = no error; 1 = a producer / converter waited for a free stage, 2 = the MMA
 * issuer for operands, 3 / 7 = the MMA issuer for the drain of an accumulator, 4 / 5 = the
 * epilogue for an accumulator, 6 = bad launch, 8 = the epilogue warps of a CTA for one another
 * (tail split of the CTA-pair kernel). */
int cuMpSGEMM_get_kernel_status(cuMpSGEMM_handle_t handle);
/* Self-test of the bounded wait: a one-CTA kernel waits, with the same routine the GEMM kernels
 * use, on a barrier that nothing signals; after limit_ms it must give up, record its code and
 * return normally.  Returns the status word (expected: 2, the "waited for operands" code) and
 * the time the wait took.  The context stays usable; nothing faults. */
int cuMpSGEMM_selftest_bounded_wait(cuMpSGEMM_handle_t handle, unsigned limit_ms,
                                    double *waited_ms);
/* Cap (bytes) for the operand workspace a strided-batch call may use at once; batches beyond
 * it are processed in chunks.  0 restores the default (8 GiB). */
void cuMpSGEMM_set_workspace_limit(cuMpSGEMM_handle_t handle, size_t bytes);
/* Compatibility switch for the exponent statistics (off by default; also set by the
 * environment variable CUMPSGEMM_COUNT_TAIL_PADDING=1 at handle creation).  The reference's
 * counting kernels walk a matrix four elements at a time and, when m*n is not a multiple of
 * 4, append zeros to the last group and count them like data
 * (reference: src/exp_stats.cu:101-116 and :222-238).  With the switch on, exp_stats_ext
 * adds the same (4 - m*n % 4) % 4 zero elements per matrix to `total` (and to `underflow`
 * when 0 is below the stage's threshold), so counts and decisions equal the reference's for
 * such shapes too; with it off only real matrix elements are counted. */
void cuMpSGEMM_set_count_tail_padding(cuMpSGEMM_handle_t handle, int enable);
/* A handle reads the tuning variables (CUMPSGEMM_TILE_N, CUMPSGEMM_PAIR, CUMPSGEMM_DRAIN_CHUNK,
 * CUMPSGEMM_FIRST_CHUNK, CUMPSGEMM_PACE, CUMPSGEMM_FUSED, CUMPSGEMM_SPLIT_K,
 * CUMPSGEMM_TAIL_SPLIT) once, when it is created, so that a GEMM call does not query the
 * environment; this reads them again. */
void cuMpSGEMM_reload_tuning_env(cuMpSGEMM_handle_t handle);
/* Host-only query (no GPU needed): how the CTA-pair kernel would schedule `total_tiles` tiles
 * of 256 x 256 with a K loop of k_pad values (a multiple of 64; tf32 != 0 for the TF32 kinds) on
 * `clusters` CTA pairs.  Tiles [0, *split_begin) run whole; each later tile (the last, partly
 * filled wave) is cut into *slices K slices of *slice_k values, *work_items work items in
 * all.  *slices == 1: nothing is cut.  Returns 0, or 1 for invalid arguments.  No counterpart
 * in the reference (its atomic split-K kernel, src/cumpsgemm.cu:272-304, is the nearest
 * relative). */
int cuMpSGEMM_plan_pair_tail(unsigned total_tiles, unsigned clusters, unsigned k_pad, int tf32,
                             unsigned *split_begin, unsigned *slices, unsigned *slice_k,
                             unsigned *work_items);
/* Per-launch device timing with CUDA events on the handle's stream (off by default).  While
 * enabled every split + GEMM launch group records three events; get_kernel_timing
 * synchronises the stream, returns the number of launch groups since the last query and the
 * summed durations of the split passes and of the GEMM kernels, and clears the record.
 * In AUTO mode both gated kinds are recorded, the deselected one with near-zero time. */
/* Optional stall breakdown of the GEMM kernels: eight 64-bit words in device memory that the
 * kernels add to (cycles the MMA issuer waited for operands [0] and for the accumulator drain
 * [1], the TMA producer for a free stage [2], one drain warp for a finished chunk [3], MMA
 * loop cycles [4], contributing CTAs [5]).  NULL (default) disables it. */
void cuMpSGEMM_set_debug_buffer(cuMpSGEMM_handle_t handle, unsigned long long *dev_words8);
void cuMpSGEMM_set_kernel_timing(cuMpSGEMM_handle_t handle, int enable);
unsigned long long cuMpSGEMM_get_kernel_timing(cuMpSGEMM_handle_t handle, double *split_ms,
                                               double *gemm_ms);

/* ---- interception-layer control (cumpsgemm::hijack_control, reference:
 *      src/cumpsgemm_cublas.cu:1189-1271) ---------------------------------- */
cuMpSGEMM_handle_t cuMpSGEMM_hijack_get_internal_global_handle(void);
/* returns 0, or 1 if the mode is rejected (CUMPSGEMM_FP32_SIMT; the C++ function throws) */
int cuMpSGEMM_hijack_set_compute_mode(int mode);
void cuMpSGEMM_hijack_unset_compute_mode(void);
void cuMpSGEMM_hijack_reset_exp_stats_buffer_id(void);
void cuMpSGEMM_hijack_set_exp_stats_params(float ignore_threshold, float underflow_threshold,
                                           float underflow_tolerance_rate);
void cuMpSGEMM_hijack_enable_restoring_AB_after_scaling(void);
void cuMpSGEMM_hijack_disable_restoring_AB_after_scaling(void);
/* copies at most size-1 characters and NUL-terminates; returns the full length */
size_t cuMpSGEMM_hijack_get_last_called_function_str(char *buf, size_t size);
void cuMpSGEMM_hijack_set_last_called_function_str(const char *str);
void cuMpSGEMM_hijack_clear_last_called_function_str(void);
void cuMpSGEMM_hijack_enable_custom_gemm_Mx2x2(void);
void cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2(void);
int cuMpSGEMM_hijack_is_library_loaded(void);
/* C callback form of hijack_control::set_control_function; NULL unsets. */
typedef int (*cuMpSGEMM_control_function_c_t)(int op_A, int op_B, unsigned m, unsigned n,
                                              unsigned k);
void cuMpSGEMM_hijack_set_control_function(cuMpSGEMM_control_function_c_t fn);
/* The mode the rule chain would pick for a call (control function, then
 * libcumpsgemm_rule.so, then the built-in default).  Reference:
 * cuMpSGEMM_get_compute_mode_internal, src/cumpsgemm_cublas.cu:198-220. */
cuMpSGEMM_compute_mode_t cuMpSGEMM_get_compute_mode_internal(
    const char *const func_name, cublasHandle_t const cublas_handle,
    const cublasOperation_t op_A, const cublasOperation_t op_B, const unsigned m,
    const unsigned n, const unsigned k);

/* ---- multi-GPU support: staged statistics and a GEMM that takes decided
 *      statistics slots.  No counterpart in the reference. ------------------ */
/* Take the next statistics slot and zero it. */
unsigned cuMpSGEMM_exp_stats_begin(cuMpSGEMM_handle_t handle);
/* stage: 1 = max exponent + absolute-threshold counts, 2 = relative-threshold recount
 * (runs on the device only if decision 1 left the slot undecided),
 * 3 = max exponent only. */
void cuMpSGEMM_exp_stats_stage_s(cuMpSGEMM_handle_t handle, int stage, unsigned id, unsigned m,
                                 unsigned n, const float *ptr, unsigned ld, unsigned batch_size,
                                 unsigned stride);
void cuMpSGEMM_exp_stats_stage_c(cuMpSGEMM_handle_t handle, int stage, unsigned id, unsigned m,
                                 unsigned n, const cuComplex *ptr, unsigned ld,
                                 unsigned batch_size, unsigned stride);
/* decision: 1 or 2 (reference: src/exp_stats.cu:169-184, :277-293). */
void cuMpSGEMM_exp_stats_decide(cuMpSGEMM_handle_t handle, int decision, unsigned id);
/* Copy a slot to / from four 64-bit words in device memory:
 * {max exponent bits, total, underflow, mode}.  Ranks all-reduce words 0 (max) and
 * 1..2 (sum) between a stage and its decision. */
void cuMpSGEMM_exp_stats_export(cuMpSGEMM_handle_t handle, unsigned id,
                                unsigned long long *dev_words4);
void cuMpSGEMM_exp_stats_import(cuMpSGEMM_handle_t handle, unsigned id,
                                const unsigned long long *dev_words4);
/* Strided-batch GEMM whose scaling / kind selection comes from statistics slots that were
 * already decided (by the calls above).  mode is CUMPSGEMM_AUTO (flag slot derived from the
 * two statistics slots) or CUMPSGEMM_FP16TCEC_SCALING (both operands scaled). */
cublasStatus_t cuMpSGEMM_sgemm_strided_batch_with_stats(
    cuMpSGEMM_handle_t handle, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m,
    uint64_t n, uint64_t k, const float *alpha, const float *a, uint64_t lda, uint64_t stridea,
    const float *b, uint64_t ldb, uint64_t strideb, const float *beta, float *c, uint64_t ldc,
    uint64_t stridec, uint64_t batch_count, cuMpSGEMM_compute_mode_t mode, unsigned stats_id_a,
    unsigned stats_id_b);
cublasStatus_t cuMpSGEMM_cgemm_strided_batch_with_stats(
    cuMpSGEMM_handle_t handle, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m,
    uint64_t n, uint64_t k, const cuComplex *alpha, const cuComplex *a, uint64_t lda,
    uint64_t stridea, const cuComplex *b, uint64_t ldb, uint64_t strideb, const cuComplex *beta,
    cuComplex *c, uint64_t ldc, uint64_t stridec, uint64_t batch_count,
    cuMpSGEMM_compute_mode_t mode, unsigned stats_id_a, unsigned stats_id_b);

/* ---- two-by-two inner problems ------------------------------------------- */
/* C = alpha op(A) op(B) + beta C in plain FP32 for the shapes the reference hands to the
 * third-party cuGEMM-Mx2x2 kernels (src/cumpsgemm_cublas.cu:269-338, :647-725):
 *   *_Mx2x2: op(A) is m x 2, op(B) is 2 x 2, C is m x 2;
 *   *_2xNx2: op(A) is 2 x 2, op(B) is 2 x n, C is 2 x n;
 * m resp. n a power of two (anything else returns CUBLAS_STATUS_INVALID_VALUE).  Column-major
 * device pointers, host alpha / beta, leading dimensions and batch strides in elements;
 * batch_count == 1 with any strides is the single GEMM.  The interception layer takes this
 * route for such shapes when CUMPSGEMM_CUSTOM_GEMM_MX2X2=1 or after
 * hijack_control::enable_custom_gemm_Mx2x2(), whatever the compute mode, as the reference
 * does. */
cublasStatus_t cuMpSGEMM_sgemm_Mx2x2(cuMpSGEMM_handle_t handle, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t m, const float *alpha,
                                     const float *a, uint64_t lda, uint64_t stridea,
                                     const float *b, uint64_t ldb, uint64_t strideb,
                                     const float *beta, float *c, uint64_t ldc, uint64_t stridec,
                                     uint64_t batch_count);
cublasStatus_t cuMpSGEMM_cgemm_Mx2x2(cuMpSGEMM_handle_t handle, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t m, const cuComplex *alpha,
                                     const cuComplex *a, uint64_t lda, uint64_t stridea,
                                     const cuComplex *b, uint64_t ldb, uint64_t strideb,
                                     const cuComplex *beta, cuComplex *c, uint64_t ldc,
                                     uint64_t stridec, uint64_t batch_count);
cublasStatus_t cuMpSGEMM_sgemm_2xNx2(cuMpSGEMM_handle_t handle, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t n, const float *alpha,
                                     const float *a, uint64_t lda, uint64_t stridea,
                                     const float *b, uint64_t ldb, uint64_t strideb,
                                     const float *beta, float *c, uint64_t ldc, uint64_t stridec,
                                     uint64_t batch_count);
cublasStatus_t cuMpSGEMM_cgemm_2xNx2(cuMpSGEMM_handle_t handle, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t n, const cuComplex *alpha,
                                     const cuComplex *a, uint64_t lda, uint64_t stridea,
                                     const cuComplex *b, uint64_t ldb, uint64_t strideb,
                                     const cuComplex *beta, cuComplex *c, uint64_t ldc,
                                     uint64_t stridec, uint64_t batch_count);

/* ---- allocation-free FP32 GEMM ------------------------------------------- */
/* No counterpart in the reference.  For callers that may not allocate device memory (a
 * process whose memory budget is fixed at start-up, a loop that cannot take the device
 * synchronisation cudaMalloc / cudaFree imply, code without a handle): same arithmetic as
 * cuMpSGEMM_sgemm in FP16TCEC or TF32TCEC mode, but the split operand panels live in a 32 MiB
 * array built into the library instead of a workspace obtained with cudaMalloc, and no handle
 * is needed.  The call issues kernel launches on `stream` and nothing else.
 *   - Problems whose panels exceed 32 MiB return CUBLAS_STATUS_INVALID_VALUE with an error
 *     line and launch nothing.  FP16TCEC panels take 4*(round_up(m,tile_m)+round_up(n,tile_n))*
 *     round_up(k,64) bytes, TF32TCEC twice that, where tile_m x tile_n is the tile the library
 *     picks for the shape (256 x 256 with the CTA-pair kernel, else 128 x 256/128/64; the
 *     CUMPSGEMM_TILE_N / CUMPSGEMM_PAIR overrides count).  Whatever the tile,
 *     4*(round_up(m,256)+round_up(n,256))*round_up(k,64) <= 32 MiB always fits (FP16TCEC;
 *     m=n=k=2048 fits exactly).
 *   - The first call on a device resolves the array's device address and configures the
 *     kernels; issue it before any stream capture on that device.
 *   - The array is shared by all calls on a GPU: calls that overlap in time on one GPU race.
 *     Each call rewrites all of the region it reads, so no clearing is needed between calls.
 *   - alpha / beta are host pointers; op C is rejected; no status word is kept (waits inside
 *     the kernel remain bounded). */
cublasStatus_t cuMpSGEMM_sgemm_static_scratch(
    cudaStream_t stream, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m, uint64_t n,
    uint64_t k, const float *alpha, const float *a, uint64_t lda, const float *b, uint64_t ldb,
    const float *beta, float *c, uint64_t ldc, cuMpSGEMM_compute_mode_t compute_mode);

#ifdef __cplusplus
}
#endif
#endif
