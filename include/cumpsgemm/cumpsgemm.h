/* C ABI of the B200 (sm_100a) cuMpSGEMM library.
 *
 * Every entry point here replaces the identically named entry point of the
 * reference (include/cumpsgemm/cumpsgemm.h:7-57, implemented in
 * src/handle.cu:7-52 and src/cumpsgemm.cu:549-605).  Prototypes are identical
 * so that a program or binding written against the reference links or
 * dlopens this library unchanged:
 *   - all matrices are column-major and live in device memory,
 *   - alpha / beta are read from host memory at call time,
 *   - sizes, leading dimensions and strides are counted in elements of the
 *     matrix type (float or cuComplex), as 64-bit unsigned integers,
 *   - work is enqueued on the handle's stream and the call returns without
 *     synchronising.
 */
#ifndef CUMPSGEMM_B200_CUMPSGEMM_H
#define CUMPSGEMM_B200_CUMPSGEMM_H
#include "detail/common.h"
#include <cublas_v2.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Reference: cuMpSGEMM_create, src/handle.cu:7-38.  Allocates the handle, the
 * exponent-statistics and dynamic-launch ring buffers on the current device. */
cublasStatus_t cuMpSGEMM_create(cuMpSGEMM_handle_t *const handle);

/* Reference: cuMpSGEMM_destroy, src/handle.cu:40-46.  Also releases the
 * operand workspace (the reference leaks its workspace). */
cublasStatus_t cuMpSGEMM_destroy(cuMpSGEMM_handle_t handle);

/* Reference: cuMpSGEMM_set_stream, src/handle.cu:48-52. */
cublasStatus_t cuMpSGEMM_set_stream(cuMpSGEMM_handle_t handle,
                                    const cudaStream_t cuda_stream);

/* Reference: src/cumpsgemm_cublas.cu:163-196.  Static string, never NULL. */
const char *cuMpSGEMM_get_compute_mode_string(const cuMpSGEMM_compute_mode_t mode);

/* User-replaceable rule (libcumpsgemm_rule.so).  Reference declaration:
 * include/cumpsgemm/cumpsgemm.h:18-21; default body:
 * src/default_cumpsgemm_rule.cu:6-49. */
cuMpSGEMM_compute_mode_t cuMpSGEMM_get_compute_mode(
    const char *const func_name, cublasHandle_t const cublas_handle,
    const cublasOperation_t op_A, const cublasOperation_t op_B,
    const unsigned m, const unsigned n, const unsigned k);

/* C = alpha * op(A) * op(B) + beta * C, FP32.  Reference: src/cumpsgemm.cu:550-563.
 * op_A / op_B must not be CUBLAS_OP_C (returns CUBLAS_STATUS_INVALID_VALUE where
 * the reference asserts). */
cublasStatus_t cuMpSGEMM_sgemm(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
    const uint64_t k, const float *alpha, const float *const a_dmem_ptr,
    const uint64_t lda, const float *const b_dmem_ptr, const uint64_t ldb,
    const float *beta, float *const c_dmem_ptr, const uint64_t ldc,
    const cuMpSGEMM_compute_mode_t compute_mode);

/* Complex64 GEMM (four real products).  Reference: src/cumpsgemm.cu:565-576. */
cublasStatus_t cuMpSGEMM_cgemm(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
    const uint64_t k, const cuComplex *alpha, const cuComplex *const a_dmem_ptr,
    const uint64_t lda, const cuComplex *const b_dmem_ptr, const uint64_t ldb,
    const cuComplex *beta, cuComplex *const c_dmem_ptr, const uint64_t ldc,
    const cuMpSGEMM_compute_mode_t compute_mode);

/* Strided-batch FP32 GEMM.  Reference: src/cumpsgemm.cu:578-591. */
cublasStatus_t cuMpSGEMM_sgemm_strided_batch(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
    const uint64_t k, const float *alpha, const float *const a_dmem_ptr,
    const uint64_t lda, const uint64_t stridea, const float *const b_dmem_ptr,
    const uint64_t ldb, const uint64_t strideb, const float *beta,
    float *const c_dmem_ptr, const uint64_t ldc, const uint64_t stridec,
    const uint64_t batch_count, const cuMpSGEMM_compute_mode_t compute_mode);

/* Strided-batch complex64 GEMM.  Reference: src/cumpsgemm.cu:593-604. */
cublasStatus_t cuMpSGEMM_cgemm_strided_batch(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
    const uint64_t k, const cuComplex *alpha, const cuComplex *const a_dmem_ptr,
    const uint64_t lda, const uint64_t stridea,
    const cuComplex *const b_dmem_ptr, const uint64_t ldb,
    const uint64_t strideb, const cuComplex *beta, cuComplex *const c_dmem_ptr,
    const uint64_t ldc, const uint64_t stridec, const uint64_t batch_count,
    const cuMpSGEMM_compute_mode_t compute_mode);

#ifdef __cplusplus
}
#endif
#endif
