// C++ API of the B200 cuMpSGEMM library.
//
// Same namespace, names, argument order and defaults as the reference's
// include/cumpsgemm/cumpsgemm.hpp:8-129, so sources written against the
// reference compile unchanged.  T is float or cuComplex; explicit
// instantiations for both live in the library.
#ifndef CUMPSGEMM_B200_CUMPSGEMM_HPP
#define CUMPSGEMM_B200_CUMPSGEMM_HPP
#include "cumpsgemm.h"
#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace cumpsgemm {
using handle_t = cuMpSGEMM_handle_t;
inline void create(handle_t &handle) { cuMpSGEMM_create(&handle); }
inline void destroy(handle_t handle) { cuMpSGEMM_destroy(handle); }
inline void set_stream(handle_t &handle, cudaStream_t cuda_stream) {
  cuMpSGEMM_set_stream(handle, cuda_stream);
}

// Reference: src/cumpsgemm.cu:228-419.  used_kernel_module_id receives the
// index of the tile configuration chosen (0 = 128x256, 1 = 128x128,
// 2 = 128x64); AUTO reports the configuration shared by both gated launches.
template <class T>
cublasStatus_t gemm(cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
                    const cublasOperation_t op_B, const uint64_t m,
                    const uint64_t n, const uint64_t k, const T *alpha,
                    const T *const a_dmem_ptr, const uint64_t lda,
                    const T *const b_dmem_ptr, const uint64_t ldb,
                    const T *beta, T *const c_dmem_ptr, const uint64_t ldc,
                    const cuMpSGEMM_compute_mode_t compute_mode,
                    unsigned *const used_kernel_module_id = nullptr);

// Reference: src/cumpsgemm.cu:421-547.
template <class T>
cublasStatus_t gemm_stridedBatch(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
    const uint64_t k, const T *alpha, const T *const a_dmem_ptr,
    const uint64_t lda, const uint64_t stridea, const T *const b_dmem_ptr,
    const uint64_t ldb, const uint64_t strideb, const T *beta,
    T *const c_dmem_ptr, const uint64_t ldc, const uint64_t stridec,
    const uint64_t batch_count, const cuMpSGEMM_compute_mode_t compute_mode,
    unsigned *const used_kernel_module_id = nullptr);

// ---- exponent statistics (reference: src/exp_stats.cu:502-564, 607-646) ----
// Each call takes the next ring slot and returns its id.
template <class T>
unsigned exp_stats_ext(cuMpSGEMM_handle_t handle, const unsigned m,
                       const unsigned n, const T *const ptr, const unsigned ld,
                       const unsigned batch_size = 1,
                       const unsigned stride = 0);

template <class T>
unsigned exp_max_ext(cuMpSGEMM_handle_t handle, const unsigned m,
                     const unsigned n, const T *const ptr, const unsigned ld,
                     const unsigned batch_size = 1, const unsigned stride = 0);

// {underflow count, total count}, in that order (reference: src/exp_stats.cu:628).
std::pair<std::size_t, std::size_t> get_exp_stats(cuMpSGEMM_handle_t handle,
                                                  const unsigned buffer_id);

unsigned get_current_exp_stats_buffer_id(cuMpSGEMM_handle_t handle);

void reset_exp_stats_buffer_id(cuMpSGEMM_handle_t handle);

void set_exp_stats_params(cuMpSGEMM_handle_t handle,
                          const float ignore_threshold,
                          const float underflow_threshold,
                          const float underflow_ratio_tolerance);

void enable_exp_stats(cuMpSGEMM_handle_t handle);

void disable_exp_stats(cuMpSGEMM_handle_t handle);

// Power of two 2^floor(log2 max|x|) recorded in a statistics slot
// (reference: src/dynamic_scaling.cu:352-361).  Synchronises the stream.
float get_max_exp(cuMpSGEMM_handle_t handle, const unsigned buffer_id);

cuMpSGEMM_compute_mode_t
get_exp_stats_compute_mode_level(cuMpSGEMM_handle_t handle,
                                 const unsigned buffer_id);

// ---- dynamic scaling (reference: src/dynamic_scaling.cu:152-350) ----
// In-place multiplication by an exact power of two, gated by the flag word
// in dynamic-launch slot `dynamic_launch_flag_buffer_id`.
template <class T>
void scale_A(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
             const unsigned dynamic_launch_flag_buffer_id, const unsigned m,
             const unsigned n, T *const ptr, const unsigned ld,
             const unsigned batch_size = 1, const unsigned stride = 0);
template <class T>
void scale_B(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
             const unsigned dynamic_launch_flag_buffer_id, const unsigned m,
             const unsigned n, T *const ptr, const unsigned ld,
             const unsigned batch_size = 1, const unsigned stride = 0);
template <class T>
void scale_C(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_A_id,
             const unsigned exp_stats_buffer_B_id,
             const unsigned dynamic_launch_flag_buffer_id, const unsigned m,
             const unsigned n, T *const ptr, const unsigned ld,
             const unsigned batch_size = 1, const unsigned stride = 0);
template <class T>
void reset_scale_A(cuMpSGEMM_handle_t handle,
                   const unsigned exp_stats_buffer_id,
                   const unsigned dynamic_launch_flag_buffer_id,
                   const unsigned m, const unsigned n, T *const ptr,
                   const unsigned ld, const unsigned batch_size = 1,
                   const unsigned stride = 0);
template <class T>
void reset_scale_B(cuMpSGEMM_handle_t handle,
                   const unsigned exp_stats_buffer_id,
                   const unsigned dynamic_launch_flag_buffer_id,
                   const unsigned m, const unsigned n, T *const ptr,
                   const unsigned ld, const unsigned batch_size = 1,
                   const unsigned stride = 0);

// ---- dynamic launch (reference: src/dynamic_launch.cu:36-70,
//      src/cumpsgemm.cu:776-812) ----
unsigned get_current_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle);
unsigned get_next_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle);
cuMpSGEMM_compute_mode_t
get_dynamic_launch_gemm_compute_mode(cuMpSGEMM_handle_t handle,
                                     const unsigned buffer_id);
std::pair<int, int>
get_dynamic_launch_scaling_mode_AB(cuMpSGEMM_handle_t handle,
                                   const unsigned buffer_id);
void set_dynamic_launch_buffer_by_exp_stats(
    cuMpSGEMM_handle *handle, const unsigned dynamic_launch_buffer_id,
    const unsigned A_exp_stats_buffer_id, const unsigned B_exp_stats_buffer_id);

// ---- named timers around the statistics / scaling / GEMM launches
//      (reference: src/cumpsgemm.cu:814-849).  Timer names are kept:
//      "exp_stats_init", "exp_stats_1", "exp_stats_set_1", "exp_stats_2",
//      "exp_stats_set_2", "exp_max_init", "exp_max", "scaling_AB",
//      "scaling_C", "gemm_kernel". ----
void enable_exp_stats_profiling(cuMpSGEMM_handle *const handle);
void disable_exp_stats_profiling(cuMpSGEMM_handle *const handle);
void reset_exp_stats_profiling(cuMpSGEMM_handle *const handle);
void print_exp_stats_profiling(cuMpSGEMM_handle *const handle,
                               unsigned csv = false);

namespace debug {
struct stats_t {
  double time_sum; // seconds
  std::uint64_t n;
};
std::unordered_map<std::string, stats_t>
get_exp_stats_profiling_result(cuMpSGEMM_handle *const handle);
} // namespace debug
} // namespace cumpsgemm
#endif
