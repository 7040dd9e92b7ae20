// extern "C" forwarding layer declared in include/cumpsgemm/cumpsgemm_ext.h.
#include "internal.hpp"

#include <cstring>
#include <cumpsgemm/cumpsgemm_ext.h>
#include <cumpsgemm/hijack_control.hpp>
#include <stdexcept>

using namespace cumpsgemm_b200;

namespace {
__global__ void export_slot_kernel(unsigned long long *out, const float *mx,
                                   const unsigned long long *total,
                                   const unsigned long long *uf, const int *mode) {
  out[0] = __float_as_uint(*mx);
  out[1] = *total;
  out[2] = *uf;
  out[3] = static_cast<unsigned long long>(*mode);
}
__global__ void import_slot_kernel(const unsigned long long *in, float *mx,
                                   unsigned long long *total, unsigned long long *uf, int *mode) {
  *mx = __uint_as_float(static_cast<unsigned int>(in[0]));
  *total = in[1];
  *uf = in[2];
  *mode = static_cast<int>(in[3]);
}

template <class T>
cublasStatus_t gemm_with_decided_stats(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                       cublasOperation_t op_B, uint64_t m, uint64_t n, uint64_t k,
                                       const T *alpha, const T *a, uint64_t lda, uint64_t stridea,
                                       const T *b, uint64_t ldb, uint64_t strideb, const T *beta,
                                       T *c, uint64_t ldc, uint64_t stridec, uint64_t batch,
                                       cuMpSGEMM_compute_mode_t mode, unsigned id_a,
                                       unsigned id_b) {
  if (h == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  DeviceGuard guard(h->device);
  unsigned flag_id;
  cuMpSGEMM_compute_mode_t gemm_mode;
  if (mode == CUMPSGEMM_AUTO) {
    flag_id = next_dyn_launch_id(h);
    cumpsgemm::set_dynamic_launch_buffer_by_exp_stats(h, flag_id, id_a, id_b);
    gemm_mode = CUMPSGEMM_AUTO;
  } else if (mode == CUMPSGEMM_FP16TCEC_SCALING) {
    flag_id = 1;
    gemm_mode = CUMPSGEMM_FP16TCEC;
  } else {
    return CUBLAS_STATUS_INVALID_VALUE;
  }
  const DynParams *dyn = prepare_dyn_params(h, flag_id, id_a, id_b);
  return gemm_dispatch<T>(h, op_A, op_B, m, n, k, alpha, a, lda, stridea, b, ldb, strideb, beta, c,
                          ldc, stridec, batch, gemm_mode, dyn, nullptr);
}
} // namespace

extern "C" {

unsigned cuMpSGEMM_exp_stats_ext_s(cuMpSGEMM_handle_t h, unsigned m, unsigned n, const float *ptr,
                                   unsigned ld, unsigned batch, unsigned stride) {
  return cumpsgemm::exp_stats_ext<float>(h, m, n, ptr, ld, batch, stride);
}
unsigned cuMpSGEMM_exp_stats_ext_c(cuMpSGEMM_handle_t h, unsigned m, unsigned n,
                                   const cuComplex *ptr, unsigned ld, unsigned batch,
                                   unsigned stride) {
  return cumpsgemm::exp_stats_ext<cuComplex>(h, m, n, ptr, ld, batch, stride);
}
unsigned cuMpSGEMM_exp_max_ext_s(cuMpSGEMM_handle_t h, unsigned m, unsigned n, const float *ptr,
                                 unsigned ld, unsigned batch, unsigned stride) {
  return cumpsgemm::exp_max_ext<float>(h, m, n, ptr, ld, batch, stride);
}
unsigned cuMpSGEMM_exp_max_ext_c(cuMpSGEMM_handle_t h, unsigned m, unsigned n, const cuComplex *ptr,
                                 unsigned ld, unsigned batch, unsigned stride) {
  return cumpsgemm::exp_max_ext<cuComplex>(h, m, n, ptr, ld, batch, stride);
}
void cuMpSGEMM_get_exp_stats(cuMpSGEMM_handle_t h, unsigned id, size_t *uf, size_t *total) {
  const auto r = cumpsgemm::get_exp_stats(h, id);
  if (uf) *uf = r.first;
  if (total) *total = r.second;
}
unsigned cuMpSGEMM_get_current_exp_stats_buffer_id(cuMpSGEMM_handle_t h) {
  return cumpsgemm::get_current_exp_stats_buffer_id(h);
}
void cuMpSGEMM_reset_exp_stats_buffer_id(cuMpSGEMM_handle_t h) {
  cumpsgemm::reset_exp_stats_buffer_id(h);
}
void cuMpSGEMM_set_exp_stats_params(cuMpSGEMM_handle_t h, float ig, float uf, float tol) {
  cumpsgemm::set_exp_stats_params(h, ig, uf, tol);
}
void cuMpSGEMM_enable_exp_stats(cuMpSGEMM_handle_t h) { cumpsgemm::enable_exp_stats(h); }
void cuMpSGEMM_disable_exp_stats(cuMpSGEMM_handle_t h) { cumpsgemm::disable_exp_stats(h); }
float cuMpSGEMM_get_max_exp(cuMpSGEMM_handle_t h, unsigned id) {
  return cumpsgemm::get_max_exp(h, id);
}
int cuMpSGEMM_get_exp_stats_compute_mode_level(cuMpSGEMM_handle_t h, unsigned id) {
  return static_cast<int>(cumpsgemm::get_exp_stats_compute_mode_level(h, id));
}

#define SCALE_WRAPPERS(SUFFIX, T)                                                               \
  void cuMpSGEMM_scale_A_##SUFFIX(cuMpSGEMM_handle_t h, unsigned sid, unsigned fid, unsigned m, \
                                  unsigned n, T *ptr, unsigned ld, unsigned batch,              \
                                  unsigned stride) {                                            \
    cumpsgemm::scale_A<T>(h, sid, fid, m, n, ptr, ld, batch, stride);                           \
  }                                                                                             \
  void cuMpSGEMM_scale_B_##SUFFIX(cuMpSGEMM_handle_t h, unsigned sid, unsigned fid, unsigned m, \
                                  unsigned n, T *ptr, unsigned ld, unsigned batch,              \
                                  unsigned stride) {                                            \
    cumpsgemm::scale_B<T>(h, sid, fid, m, n, ptr, ld, batch, stride);                           \
  }                                                                                             \
  void cuMpSGEMM_scale_C_##SUFFIX(cuMpSGEMM_handle_t h, unsigned sida, unsigned sidb,           \
                                  unsigned fid, unsigned m, unsigned n, T *ptr, unsigned ld,    \
                                  unsigned batch, unsigned stride) {                            \
    cumpsgemm::scale_C<T>(h, sida, sidb, fid, m, n, ptr, ld, batch, stride);                    \
  }                                                                                             \
  void cuMpSGEMM_reset_scale_A_##SUFFIX(cuMpSGEMM_handle_t h, unsigned sid, unsigned fid,       \
                                        unsigned m, unsigned n, T *ptr, unsigned ld,            \
                                        unsigned batch, unsigned stride) {                      \
    cumpsgemm::reset_scale_A<T>(h, sid, fid, m, n, ptr, ld, batch, stride);                     \
  }                                                                                             \
  void cuMpSGEMM_reset_scale_B_##SUFFIX(cuMpSGEMM_handle_t h, unsigned sid, unsigned fid,       \
                                        unsigned m, unsigned n, T *ptr, unsigned ld,            \
                                        unsigned batch, unsigned stride) {                      \
    cumpsgemm::reset_scale_B<T>(h, sid, fid, m, n, ptr, ld, batch, stride);                     \
  }
SCALE_WRAPPERS(s, float)
SCALE_WRAPPERS(c, cuComplex)
#undef SCALE_WRAPPERS

unsigned cuMpSGEMM_get_current_dynamic_launch_buffer_id(cuMpSGEMM_handle_t h) {
  return cumpsgemm::get_current_dynamic_launch_buffer_id(h);
}
unsigned cuMpSGEMM_get_next_dynamic_launch_buffer_id(cuMpSGEMM_handle_t h) {
  return cumpsgemm::get_next_dynamic_launch_buffer_id(h);
}
int cuMpSGEMM_get_dynamic_launch_gemm_compute_mode(cuMpSGEMM_handle_t h, unsigned id) {
  return static_cast<int>(cumpsgemm::get_dynamic_launch_gemm_compute_mode(h, id));
}
void cuMpSGEMM_get_dynamic_launch_scaling_mode_AB(cuMpSGEMM_handle_t h, unsigned id, int *sa,
                                                  int *sb) {
  const auto r = cumpsgemm::get_dynamic_launch_scaling_mode_AB(h, id);
  if (sa) *sa = r.first;
  if (sb) *sb = r.second;
}
void cuMpSGEMM_set_dynamic_launch_buffer_by_exp_stats(cuMpSGEMM_handle_t h, unsigned fid,
                                                      unsigned ida, unsigned idb) {
  cumpsgemm::set_dynamic_launch_buffer_by_exp_stats(h, fid, ida, idb);
}
void cuMpSGEMM_set_dynamic_launch_flag_buffer_id(cuMpSGEMM_handle_t h, unsigned id) {
  h->dyn_launch.enabled_id = id;
  h->dyn_launch.enabled = true;
}
void cuMpSGEMM_unset_dynamic_launch_flag_buffer_id(cuMpSGEMM_handle_t h) {
  h->dyn_launch.enabled_id = 0;
  h->dyn_launch.enabled = false;
}

void cuMpSGEMM_enable_exp_stats_profiling(cuMpSGEMM_handle_t h) {
  cumpsgemm::enable_exp_stats_profiling(h);
}
void cuMpSGEMM_disable_exp_stats_profiling(cuMpSGEMM_handle_t h) {
  cumpsgemm::disable_exp_stats_profiling(h);
}
void cuMpSGEMM_reset_exp_stats_profiling(cuMpSGEMM_handle_t h) {
  cumpsgemm::reset_exp_stats_profiling(h);
}
void cuMpSGEMM_print_exp_stats_profiling(cuMpSGEMM_handle_t h, unsigned csv) {
  cumpsgemm::print_exp_stats_profiling(h, csv);
}
int cuMpSGEMM_get_exp_stats_profiling_result(cuMpSGEMM_handle_t h, const char *name,
                                             double *time_sum_s, unsigned long long *n) {
  const auto r = cumpsgemm::debug::get_exp_stats_profiling_result(h);
  const auto it = r.find(name);
  if (it == r.end()) return 0;
  if (time_sum_s) *time_sum_s = it->second.time_sum;
  if (n) *n = it->second.n;
  return 1;
}

cublasStatus_t cuMpSGEMM_sgemm_module(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                      cublasOperation_t op_B, uint64_t m, uint64_t n, uint64_t k,
                                      const float *alpha, const float *a, uint64_t lda,
                                      const float *b, uint64_t ldb, const float *beta, float *c,
                                      uint64_t ldc, cuMpSGEMM_compute_mode_t mode,
                                      unsigned *used_kernel_module_id) {
  return cumpsgemm::gemm<float>(h, op_A, op_B, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, mode,
                                used_kernel_module_id);
}

int cuMpSGEMM_get_kernel_status(cuMpSGEMM_handle_t h) {
  if (h == nullptr) return -1;
  DeviceGuard guard(h->device);
  int v = 0;
  if (cudaMemcpyAsync(&v, h->dev_status, sizeof(int), cudaMemcpyDeviceToHost, h->cuda_stream) !=
      cudaSuccess)
    return -2;
  if (cudaStreamSynchronize(h->cuda_stream) != cudaSuccess) return -3;
  if (v != 0) cudaMemsetAsync(h->dev_status, 0, sizeof(int), h->cuda_stream);
  return v;
}

int cuMpSGEMM_selftest_bounded_wait(cuMpSGEMM_handle_t h, unsigned limit_ms,
                                    double *waited_ms) {
  if (h == nullptr) return -1;
  DeviceGuard guard(h->device);
  // the handle's status word doubles as the self-test's status; one DynParams record as scratch
  unsigned long long *dev_ns = reinterpret_cast<unsigned long long *>(
      h->dev_dyn_params + (h->dyn_params_length - 1));
  cudaMemsetAsync(h->dev_status, 0, sizeof(int), h->cuda_stream);
  if (launch_bounded_wait_selftest(h->dev_status, 1000000ull * limit_ms, dev_ns,
                                   h->cuda_stream) != cudaSuccess)
    return -2;
  unsigned long long ns = 0;
  cudaMemcpyAsync(&ns, dev_ns, sizeof(ns), cudaMemcpyDeviceToHost, h->cuda_stream);
  const int status = cuMpSGEMM_get_kernel_status(h); // synchronises and clears
  if (waited_ms) *waited_ms = static_cast<double>(ns) * 1e-6;
  return status;
}

void cuMpSGEMM_set_workspace_limit(cuMpSGEMM_handle_t h, size_t bytes) {
  h->workspace_limit_bytes = bytes;
}

void cuMpSGEMM_reload_tuning_env(cuMpSGEMM_handle_t h) { h->tuning = read_tuning_env(); }

void cuMpSGEMM_set_count_tail_padding(cuMpSGEMM_handle_t h, int enable) {
  h->exp_stats.count_tail_padding = (enable != 0);
}

void cuMpSGEMM_set_debug_buffer(cuMpSGEMM_handle_t h, unsigned long long *dev_words8) {
  h->debug_buffer = dev_words8;
}

void cuMpSGEMM_set_kernel_timing(cuMpSGEMM_handle_t h, int enable) {
  h->kernel_timing = enable != 0;
}

unsigned long long cuMpSGEMM_get_kernel_timing(cuMpSGEMM_handle_t h, double *split_ms,
                                               double *gemm_ms) {
  DeviceGuard guard(h->device);
  cudaStreamSynchronize(h->cuda_stream);
  double s = 0, g = 0;
  unsigned long long n = 0;
  for (auto &tt : h->timing_events) {
    float a = 0.f, b = 0.f;
    if (cudaEventElapsedTime(&a, tt.e[0], tt.e[1]) == cudaSuccess &&
        cudaEventElapsedTime(&b, tt.e[1], tt.e[2]) == cudaSuccess) {
      s += a;
      g += b;
      ++n;
    }
    for (auto &e : tt.e) cudaEventDestroy(e);
  }
  h->timing_events.clear();
  if (split_ms) *split_ms = s;
  if (gemm_ms) *gemm_ms = g;
  return n;
}

// ---- hijack control
cuMpSGEMM_handle_t cuMpSGEMM_hijack_get_internal_global_handle(void) {
  return cumpsgemm::hijack_control::get_internal_global_handle();
}
int cuMpSGEMM_hijack_set_compute_mode(int mode) {
  try {
    cumpsgemm::hijack_control::set_compute_mode(static_cast<cuMpSGEMM_compute_mode_t>(mode));
  } catch (const std::runtime_error &) {
    return 1;
  }
  return 0;
}
void cuMpSGEMM_hijack_unset_compute_mode(void) { cumpsgemm::hijack_control::unset_compute_mode(); }
void cuMpSGEMM_hijack_reset_exp_stats_buffer_id(void) {
  cumpsgemm::hijack_control::reset_exp_stats_buffer_id();
}
void cuMpSGEMM_hijack_set_exp_stats_params(float ig, float uf, float tol) {
  cumpsgemm::hijack_control::set_exp_stats_params(ig, uf, tol);
}
void cuMpSGEMM_hijack_enable_restoring_AB_after_scaling(void) {
  cumpsgemm::hijack_control::enable_restoring_AB_after_scaling();
}
void cuMpSGEMM_hijack_disable_restoring_AB_after_scaling(void) {
  cumpsgemm::hijack_control::disable_restoring_AB_after_scaling();
}
size_t cuMpSGEMM_hijack_get_last_called_function_str(char *buf, size_t size) {
  const std::string s = cumpsgemm::hijack_control::get_last_called_function_str();
  if (buf != nullptr && size > 0) {
    const size_t ncopy = s.size() < size - 1 ? s.size() : size - 1;
    std::memcpy(buf, s.data(), ncopy);
    buf[ncopy] = '\0';
  }
  return s.size();
}
void cuMpSGEMM_hijack_set_last_called_function_str(const char *str) {
  cumpsgemm::hijack_control::set_last_called_function_str(str != nullptr ? str : "");
}
void cuMpSGEMM_hijack_enable_custom_gemm_Mx2x2(void) {
  cumpsgemm::hijack_control::enable_custom_gemm_Mx2x2();
}
void cuMpSGEMM_hijack_disable_custom_gemm_Mx2x2(void) {
  cumpsgemm::hijack_control::disable_custom_gemm_Mx2x2();
}
void cuMpSGEMM_hijack_clear_last_called_function_str(void) {
  cumpsgemm::hijack_control::clear_last_called_function_str();
}
int cuMpSGEMM_hijack_is_library_loaded(void) {
  return cumpsgemm::hijack_control::is_library_loaded() ? 1 : 0;
}
void cuMpSGEMM_hijack_set_control_function(cuMpSGEMM_control_function_c_t fn) {
  if (fn == nullptr) {
    cumpsgemm::hijack_control::unset_control_function();
    return;
  }
  cumpsgemm::hijack_control::set_control_function(
      [fn](const int a, const int b, const unsigned m, const unsigned n, const unsigned k) {
        return static_cast<cuMpSGEMM_compute_mode_t>(fn(a, b, m, n, k));
      });
}

// ---- multi-GPU support
unsigned cuMpSGEMM_exp_stats_begin(cuMpSGEMM_handle_t h) {
  DeviceGuard guard(h->device);
  const unsigned id = next_exp_stats_id(h);
  exp_stats_init_slot(h, id);
  return id;
}
void cuMpSGEMM_exp_stats_stage_s(cuMpSGEMM_handle_t h, int stage, unsigned id, unsigned m,
                                 unsigned n, const float *ptr, unsigned ld, unsigned batch,
                                 unsigned stride) {
  DeviceGuard guard(h->device);
  if (stage == 1) exp_stats_stage1<float>(h, id, m, n, ptr, ld, batch, stride);
  if (stage == 2) exp_stats_stage2<float>(h, id, m, n, ptr, ld, batch, stride);
  if (stage == 3) exp_max_only<float>(h, id, m, n, ptr, ld, batch, stride);
}
void cuMpSGEMM_exp_stats_stage_c(cuMpSGEMM_handle_t h, int stage, unsigned id, unsigned m,
                                 unsigned n, const cuComplex *ptr, unsigned ld, unsigned batch,
                                 unsigned stride) {
  DeviceGuard guard(h->device);
  if (stage == 1) exp_stats_stage1<cuComplex>(h, id, m, n, ptr, ld, batch, stride);
  if (stage == 2) exp_stats_stage2<cuComplex>(h, id, m, n, ptr, ld, batch, stride);
  if (stage == 3) exp_max_only<cuComplex>(h, id, m, n, ptr, ld, batch, stride);
}
void cuMpSGEMM_exp_stats_decide(cuMpSGEMM_handle_t h, int decision, unsigned id) {
  DeviceGuard guard(h->device);
  if (decision == 1) exp_stats_decide1(h, id);
  if (decision == 2) exp_stats_decide2(h, id);
}
void cuMpSGEMM_exp_stats_export(cuMpSGEMM_handle_t h, unsigned id, unsigned long long *w) {
  DeviceGuard guard(h->device);
  export_slot_kernel<<<1, 1, 0, h->cuda_stream>>>(w, h->exp_stats.dev_max + id,
                                                  h->exp_stats.dev_total + id,
                                                  h->exp_stats.dev_underflow + id,
                                                  h->exp_stats.dev_mode + id);
}
void cuMpSGEMM_exp_stats_import(cuMpSGEMM_handle_t h, unsigned id, const unsigned long long *w) {
  DeviceGuard guard(h->device);
  import_slot_kernel<<<1, 1, 0, h->cuda_stream>>>(w, h->exp_stats.dev_max + id,
                                                  h->exp_stats.dev_total + id,
                                                  h->exp_stats.dev_underflow + id,
                                                  h->exp_stats.dev_mode + id);
}
cublasStatus_t cuMpSGEMM_sgemm_strided_batch_with_stats(
    cuMpSGEMM_handle_t h, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m, uint64_t n,
    uint64_t k, const float *alpha, const float *a, uint64_t lda, uint64_t stridea, const float *b,
    uint64_t ldb, uint64_t strideb, const float *beta, float *c, uint64_t ldc, uint64_t stridec,
    uint64_t batch, cuMpSGEMM_compute_mode_t mode, unsigned id_a, unsigned id_b) {
  return gemm_with_decided_stats<float>(h, op_A, op_B, m, n, k, alpha, a, lda, stridea, b, ldb,
                                        strideb, beta, c, ldc, stridec, batch, mode, id_a, id_b);
}
cublasStatus_t cuMpSGEMM_cgemm_strided_batch_with_stats(
    cuMpSGEMM_handle_t h, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m, uint64_t n,
    uint64_t k, const cuComplex *alpha, const cuComplex *a, uint64_t lda, uint64_t stridea,
    const cuComplex *b, uint64_t ldb, uint64_t strideb, const cuComplex *beta, cuComplex *c,
    uint64_t ldc, uint64_t stridec, uint64_t batch, cuMpSGEMM_compute_mode_t mode, unsigned id_a,
    unsigned id_b) {
  return gemm_with_decided_stats<cuComplex>(h, op_A, op_B, m, n, k, alpha, a, lda, stridea, b, ldb,
                                            strideb, beta, c, ldc, stridec, batch, mode, id_a,
                                            id_b);
}

// ---- two-by-two inner problems (tiny_gemm.cu) ------------------------------------------------
cublasStatus_t cuMpSGEMM_sgemm_Mx2x2(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t m, const float *alpha,
                                     const float *a, uint64_t lda, uint64_t stridea,
                                     const float *b, uint64_t ldb, uint64_t strideb,
                                     const float *beta, float *c, uint64_t ldc, uint64_t stridec,
                                     uint64_t batch_count) {
  return cumpsgemm_b200::tiny_gemm<float>(h, true, op_A, op_B, m, alpha, a, lda, stridea, b, ldb,
                                          strideb, beta, c, ldc, stridec, batch_count);
}
cublasStatus_t cuMpSGEMM_cgemm_Mx2x2(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t m, const cuComplex *alpha,
                                     const cuComplex *a, uint64_t lda, uint64_t stridea,
                                     const cuComplex *b, uint64_t ldb, uint64_t strideb,
                                     const cuComplex *beta, cuComplex *c, uint64_t ldc,
                                     uint64_t stridec, uint64_t batch_count) {
  return cumpsgemm_b200::tiny_gemm<cuComplex>(h, true, op_A, op_B, m, alpha, a, lda, stridea, b,
                                              ldb, strideb, beta, c, ldc, stridec, batch_count);
}
cublasStatus_t cuMpSGEMM_sgemm_2xNx2(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t n, const float *alpha,
                                     const float *a, uint64_t lda, uint64_t stridea,
                                     const float *b, uint64_t ldb, uint64_t strideb,
                                     const float *beta, float *c, uint64_t ldc, uint64_t stridec,
                                     uint64_t batch_count) {
  return cumpsgemm_b200::tiny_gemm<float>(h, false, op_A, op_B, n, alpha, a, lda, stridea, b, ldb,
                                          strideb, beta, c, ldc, stridec, batch_count);
}
cublasStatus_t cuMpSGEMM_cgemm_2xNx2(cuMpSGEMM_handle_t h, cublasOperation_t op_A,
                                     cublasOperation_t op_B, uint64_t n, const cuComplex *alpha,
                                     const cuComplex *a, uint64_t lda, uint64_t stridea,
                                     const cuComplex *b, uint64_t ldb, uint64_t strideb,
                                     const cuComplex *beta, cuComplex *c, uint64_t ldc,
                                     uint64_t stridec, uint64_t batch_count) {
  return cumpsgemm_b200::tiny_gemm<cuComplex>(h, false, op_A, op_B, n, alpha, a, lda, stridea, b,
                                              ldb, strideb, beta, c, ldc, stridec, batch_count);
}

} // extern "C"
