// C entry points around the reference's own statistics / scaling / flag code, compiled
// unmodified from the reference tree (src/exp_stats.cu, src/dynamic_scaling.cu,
// src/dynamic_launch.cu) against the stand-in cutf headers in cutf_stub/.
//
// TEST INFRASTRUCTURE ONLY.  The resulting oracle/_ref/libref_stats.so is the checker that
// pins the product's statistics, decisions, flag words and scaled matrices to what the
// reference's kernels produce on the same device buffers; nothing the product ships links
// or loads it.  The handle built here holds exactly the pieces those three files touch
// (src/handle.hpp:7-29: num_sms, cuda_stream, exp_stats_handle, dynamic_launch_handle).
#include <cstddef>

#include "dynamic_launch.hpp"
#include "dynamic_scaling.hpp"
#include "exp_stats.hpp"
#include <cuComplex.h>
#include <cumpsgemm/cumpsgemm.hpp>

extern "C" {

void *ref_create(void) {
  auto *h = new cuMpSGEMM_handle;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  h->num_sms = static_cast<unsigned>(sms);
  h->cuda_stream = 0;
  h->temp_working_memory = nullptr;
  h->temp_working_memory_float_count = 0;
  init_exp_stats_counter_buffer(h);
  init_dynamic_launch_flag_buffer(h);
  cudaStreamSynchronize(h->cuda_stream);
  return h;
}

void ref_destroy(void *hv) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cudaStreamSynchronize(h->cuda_stream);
  destroy_exp_stats_counter_buffer(h);
  destroy_launch_flag_buffer(h);
  delete h;
}

void ref_set_stream(void *hv, cudaStream_t s) { static_cast<cuMpSGEMM_handle *>(hv)->cuda_stream = s; }

void ref_set_exp_stats_params(void *hv, float ignore_threshold, float underflow_threshold,
                              float underflow_tolerance_rate) {
  cumpsgemm::set_exp_stats_params(static_cast<cuMpSGEMM_handle *>(hv), ignore_threshold,
                                  underflow_threshold, underflow_tolerance_rate);
}

// Statistics: return the slot id the call used.
unsigned ref_exp_stats_ext_s(void *hv, unsigned m, unsigned n, const float *ptr, unsigned ld,
                             unsigned batch, unsigned stride) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cumpsgemm::exp_stats::exp_stats_ext<float>(h, m, n, ptr, ld, batch, stride);
  return cumpsgemm::exp_stats::get_current_exp_stats_buffer_id(h);
}
unsigned ref_exp_stats_ext_c(void *hv, unsigned m, unsigned n, const cuComplex *ptr, unsigned ld,
                             unsigned batch, unsigned stride) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cumpsgemm::exp_stats::exp_stats_ext<cuComplex>(h, m, n, ptr, ld, batch, stride);
  return cumpsgemm::exp_stats::get_current_exp_stats_buffer_id(h);
}
unsigned ref_exp_max_ext_s(void *hv, unsigned m, unsigned n, const float *ptr, unsigned ld,
                           unsigned batch, unsigned stride) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cumpsgemm::exp_stats::exp_max_ext<float>(h, m, n, ptr, ld, batch, stride);
  return cumpsgemm::exp_stats::get_current_exp_stats_buffer_id(h);
}
unsigned ref_exp_max_ext_c(void *hv, unsigned m, unsigned n, const cuComplex *ptr, unsigned ld,
                           unsigned batch, unsigned stride) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cumpsgemm::exp_stats::exp_max_ext<cuComplex>(h, m, n, ptr, ld, batch, stride);
  return cumpsgemm::exp_stats::get_current_exp_stats_buffer_id(h);
}

void ref_get_exp_stats(void *hv, unsigned id, unsigned long long *underflow,
                       unsigned long long *total) {
  const auto r = cumpsgemm::exp_stats::get_exp_stats(static_cast<cuMpSGEMM_handle *>(hv), id);
  *underflow = r.first;
  *total = r.second;
}
float ref_get_max_exp(void *hv, unsigned id) {
  return cumpsgemm::dynamic_scaling::get_max_exp(static_cast<cuMpSGEMM_handle *>(hv), id);
}
int ref_get_compute_mode_level(void *hv, unsigned id) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cudaStreamSynchronize(h->cuda_stream);
  return static_cast<int>(cumpsgemm::exp_stats::get_compute_mode_level(h, id));
}

// Flag words
unsigned ref_next_flag_id(void *hv) {
  return cumpsgemm::dynamic_launch::get_next_dynamic_launch_flag_buffer_id(
      static_cast<cuMpSGEMM_handle *>(hv));
}
void ref_set_flag_by_exp_stats(void *hv, unsigned flag_id, unsigned id_a, unsigned id_b) {
  cumpsgemm::dynamic_scaling::set_dynamic_launch_buffer_by_exp_stats(
      static_cast<cuMpSGEMM_handle *>(hv), flag_id, id_a, id_b);
}
int ref_get_flag(void *hv, unsigned flag_id) {
  auto *h = static_cast<cuMpSGEMM_handle *>(hv);
  cudaStreamSynchronize(h->cuda_stream);
  return cumpsgemm::dynamic_launch::get_dynamic_launch_buffer(h, flag_id);
}

// Scaling.  what: 0 scale_A, 1 scale_B, 2 scale_C, 3 reset_scale_A, 4 reset_scale_B.
// (The reference's argument order is ld, stride, batch.)
#define REF_SCALE(SUFFIX, T)                                                                     \
  void ref_scale_##SUFFIX(void *hv, int what, unsigned m, unsigned n, T *ptr, unsigned ld,       \
                          unsigned batch, unsigned stride, unsigned id_a, unsigned id_b,         \
                          unsigned flag_id) {                                                    \
    auto *h = static_cast<cuMpSGEMM_handle *>(hv);                                               \
    namespace ds = cumpsgemm::dynamic_scaling;                                                   \
    switch (what) {                                                                              \
    case 0: ds::scale_A<T>(h, m, n, ptr, ld, stride, batch, id_a, flag_id); break;               \
    case 1: ds::scale_B<T>(h, m, n, ptr, ld, stride, batch, id_a, flag_id); break;               \
    case 2: ds::scale_C<T>(h, m, n, ptr, ld, stride, batch, id_a, id_b, flag_id); break;         \
    case 3: ds::reset_scale_A<T>(h, m, n, ptr, ld, stride, batch, id_a, flag_id); break;         \
    default: ds::reset_scale_B<T>(h, m, n, ptr, ld, stride, batch, id_a, flag_id); break;        \
    }                                                                                            \
  }
REF_SCALE(s, float)
REF_SCALE(c, cuComplex)
#undef REF_SCALE

} // extern "C"
