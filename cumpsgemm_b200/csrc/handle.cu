// Handle life cycle, logging helpers and the mode-name table.
//
// Reference counterparts: src/handle.cu:7-52 (create / destroy / set_stream),
// src/utils.hpp:5-42 (logging), src/cumpsgemm_cublas.cu:163-196 (mode names).
#include "internal.hpp"

#include <new>
#include <string>

namespace cumpsgemm_b200 {
void configure_mode_buffer(cuMpSGEMM_handle *h);
void init_flag_buffer(cuMpSGEMM_handle *h);

bool env_flag(const char *name, bool default_value) {
  const char *env = std::getenv(name);
  if (env == nullptr) return default_value;
  return std::string(env) != "0";
}
void log_info(const std::string &s) {
  if (env_flag("CUMPSGEMM_INFO", false)) {
    std::fprintf(stdout, "[cuMpSGEMM LOG] %s\n", s.c_str());
    std::fflush(stdout);
  }
}
void log_error(const std::string &s) {
  if (env_flag("CUMPSGEMM_ERROR_LOG", true)) {
    std::fprintf(stdout, "[cuMpSGEMM ERROR] %s\n", s.c_str());
    std::fflush(stdout);
  }
}
Tuning read_tuning_env() {
  Tuning t;
  auto as_int = [](const char *name, int dflt) {
    const char *e = std::getenv(name);
    return (e != nullptr && e[0] != '\0') ? std::atoi(e) : dflt;
  };
  const int tn = as_int("CUMPSGEMM_TILE_N", 0);
  t.tile_n = (tn == 256 || tn == 128 || tn == 64) ? tn : 0;
  const int pr = as_int("CUMPSGEMM_PAIR", -1);
  t.pair = (pr == 0 || pr == 1) ? pr : -1;
  t.drain_chunk = as_int("CUMPSGEMM_DRAIN_CHUNK", 0);
  t.first_chunk = as_int("CUMPSGEMM_FIRST_CHUNK", 0);
  t.pace = as_int("CUMPSGEMM_PACE", 1) != 0 ? 1 : 0;
  const int fu = as_int("CUMPSGEMM_FUSED", -1);
  t.fused = (fu == 0 || fu == 1) ? fu : -1;
  const int sk = as_int("CUMPSGEMM_SPLIT_K", -1);
  t.split_k = (sk >= 0) ? sk : -1;
  const int ts = as_int("CUMPSGEMM_TAIL_SPLIT", -1);
  t.tail_split = (ts >= 0) ? ts : -1;
  return t;
}
void log_warning(const std::string &s) {
  if (env_flag("CUMPSGEMM_ERROR_LOG", false)) {
    std::fprintf(stdout, "[cuMpSGEMM WARNING] %s\n", s.c_str());
    std::fflush(stdout);
  }
}
} // namespace cumpsgemm_b200

using namespace cumpsgemm_b200;

extern "C" cublasStatus_t cuMpSGEMM_create(cuMpSGEMM_handle_t *const handle) {
  if (handle == nullptr) return CUBLAS_STATUS_INVALID_VALUE;
  cuMpSGEMM_handle *h = new (std::nothrow) cuMpSGEMM_handle;
  if (h == nullptr) return CUBLAS_STATUS_ALLOC_FAILED;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    delete h;
    return CUBLAS_STATUS_NOT_INITIALIZED;
  }
  h->device = dev;
  int sms = 0, cc_major = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev);
  h->num_sms = static_cast<unsigned>(sms);
  if (cc_major != 10) {
    log_error("this build contains sm_100a kernels only; device compute capability major is " +
              std::to_string(cc_major));
    delete h;
    return CUBLAS_STATUS_ARCH_MISMATCH;
  }

  bool ok = true;
  auto &es = h->exp_stats;
  ok &= cudaMalloc(&es.dev_total, sizeof(unsigned long long) * es.buffer_length) == cudaSuccess;
  ok &= cudaMalloc(&es.dev_underflow, sizeof(unsigned long long) * es.buffer_length) == cudaSuccess;
  ok &= cudaMalloc(&es.dev_max, sizeof(float) * es.buffer_length) == cudaSuccess;
  ok &= cudaMalloc(&es.dev_mode, sizeof(int) * es.buffer_length) == cudaSuccess;
  ok &= cudaMalloc(&h->dyn_launch.flag_buffer, sizeof(int) * h->dyn_launch.flag_buffer_length) ==
        cudaSuccess;
  ok &= cudaMalloc(&h->dev_dyn_params, sizeof(DynParams) * h->dyn_params_length) == cudaSuccess;
  ok &= cudaMalloc(&h->dev_status, (2 + kPairTailCounters) * sizeof(int)) == cudaSuccess; // status, wave counter, tail-split counters
  ok &= cudaEventCreateWithFlags(&h->order_event, cudaEventDisableTiming) == cudaSuccess;
  const size_t scan_scratch_bytes = static_cast<size_t>(h->num_sms) * 8 * 24 * 2 + 16;
  ok &= cudaMalloc(&es.dev_scan_scratch, scan_scratch_bytes) == cudaSuccess;
  if (!ok) {
    cuMpSGEMM_destroy(h);
    return CUBLAS_STATUS_ALLOC_FAILED;
  }
  cudaMemsetAsync(es.dev_total, 0, sizeof(unsigned long long) * es.buffer_length, h->cuda_stream);
  cudaMemsetAsync(es.dev_underflow, 0, sizeof(unsigned long long) * es.buffer_length,
                  h->cuda_stream);
  cudaMemsetAsync(es.dev_max, 0, sizeof(float) * es.buffer_length, h->cuda_stream);
  cudaMemsetAsync(es.dev_mode, 0, sizeof(int) * es.buffer_length, h->cuda_stream);
  cudaMemsetAsync(h->dyn_launch.flag_buffer, 0, sizeof(int) * h->dyn_launch.flag_buffer_length,
                  h->cuda_stream);
  cudaMemsetAsync(h->dev_status, 0, (2 + kPairTailCounters) * sizeof(int), h->cuda_stream);
  cudaMemsetAsync(es.dev_scan_scratch, 0, scan_scratch_bytes, h->cuda_stream);
  configure_mode_buffer(h);
  init_flag_buffer(h);
  if (cudaStreamSynchronize(h->cuda_stream) != cudaSuccess) {
    cuMpSGEMM_destroy(h);
    return CUBLAS_STATUS_EXECUTION_FAILED;
  }
  h->exp_stats.count_tail_padding = env_flag("CUMPSGEMM_COUNT_TAIL_PADDING", false);
  h->tuning = read_tuning_env();
  const char *ws_env = std::getenv("CUMPSGEMM_WORKSPACE_LIMIT_MB");
  if (ws_env != nullptr) h->workspace_limit_bytes = std::strtoull(ws_env, nullptr, 10) << 20;
  *handle = h;
  return CUBLAS_STATUS_SUCCESS;
}

extern "C" cublasStatus_t cuMpSGEMM_destroy(cuMpSGEMM_handle_t handle) {
  if (handle == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  DeviceGuard guard(handle->device);
  cudaFree(handle->exp_stats.dev_total);
  cudaFree(handle->exp_stats.dev_underflow);
  cudaFree(handle->exp_stats.dev_max);
  cudaFree(handle->exp_stats.dev_mode);
  cudaFree(handle->exp_stats.dev_scan_scratch);
  cudaFree(handle->dyn_launch.flag_buffer);
  cudaFree(handle->dev_dyn_params);
  cudaFree(handle->dev_status);
  cudaFree(handle->workspace);
  if (handle->order_event != nullptr) cudaEventDestroy(handle->order_event);
  delete handle;
  return CUBLAS_STATUS_SUCCESS;
}

extern "C" cublasStatus_t cuMpSGEMM_set_stream(cuMpSGEMM_handle_t handle,
                                               const cudaStream_t cuda_stream) {
  if (handle == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  if (cuda_stream != handle->cuda_stream && handle->order_event_recorded) {
    // Work already enqueued through this handle may still use its workspace, rings and
    // counters: whatever runs on the new stream is ordered behind it.  (The reference has one
    // stream per handle at a time and no such hazard, src/handle.cu:48-52, because its kernels
    // keep no operand workspace.)
    DeviceGuard guard(handle->device);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(cuda_stream, &cap) == cudaSuccess &&
        cap == cudaStreamCaptureStatusNone) {
      if (cudaStreamWaitEvent(cuda_stream, handle->order_event, 0) != cudaSuccess)
        cudaGetLastError();
    } else {
      cudaGetLastError();
    }
  }
  handle->cuda_stream = cuda_stream;
  return CUBLAS_STATUS_SUCCESS;
}

extern "C" const char *cuMpSGEMM_get_compute_mode_string(const cuMpSGEMM_compute_mode_t mode) {
  static const char *const names[] = {
      "CUBLAS",      "FP16TCEC",      "TF32TCEC", "FP16TC", "TF32TC",    "CUBLAS_SIMT",
      "CUBLAS_FP16TC", "CUBLAS_TF32TC", "DRY_RUN",  "AUTO",   "UNDEFINED", "FP16TCEC_SCALING",
      "FP32_SIMT"};
  const int i = static_cast<int>(mode);
  if (i < 0 || i >= static_cast<int>(sizeof(names) / sizeof(names[0]))) return "Unknown";
  return names[i];
}
