// cuBLAS interception layer (LD_PRELOAD target) and its run-time control.
//
// Reference counterpart: src/cumpsgemm_cublas.cu
//   :101-157   lazily created process-wide handle + environment configuration
//   :198-220   mode selection chain (control function -> libcumpsgemm_rule.so -> default rule)
//   :222-593   cuMpSGEMM_hijack_core<T>
//   :595-976   cuMpSGEMM_stridedBatched_hijack_core<T>
//   :979-1187  exported cuBLAS symbols
//   :1189-1271 cumpsgemm::hijack_control
// Differences, all deliberate:
//   * the cuBLAS handle's stream is honoured (the reference fetches it and then ignores it);
//   * AUTO / FP16TCEC_SCALING fold the operand scaling into the split pass and the un-scaling
//     into the GEMM epilogue, so A and B are never written (the reference scales them in place
//     and restores them afterwards) and beta*C is not multiplied by the un-scaling factor;
//   * alpha/beta given in device memory (CUBLAS_POINTER_MODE_DEVICE) are copied to the host;
//   * the real cuBLAS is resolved lazily with dlsym so the library has no link-time
//     dependency on a particular libcublas;
//   * the rule library is looked up under its documented name cuMpSGEMM_get_compute_mode
//     (and, for compatibility, under the name the reference actually queries).
#include "internal.hpp"

#include <cumpsgemm/cumpsgemm_ext.h>
#include <cumpsgemm/hijack_control.hpp>
#include <dlfcn.h>
#include <iomanip>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <time.h>
#include <type_traits>

using namespace cumpsgemm_b200;

namespace {

std::mutex g_mutex; // protects the globals below
constexpr int kMaxDevices = 64;
cuMpSGEMM_handle_t g_handles[kMaxDevices] = {}; // one lazily created handle per device
std::string g_last_called;
bool g_mx2x2_enabled = false;
bool g_restore_ab = true;
cumpsgemm::hijack_control::control_function_t g_control_func;
enum class HijackMode { static_mode, dynamic_mode };
HijackMode g_hijack_mode = HijackMode::dynamic_mode;
cuMpSGEMM_compute_mode_t g_static_mode = CUMPSGEMM_CUBLAS;

std::string sci(const double a) {
  std::stringstream ss;
  ss << std::scientific << a;
  return ss.str();
}

const char *op_str(const cublasOperation_t op) {
  switch (op) {
  case CUBLAS_OP_N:
    return "N";
  case CUBLAS_OP_T:
    return "T";
  case CUBLAS_OP_C:
    return "C";
  default:
    return "?";
  }
}

// ---- the real cuBLAS ---------------------------------------------------
void *real_cublas_symbol(const char *name) {
  void *p = dlsym(RTLD_NEXT, name);
  if (p != nullptr) return p;
  static void *lib = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    for (const char *n : {"libcublas.so.12", "libcublas.so.13", "libcublas.so"}) {
      lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (lib != nullptr) break;
    }
  });
  if (lib == nullptr) return nullptr;
  return dlsym(lib, name);
}

cudaStream_t stream_of(cublasHandle_t handle) {
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cudaStream_t *);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGetStream_v2"));
  cudaStream_t s = 0;
  if (fn != nullptr && handle != nullptr) fn(handle, &s);
  return s;
}

cublasMath_t math_mode_of(cublasHandle_t handle) {
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasMath_t *);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGetMathMode"));
  cublasMath_t m = CUBLAS_DEFAULT_MATH;
  if (fn != nullptr && handle != nullptr) fn(handle, &m);
  return m;
}

bool device_pointer_mode(cublasHandle_t handle) {
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasPointerMode_t *);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGetPointerMode_v2"));
  cublasPointerMode_t m = CUBLAS_POINTER_MODE_HOST;
  if (fn != nullptr && handle != nullptr) fn(handle, &m);
  return m == CUBLAS_POINTER_MODE_DEVICE;
}

template <class T> cudaDataType_t cuda_type();
template <> cudaDataType_t cuda_type<float>() { return CUDA_R_32F; }
template <> cudaDataType_t cuda_type<cuComplex>() { return CUDA_C_32F; }

// ---- optional host-side call timing (CUMPSGEMM_ENABLE_CULIP_PROFILING) --
struct CallTimer {
  bool enabled;
  cudaStream_t stream;
  std::string name;
  timespec t0;
  CallTimer(cudaStream_t s, const std::string &n)
      : enabled(env_flag("CUMPSGEMM_ENABLE_CULIP_PROFILING", false)), stream(s), name(n) {
    if (enabled) {
      cudaStreamSynchronize(stream);
      clock_gettime(CLOCK_MONOTONIC, &t0);
    }
  }
  ~CallTimer() {
    if (enabled) {
      cudaStreamSynchronize(stream);
      timespec t1;
      clock_gettime(CLOCK_MONOTONIC, &t1);
      const unsigned long ns =
          (t1.tv_sec - t0.tv_sec) * 1000000000l + (t1.tv_nsec - t0.tv_nsec);
      std::printf("[CULiP Result][%s] %luns\n", name.c_str(), ns);
      std::fflush(stdout);
    }
  }
};

template <class T>
std::string timer_name(const char *base, cublasOperation_t a, cublasOperation_t b, uint64_t m,
                       uint64_t n, uint64_t k, uint64_t batch) {
  std::string s = std::string(base) + "-" + op_str(a) + op_str(b) + "-m" + std::to_string(m) +
                  "-n" + std::to_string(n) + "-k" + std::to_string(k);
  if (batch > 0) s += "-batchCount" + std::to_string(batch);
  return s;
}

float env_float(const char *name, float dflt) {
  const char *e = std::getenv(name);
  if (e == nullptr) return dflt;
  try {
    return std::stof(e);
  } catch (...) {
    return dflt;
  }
}
int env_int(const char *name, int dflt) {
  const char *e = std::getenv(name);
  if (e == nullptr) return dflt;
  try {
    return std::stoi(e);
  } catch (...) {
    return dflt;
  }
}

cuMpSGEMM_handle_t global_handle() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    log_error("Initialization failed.");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  cuMpSGEMM_handle_t &g_handle = g_handles[dev];
  if (g_handle == nullptr) {
    log_info("Initialize cuMpSGEMM handle...");
    if (cuMpSGEMM_create(&g_handle) != CUBLAS_STATUS_SUCCESS) {
      log_error("Initialization failed.");
      g_handle = nullptr;
      return nullptr;
    }
    const float ignore_threshold = env_float("CUMPSGEMM_AUTO_IGNORE_THRESHOLD", 0.f);
    const float underflow_threshold = env_float("CUMPSGEMM_AUTO_UNDERFLOW_THRESHOLD", 1.f / 32768);
    const float tolerance = env_float("CUMPSGEMM_AUTO_UNDERFLOW_TOLERANCE_RATE", 0.f);
    const int restore = env_int("CUMPSGEMM_AUTO_RESTORE_AB_SCALING", 1);
    log_info("AUTO config: ignore_threshold=" + sci(ignore_threshold) + " @Init");
    log_info("AUTO config: underflow_threshold=" + sci(underflow_threshold) + " @Init");
    log_info("AUTO config: underflow_tolerance_rate=" + sci(tolerance) + " @Init");
    log_info("AUTO config: restore_AB_scaling=" + std::to_string(restore) + " @Init");
    log_info(std::string("CUSTOM_GEMM_MX2X2: ") +
             ((g_mx2x2_enabled || env_flag("CUMPSGEMM_CUSTOM_GEMM_MX2X2", false)) ? "enabled"
                                                                                   : "disabled") +
             " @Init");
    cumpsgemm::set_exp_stats_params(g_handle, ignore_threshold, underflow_threshold, tolerance);
    g_restore_ab = restore != 0;
  }
  return g_handle;
}

// ---- rule library --------------------------------------------------------
using rule_fn_t = cuMpSGEMM_compute_mode_t (*)(const char *, cublasHandle_t, cublasOperation_t,
                                               cublasOperation_t, unsigned, unsigned, unsigned);
rule_fn_t rule_library_function() {
  static rule_fn_t fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void *lib = dlopen("libcumpsgemm_rule.so", RTLD_NOW);
    if (lib == nullptr) {
      log_warning("Failed to load libcumpsgemm_rule.so. Default rule will be used.");
      return;
    }
    void *p = dlsym(lib, "cuMpSGEMM_get_compute_mode");
    if (p == nullptr) p = dlsym(lib, "cuMpSGEMM_get_compute_mode_internal");
    if (p == nullptr) {
      log_warning("Failed to load a function cuMpSGEMM_get_compute_mode during selecting "
                  "hijacking function. Default rule will be used.");
      return;
    }
    fn = reinterpret_cast<rule_fn_t>(p);
  });
  return fn;
}

// Read alpha / beta wherever the cuBLAS handle says they live.
template <class T>
bool fetch_scalars(cublasHandle_t h, cudaStream_t stream, const T *alpha, const T *beta, T *a_out,
                   T *b_out) {
  if (alpha == nullptr || beta == nullptr) return false;
  if (device_pointer_mode(h)) {
    if (cudaMemcpyAsync(a_out, alpha, sizeof(T), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
      return false;
    if (cudaMemcpyAsync(b_out, beta, sizeof(T), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
      return false;
    return cudaStreamSynchronize(stream) == cudaSuccess;
  }
  *a_out = *alpha;
  *b_out = *beta;
  return true;
}

void log_auto_decision(cuMpSGEMM_handle_t h, unsigned id_a, unsigned id_b, unsigned flag_id) {
  if (!env_flag("CUMPSGEMM_INFO", false)) return;
  const int gemm_mode = static_cast<int>(cumpsgemm::get_dynamic_launch_gemm_compute_mode(h, flag_id));
  const auto sc = cumpsgemm::get_dynamic_launch_scaling_mode_AB(h, flag_id);
  const auto la = cumpsgemm::get_exp_stats(h, id_a);
  const auto lb = cumpsgemm::get_exp_stats(h, id_b);
  log_info(std::string("AUTO[ignore<") + sci(h->exp_stats.ignore_threshold) + ", uf<" +
           sci(h->exp_stats.underflow_threshold) +
           ", tolerance=" + sci(h->exp_stats.underflow_tolerance_rate) + "]: GEMM_MODE=" +
           cuMpSGEMM_get_compute_mode_string(static_cast<cuMpSGEMM_compute_mode_t>(gemm_mode)) +
           ", loss_A=" + std::to_string(la.first) + "/" + std::to_string(la.second) + "(" +
           std::to_string(static_cast<double>(la.first) / la.second) +
           "), scale_A=" + std::to_string(sc.first) + ", loss_B=" + std::to_string(lb.first) +
           "/" + std::to_string(lb.second) + "(" +
           std::to_string(static_cast<double>(lb.first) / lb.second) +
           "), scale_B=" + std::to_string(sc.second));
}

// Shared body of the single and the strided-batch interception.  batch == 0 marks the
// non-batched entry points (log grammar differs).
template <class T>
cublasStatus_t hijack_core(const char *func_name, cublasHandle_t cublas_handle,
                           cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m, uint64_t n,
                           uint64_t k, const T *alpha, const T *a, uint64_t lda, uint64_t stridea,
                           const T *b, uint64_t ldb, uint64_t strideb, const T *beta, T *c,
                           uint64_t ldc, uint64_t stridec, uint64_t batch, bool batched) {
  if (m == 0 || n == 0 || k == 0 || lda == 0 || ldb == 0 || ldc == 0 || (batched && batch == 0))
    return CUBLAS_STATUS_INVALID_VALUE;
  cuMpSGEMM_handle_t h = global_handle();
  if (h == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  const cudaStream_t stream = stream_of(cublas_handle);

  const cuMpSGEMM_compute_mode_t mode = cuMpSGEMM_get_compute_mode_internal(
      func_name, cublas_handle, op_A, op_B, static_cast<unsigned>(m), static_cast<unsigned>(n),
      static_cast<unsigned>(k));
  // One handle per device serves every caller: a call owns it from here to its last launch.
  // Calls on different streams are ordered on the device by cuMpSGEMM_set_stream.
  std::lock_guard<std::mutex> call_lock(h->call_mutex);

  const bool dynamic = (g_hijack_mode == HijackMode::dynamic_mode);
  log_info(std::string(func_name) + " op=(" + op_str(op_A) + ", " + op_str(op_B) + "), shape=(" +
           std::to_string(m) + ", " + std::to_string(n) + ", " + std::to_string(k) + ")" +
           (batched ? ", batch=" + std::to_string(batch) : std::string("")) +
           ", mode=" + cuMpSGEMM_get_compute_mode_string(mode) + "[" +
           (dynamic ? "dynamic" : "static") + "][exp_stats:" + (h->exp_stats.enabled ? "1" : "0") +
           "]");
  cumpsgemm::hijack_control::set_last_called_function_str(
      std::string(func_name) + "," + op_str(op_A) + "," + op_str(op_B) + "," + std::to_string(m) +
      "," + std::to_string(n) + "," + std::to_string(k) + "," +
      std::to_string(batched ? batch : 1) + "," + cuMpSGEMM_get_compute_mode_string(mode));

  if (mode == CUMPSGEMM_DRY_RUN) return CUBLAS_STATUS_SUCCESS;

  // Two-by-two inner problems with a power-of-two long side go to the dedicated FP32 kernels
  // whatever the mode, when switched on (reference: src/cumpsgemm_cublas.cu:269-338, :647-725;
  // (m, 2, 2) is tested before (2, n, 2), so m == n == 2 takes the first route).
  if (k == 2 && (g_mx2x2_enabled || env_flag("CUMPSGEMM_CUSTOM_GEMM_MX2X2", false))) {
    const bool long_m = n == 2 && (m & (m - 1)) == 0;
    const bool long_n = !long_m && m == 2 && (n & (n - 1)) == 0;
    if (long_m || long_n) {
      T alpha_t, beta_t;
      if (!fetch_scalars<T>(cublas_handle, stream, alpha, beta, &alpha_t, &beta_t))
        return CUBLAS_STATUS_INVALID_VALUE;
      cuMpSGEMM_set_stream(h, stream);
      const std::string tname = std::string(std::is_same<T, float>::value ? "s" : "c") + "gemm_" +
                                (batched ? "strided_batch_" : "") +
                                (long_m ? "Mx2x2" : "2xNx2");
      CallTimer timer(stream,
                      timer_name<T>(tname.c_str(), op_A, op_B, m, n, k, batched ? batch : 0));
      log_info(long_m ? " +---> gemm_Mx2x2" : " +---> gemm_2xNx2");
      return tiny_gemm<T>(h, long_m, op_A, op_B, long_m ? m : n, &alpha_t, a, lda, stridea, b,
                          ldb, strideb, &beta_t, c, ldc, stridec, batched ? batch : 1);
    }
  }

  if (mode == CUMPSGEMM_CUBLAS || mode == CUMPSGEMM_CUBLAS_FP16TC ||
      mode == CUMPSGEMM_CUBLAS_TF32TC || mode == CUMPSGEMM_CUBLAS_SIMT) {
    // ---------------------------------------------------------------- pass-through
    cublasGemmAlgo_t algo = CUBLAS_GEMM_DEFAULT;
    cublasComputeType_t compute_type = CUBLAS_COMPUTE_32F;
    if (mode == CUMPSGEMM_CUBLAS_TF32TC) {
      algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
      compute_type = CUBLAS_COMPUTE_32F_FAST_TF32;
    } else if (mode == CUMPSGEMM_CUBLAS_FP16TC) {
      algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
      compute_type = CUBLAS_COMPUTE_32F_FAST_16F;
    } else if (mode == CUMPSGEMM_CUBLAS) {
      // keep what the application asked its own handle for
      const std::string f(func_name);
      if (f.rfind("cublasSgemm", 0) == 0 || f.rfind("cublasCgemm", 0) == 0) {
        switch (math_mode_of(cublas_handle)) {
        case CUBLAS_TF32_TENSOR_OP_MATH:
          algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
          compute_type = CUBLAS_COMPUTE_32F_FAST_TF32;
          break;
        case CUBLAS_TENSOR_OP_MATH:
          algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
          compute_type = CUBLAS_COMPUTE_32F_FAST_16F;
          break;
        default:
          break;
        }
      }
    }
    CallTimer timer(stream, timer_name<T>(func_name, op_A, op_B, m, n, k, batched ? batch : 0));
    cublasStatus_t res;
    // The 64-bit entry points of the real cuBLAS take every size this layer accepts.
    if (!batched) {
      using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int64_t,
                                      int64_t, int64_t, const void *, const void *, cudaDataType,
                                      int64_t, const void *, cudaDataType, int64_t, const void *,
                                      void *, cudaDataType, int64_t, cublasComputeType_t,
                                      cublasGemmAlgo_t);
      static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmEx_64"));
      if (fn == nullptr) {
        log_error(std::string("Could not load the cuBLAS function \"") + func_name + "\"");
        return CUBLAS_STATUS_NOT_INITIALIZED;
      }
      res = fn(cublas_handle, op_A, op_B, static_cast<int64_t>(m), static_cast<int64_t>(n),
               static_cast<int64_t>(k), alpha, a, cuda_type<T>(), static_cast<int64_t>(lda), b,
               cuda_type<T>(), static_cast<int64_t>(ldb), beta, c, cuda_type<T>(),
               static_cast<int64_t>(ldc), compute_type, algo);
    } else {
      using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int64_t,
                                      int64_t, int64_t, const void *, const void *, cudaDataType,
                                      int64_t, long long int, const void *, cudaDataType, int64_t,
                                      long long int, const void *, void *, cudaDataType, int64_t,
                                      long long int, int64_t, cublasComputeType_t,
                                      cublasGemmAlgo_t);
      static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmStridedBatchedEx_64"));
      if (fn == nullptr) {
        log_error(std::string("Could not load the cuBLAS function \"") + func_name + "\"");
        return CUBLAS_STATUS_NOT_INITIALIZED;
      }
      res = fn(cublas_handle, op_A, op_B, static_cast<int64_t>(m), static_cast<int64_t>(n),
               static_cast<int64_t>(k), alpha, a, cuda_type<T>(), static_cast<int64_t>(lda),
               static_cast<long long>(stridea), b, cuda_type<T>(), static_cast<int64_t>(ldb),
               static_cast<long long>(strideb), beta, c, cuda_type<T>(), static_cast<int64_t>(ldc),
               static_cast<long long>(stridec), static_cast<int64_t>(batch), compute_type, algo);
    }
    if (h->exp_stats.enabled) {
      // statistics of the result, as the reference records for pass-through calls
      cuMpSGEMM_set_stream(h, stream);
      cumpsgemm::exp_stats_ext<T>(h, static_cast<unsigned>(m), static_cast<unsigned>(n), c,
                                  static_cast<unsigned>(ldc),
                                  static_cast<unsigned>(batched ? batch : 1),
                                  static_cast<unsigned>(batched ? stridec : 0));
    }
    return res;
  }

  // ------------------------------------------------------------------ cuMpSGEMM kernels
  T alpha_h, beta_h;
  if (!fetch_scalars<T>(cublas_handle, stream, alpha, beta, &alpha_h, &beta_h))
    return CUBLAS_STATUS_INVALID_VALUE;
  cuMpSGEMM_set_stream(h, stream);
  const std::string tname = std::string(std::is_same<T, float>::value ? "s" : "c") + "gemm_" +
                            (batched ? "strided_batch_" : "") +
                            cuMpSGEMM_get_compute_mode_string(mode);
  CallTimer timer(stream, timer_name<T>(tname.c_str(), op_A, op_B, m, n, k, batched ? batch : 0));
  const uint64_t nb = batched ? batch : 1;
  if (mode == CUMPSGEMM_AUTO || mode == CUMPSGEMM_FP16TCEC_SCALING) {
    unsigned id_a = 0, id_b = 0, flag_id = 0;
    const cublasStatus_t res = gemm_with_statistics<T>(
        h, op_A, op_B, m, n, k, &alpha_h, a, lda, stridea, b, ldb, strideb, &beta_h, c, ldc,
        stridec, nb, mode, &id_a, &id_b, &flag_id);
    if (mode == CUMPSGEMM_AUTO && res == CUBLAS_STATUS_SUCCESS)
      log_auto_decision(h, id_a, id_b, flag_id);
    return res;
  }
  return gemm_dispatch<T>(h, op_A, op_B, m, n, k, &alpha_h, a, lda, stridea, b, ldb, strideb,
                          &beta_h, c, ldc, stridec, nb, mode, nullptr, nullptr);
}

// Pointer-array batches (cublas{S,C}gemmBatched, cublasGemmBatchedEx with FP32 types).  The
// reference does not intercept these.  FP16TCEC / TF32TCEC (and the non-corrected modes) run on
// the cuMpSGEMM kernels; every other mode, including AUTO and FP16TCEC_SCALING whose statistics
// kernels take strided batches only, is forwarded to the real cublasGemmBatchedEx.
template <class T>
cublasStatus_t hijack_batched_core(const char *func_name, cublasHandle_t cublas_handle,
                                   cublasOperation_t op_A, cublasOperation_t op_B, int m, int n,
                                   int k, const T *alpha, const T *const *a_array, int lda,
                                   const T *const *b_array, int ldb, const T *beta,
                                   T *const *c_array, int ldc, int batch) {
  if (m <= 0 || n <= 0 || k <= 0 || lda <= 0 || ldb <= 0 || ldc <= 0 || batch <= 0)
    return CUBLAS_STATUS_INVALID_VALUE;
  cuMpSGEMM_handle_t h = global_handle();
  if (h == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  const cudaStream_t stream = stream_of(cublas_handle);
  const cuMpSGEMM_compute_mode_t mode = cuMpSGEMM_get_compute_mode_internal(
      func_name, cublas_handle, op_A, op_B, static_cast<unsigned>(m), static_cast<unsigned>(n),
      static_cast<unsigned>(k));
  std::lock_guard<std::mutex> call_lock(h->call_mutex);
  const bool dynamic = (g_hijack_mode == HijackMode::dynamic_mode);
  log_info(std::string(func_name) + " op=(" + op_str(op_A) + ", " + op_str(op_B) + "), shape=(" +
           std::to_string(m) + ", " + std::to_string(n) + ", " + std::to_string(k) +
           "), batch=" + std::to_string(batch) +
           ", mode=" + cuMpSGEMM_get_compute_mode_string(mode) + "[" +
           (dynamic ? "dynamic" : "static") + "][exp_stats:" + (h->exp_stats.enabled ? "1" : "0") +
           "]");
  cumpsgemm::hijack_control::set_last_called_function_str(
      std::string(func_name) + "," + op_str(op_A) + "," + op_str(op_B) + "," + std::to_string(m) +
      "," + std::to_string(n) + "," + std::to_string(k) + "," + std::to_string(batch) + "," +
      cuMpSGEMM_get_compute_mode_string(mode));
  if (mode == CUMPSGEMM_DRY_RUN) return CUBLAS_STATUS_SUCCESS;

  const bool own_kernels = (mode == CUMPSGEMM_FP16TCEC || mode == CUMPSGEMM_TF32TCEC ||
                            mode == CUMPSGEMM_FP16TC || mode == CUMPSGEMM_TF32TC);
  if (!own_kernels) {
    cublasGemmAlgo_t algo = CUBLAS_GEMM_DEFAULT;
    cublasComputeType_t compute_type = CUBLAS_COMPUTE_32F;
    if (mode == CUMPSGEMM_CUBLAS_TF32TC) {
      algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
      compute_type = CUBLAS_COMPUTE_32F_FAST_TF32;
    } else if (mode == CUMPSGEMM_CUBLAS_FP16TC) {
      algo = CUBLAS_GEMM_DEFAULT_TENSOR_OP;
      compute_type = CUBLAS_COMPUTE_32F_FAST_16F;
    }
    using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int,
                                    int, const void *, const void *const[], cudaDataType, int,
                                    const void *const[], cudaDataType, int, const void *,
                                    void *const[], cudaDataType, int, int, cublasComputeType_t,
                                    cublasGemmAlgo_t);
    static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmBatchedEx"));
    if (fn == nullptr) {
      log_error(std::string("Could not load the cuBLAS function \"") + func_name + "\"");
      return CUBLAS_STATUS_NOT_INITIALIZED;
    }
    return fn(cublas_handle, op_A, op_B, m, n, k, alpha,
              reinterpret_cast<const void *const *>(a_array), cuda_type<T>(), lda,
              reinterpret_cast<const void *const *>(b_array), cuda_type<T>(), ldb, beta,
              reinterpret_cast<void *const *>(c_array), cuda_type<T>(), ldc, batch, compute_type,
              algo);
  }
  T alpha_h, beta_h;
  if (!fetch_scalars<T>(cublas_handle, stream, alpha, beta, &alpha_h, &beta_h))
    return CUBLAS_STATUS_INVALID_VALUE;
  cuMpSGEMM_set_stream(h, stream);
  return gemm_dispatch<T>(h, op_A, op_B, m, n, k, &alpha_h, nullptr, lda, 0, nullptr, ldb, 0,
                          &beta_h, nullptr, ldc, 0, batch, mode, nullptr, nullptr, a_array, b_array,
                          c_array);
}

} // namespace

// ---------------------------------------------------------------- mode selection
extern "C" cuMpSGEMM_compute_mode_t cuMpSGEMM_get_compute_mode_internal(
    const char *const func_name, cublasHandle_t const cublas_handle, const cublasOperation_t op_A,
    const cublasOperation_t op_B, const unsigned m, const unsigned n, const unsigned k) {
  if (g_hijack_mode == HijackMode::dynamic_mode) {
    cumpsgemm::hijack_control::control_function_t f;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      f = g_control_func;
    }
    if (f) return f(op_A, op_B, m, n, k);
    const rule_fn_t rule = rule_library_function();
    if (rule != nullptr) return rule(func_name, cublas_handle, op_A, op_B, m, n, k);
    return cuMpSGEMM_get_compute_mode(func_name, cublas_handle, op_A, op_B, m, n, k);
  }
  return g_static_mode;
}

// ---------------------------------------------------------------- intercepted cuBLAS symbols
extern "C" {

cublasStatus_t cublasSgemm_v2(cublasHandle_t handle, cublasOperation_t transa,
                              cublasOperation_t transb, int m, int n, int k, const float *alpha,
                              const float *A, int lda, const float *B, int ldb, const float *beta,
                              float *C, int ldc) {
  if (m < 0 || n < 0 || k < 0 || lda < 0 || ldb < 0 || ldc < 0) return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<float>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, 0, B, ldb, 0,
                            beta, C, ldc, 0, 0, false);
}

cublasStatus_t cublasCgemm_v2(cublasHandle_t handle, cublasOperation_t transa,
                              cublasOperation_t transb, int m, int n, int k,
                              const cuComplex *alpha, const cuComplex *A, int lda,
                              const cuComplex *B, int ldb, const cuComplex *beta, cuComplex *C,
                              int ldc) {
  if (m < 0 || n < 0 || k < 0 || lda < 0 || ldb < 0 || ldc < 0) return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<cuComplex>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, 0, B,
                                ldb, 0, beta, C, ldc, 0, 0, false);
}

cublasStatus_t cublasSgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa,
                                         cublasOperation_t transb, int m, int n, int k,
                                         const float *alpha, const float *A, int lda,
                                         long long int strideA, const float *B, int ldb,
                                         long long int strideB, const float *beta, float *C,
                                         int ldc, long long int strideC, int batchCount) {
  if (m < 0 || n < 0 || k < 0 || lda < 0 || ldb < 0 || ldc < 0 || batchCount < 0 || strideA < 0 ||
      strideB < 0 || strideC < 0)
    return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<float>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, strideA, B,
                            ldb, strideB, beta, C, ldc, strideC, batchCount, true);
}

cublasStatus_t cublasCgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa,
                                         cublasOperation_t transb, int m, int n, int k,
                                         const cuComplex *alpha, const cuComplex *A, int lda,
                                         long long int strideA, const cuComplex *B, int ldb,
                                         long long int strideB, const cuComplex *beta,
                                         cuComplex *C, int ldc, long long int strideC,
                                         int batchCount) {
  if (m < 0 || n < 0 || k < 0 || lda < 0 || ldb < 0 || ldc < 0 || batchCount < 0 || strideA < 0 ||
      strideB < 0 || strideC < 0)
    return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<cuComplex>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, strideA,
                                B, ldb, strideB, beta, C, ldc, strideC, batchCount, true);
}

cublasStatus_t cublasGemmEx(cublasHandle_t handle, cublasOperation_t transa,
                            cublasOperation_t transb, int m, int n, int k, const void *alpha,
                            const void *A, cudaDataType_t Atype, int lda, const void *B,
                            cudaDataType_t Btype, int ldb, const void *beta, void *C,
                            cudaDataType_t Ctype, int ldc, cublasComputeType_t computeType,
                            cublasGemmAlgo_t algo) {
  if (m >= 0 && n >= 0 && k >= 0 && lda >= 0 && ldb >= 0 && ldc >= 0) {
    if (Atype == CUDA_R_32F && Btype == CUDA_R_32F && Ctype == CUDA_R_32F) {
      return hijack_core<float>(__func__, handle, transa, transb, m, n, k,
                                static_cast<const float *>(alpha), static_cast<const float *>(A),
                                lda, 0, static_cast<const float *>(B), ldb, 0,
                                static_cast<const float *>(beta), static_cast<float *>(C), ldc, 0,
                                0, false);
    }
    if (Atype == CUDA_C_32F && Btype == CUDA_C_32F && Ctype == CUDA_C_32F) {
      return hijack_core<cuComplex>(
          __func__, handle, transa, transb, m, n, k, static_cast<const cuComplex *>(alpha),
          static_cast<const cuComplex *>(A), lda, 0, static_cast<const cuComplex *>(B), ldb, 0,
          static_cast<const cuComplex *>(beta), static_cast<cuComplex *>(C), ldc, 0, 0, false);
    }
  }
  // every other type combination goes to the real cuBLAS untouched
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int,
                                  int, const void *, const void *, cudaDataType_t, int,
                                  const void *, cudaDataType_t, int, const void *, void *,
                                  cudaDataType_t, int, cublasComputeType_t, cublasGemmAlgo_t);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmEx"));
  if (fn == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  CallTimer timer(stream_of(handle), timer_name<float>(__func__, transa, transb, m, n, k, 0));
  return fn(handle, transa, transb, m, n, k, alpha, A, Atype, lda, B, Btype, ldb, beta, C, Ctype,
            ldc, computeType, algo);
}

cublasStatus_t cublasGemmStridedBatchedEx(
    cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n, int k,
    const void *alpha, const void *A, cudaDataType_t Atype, int lda, long long int strideA,
    const void *B, cudaDataType_t Btype, int ldb, long long int strideB, const void *beta, void *C,
    cudaDataType_t Ctype, int ldc, long long int strideC, int batchCount,
    cublasComputeType_t computeType, cublasGemmAlgo_t algo) {
  if (m >= 0 && n >= 0 && k >= 0 && lda >= 0 && ldb >= 0 && ldc >= 0 && batchCount >= 0 &&
      strideA >= 0 && strideB >= 0 && strideC >= 0) {
    if (Atype == CUDA_R_32F && Btype == CUDA_R_32F && Ctype == CUDA_R_32F) {
      return hijack_core<float>(__func__, handle, transa, transb, m, n, k,
                                static_cast<const float *>(alpha), static_cast<const float *>(A),
                                lda, strideA, static_cast<const float *>(B), ldb, strideB,
                                static_cast<const float *>(beta), static_cast<float *>(C), ldc,
                                strideC, batchCount, true);
    }
    if (Atype == CUDA_C_32F && Btype == CUDA_C_32F && Ctype == CUDA_C_32F) {
      return hijack_core<cuComplex>(
          __func__, handle, transa, transb, m, n, k, static_cast<const cuComplex *>(alpha),
          static_cast<const cuComplex *>(A), lda, strideA, static_cast<const cuComplex *>(B), ldb,
          strideB, static_cast<const cuComplex *>(beta), static_cast<cuComplex *>(C), ldc, strideC,
          batchCount, true);
    }
  }
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int,
                                  int, const void *, const void *, cudaDataType_t, int,
                                  long long int, const void *, cudaDataType_t, int, long long int,
                                  const void *, void *, cudaDataType_t, int, long long int, int,
                                  cublasComputeType_t, cublasGemmAlgo_t);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmStridedBatchedEx"));
  if (fn == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  CallTimer timer(stream_of(handle),
                  timer_name<float>(__func__, transa, transb, m, n, k, batchCount));
  return fn(handle, transa, transb, m, n, k, alpha, A, Atype, lda, strideA, B, Btype, ldb, strideB,
            beta, C, Ctype, ldc, strideC, batchCount, computeType, algo);
}

// ---- pointer-array batches
cublasStatus_t cublasSgemmBatched(cublasHandle_t handle, cublasOperation_t transa,
                                  cublasOperation_t transb, int m, int n, int k,
                                  const float *alpha, const float *const Aarray[], int lda,
                                  const float *const Barray[], int ldb, const float *beta,
                                  float *const Carray[], int ldc, int batchCount) {
  return hijack_batched_core<float>(__func__, handle, transa, transb, m, n, k, alpha, Aarray, lda,
                                    Barray, ldb, beta, Carray, ldc, batchCount);
}

cublasStatus_t cublasCgemmBatched(cublasHandle_t handle, cublasOperation_t transa,
                                  cublasOperation_t transb, int m, int n, int k,
                                  const cuComplex *alpha, const cuComplex *const Aarray[], int lda,
                                  const cuComplex *const Barray[], int ldb, const cuComplex *beta,
                                  cuComplex *const Carray[], int ldc, int batchCount) {
  return hijack_batched_core<cuComplex>(__func__, handle, transa, transb, m, n, k, alpha, Aarray,
                                        lda, Barray, ldb, beta, Carray, ldc, batchCount);
}

cublasStatus_t cublasGemmBatchedEx(cublasHandle_t handle, cublasOperation_t transa,
                                   cublasOperation_t transb, int m, int n, int k,
                                   const void *alpha, const void *const Aarray[],
                                   cudaDataType_t Atype, int lda, const void *const Barray[],
                                   cudaDataType_t Btype, int ldb, const void *beta,
                                   void *const Carray[], cudaDataType_t Ctype, int ldc,
                                   int batchCount, cublasComputeType_t computeType,
                                   cublasGemmAlgo_t algo) {
  if (Atype == CUDA_R_32F && Btype == CUDA_R_32F && Ctype == CUDA_R_32F) {
    return hijack_batched_core<float>(
        __func__, handle, transa, transb, m, n, k, static_cast<const float *>(alpha),
        reinterpret_cast<const float *const *>(Aarray), lda,
        reinterpret_cast<const float *const *>(Barray), ldb, static_cast<const float *>(beta),
        reinterpret_cast<float *const *>(Carray), ldc, batchCount);
  }
  if (Atype == CUDA_C_32F && Btype == CUDA_C_32F && Ctype == CUDA_C_32F) {
    return hijack_batched_core<cuComplex>(
        __func__, handle, transa, transb, m, n, k, static_cast<const cuComplex *>(alpha),
        reinterpret_cast<const cuComplex *const *>(Aarray), lda,
        reinterpret_cast<const cuComplex *const *>(Barray), ldb,
        static_cast<const cuComplex *>(beta), reinterpret_cast<cuComplex *const *>(Carray), ldc,
        batchCount);
  }
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int,
                                  int, const void *, const void *const[], cudaDataType_t, int,
                                  const void *const[], cudaDataType_t, int, const void *,
                                  void *const[], cudaDataType_t, int, int, cublasComputeType_t,
                                  cublasGemmAlgo_t);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmBatchedEx"));
  if (fn == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  return fn(handle, transa, transb, m, n, k, alpha, Aarray, Atype, lda, Barray, Btype, ldb, beta,
            Carray, Ctype, ldc, batchCount, computeType, algo);
}

// ---- 64-bit integer interface of cuBLAS 12 (cublas_api.h: cublasSgemm_v2_64, ...).  The
//      reference does not intercept these; applications built with CUBLAS_64 reach them.
#define CUMPSGEMM_NEG6(a, b, c, d, e, f) ((a) < 0 || (b) < 0 || (c) < 0 || (d) < 0 || (e) < 0 || (f) < 0)

cublasStatus_t cublasSgemm_v2_64(cublasHandle_t handle, cublasOperation_t transa,
                                 cublasOperation_t transb, int64_t m, int64_t n, int64_t k,
                                 const float *alpha, const float *A, int64_t lda, const float *B,
                                 int64_t ldb, const float *beta, float *C, int64_t ldc) {
  if (CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc)) return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<float>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, 0, B, ldb, 0,
                            beta, C, ldc, 0, 0, false);
}

cublasStatus_t cublasCgemm_v2_64(cublasHandle_t handle, cublasOperation_t transa,
                                 cublasOperation_t transb, int64_t m, int64_t n, int64_t k,
                                 const cuComplex *alpha, const cuComplex *A, int64_t lda,
                                 const cuComplex *B, int64_t ldb, const cuComplex *beta,
                                 cuComplex *C, int64_t ldc) {
  if (CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc)) return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<cuComplex>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, 0, B,
                                ldb, 0, beta, C, ldc, 0, 0, false);
}

cublasStatus_t cublasSgemmStridedBatched_64(cublasHandle_t handle, cublasOperation_t transa,
                                            cublasOperation_t transb, int64_t m, int64_t n,
                                            int64_t k, const float *alpha, const float *A,
                                            int64_t lda, long long int strideA, const float *B,
                                            int64_t ldb, long long int strideB, const float *beta,
                                            float *C, int64_t ldc, long long int strideC,
                                            int64_t batchCount) {
  if (CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc) || batchCount < 0 || strideA < 0 || strideB < 0 ||
      strideC < 0)
    return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<float>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, strideA, B,
                            ldb, strideB, beta, C, ldc, strideC, batchCount, true);
}

cublasStatus_t cublasCgemmStridedBatched_64(cublasHandle_t handle, cublasOperation_t transa,
                                            cublasOperation_t transb, int64_t m, int64_t n,
                                            int64_t k, const cuComplex *alpha, const cuComplex *A,
                                            int64_t lda, long long int strideA, const cuComplex *B,
                                            int64_t ldb, long long int strideB,
                                            const cuComplex *beta, cuComplex *C, int64_t ldc,
                                            long long int strideC, int64_t batchCount) {
  if (CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc) || batchCount < 0 || strideA < 0 || strideB < 0 ||
      strideC < 0)
    return CUBLAS_STATUS_INVALID_VALUE;
  return hijack_core<cuComplex>(__func__, handle, transa, transb, m, n, k, alpha, A, lda, strideA,
                                B, ldb, strideB, beta, C, ldc, strideC, batchCount, true);
}

cublasStatus_t cublasGemmEx_64(cublasHandle_t handle, cublasOperation_t transa,
                               cublasOperation_t transb, int64_t m, int64_t n, int64_t k,
                               const void *alpha, const void *A, cudaDataType_t Atype, int64_t lda,
                               const void *B, cudaDataType_t Btype, int64_t ldb, const void *beta,
                               void *C, cudaDataType_t Ctype, int64_t ldc,
                               cublasComputeType_t computeType, cublasGemmAlgo_t algo) {
  if (!CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc)) {
    if (Atype == CUDA_R_32F && Btype == CUDA_R_32F && Ctype == CUDA_R_32F) {
      return hijack_core<float>(__func__, handle, transa, transb, m, n, k,
                                static_cast<const float *>(alpha), static_cast<const float *>(A),
                                lda, 0, static_cast<const float *>(B), ldb, 0,
                                static_cast<const float *>(beta), static_cast<float *>(C), ldc, 0,
                                0, false);
    }
    if (Atype == CUDA_C_32F && Btype == CUDA_C_32F && Ctype == CUDA_C_32F) {
      return hijack_core<cuComplex>(
          __func__, handle, transa, transb, m, n, k, static_cast<const cuComplex *>(alpha),
          static_cast<const cuComplex *>(A), lda, 0, static_cast<const cuComplex *>(B), ldb, 0,
          static_cast<const cuComplex *>(beta), static_cast<cuComplex *>(C), ldc, 0, 0, false);
    }
  }
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int64_t,
                                  int64_t, int64_t, const void *, const void *, cudaDataType_t,
                                  int64_t, const void *, cudaDataType_t, int64_t, const void *,
                                  void *, cudaDataType_t, int64_t, cublasComputeType_t,
                                  cublasGemmAlgo_t);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmEx_64"));
  if (fn == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  return fn(handle, transa, transb, m, n, k, alpha, A, Atype, lda, B, Btype, ldb, beta, C, Ctype,
            ldc, computeType, algo);
}

cublasStatus_t cublasGemmStridedBatchedEx_64(
    cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int64_t m,
    int64_t n, int64_t k, const void *alpha, const void *A, cudaDataType_t Atype, int64_t lda,
    long long int strideA, const void *B, cudaDataType_t Btype, int64_t ldb, long long int strideB,
    const void *beta, void *C, cudaDataType_t Ctype, int64_t ldc, long long int strideC,
    int64_t batchCount, cublasComputeType_t computeType, cublasGemmAlgo_t algo) {
  if (!CUMPSGEMM_NEG6(m, n, k, lda, ldb, ldc) && batchCount >= 0 && strideA >= 0 &&
      strideB >= 0 && strideC >= 0) {
    if (Atype == CUDA_R_32F && Btype == CUDA_R_32F && Ctype == CUDA_R_32F) {
      return hijack_core<float>(__func__, handle, transa, transb, m, n, k,
                                static_cast<const float *>(alpha), static_cast<const float *>(A),
                                lda, strideA, static_cast<const float *>(B), ldb, strideB,
                                static_cast<const float *>(beta), static_cast<float *>(C), ldc,
                                strideC, batchCount, true);
    }
    if (Atype == CUDA_C_32F && Btype == CUDA_C_32F && Ctype == CUDA_C_32F) {
      return hijack_core<cuComplex>(
          __func__, handle, transa, transb, m, n, k, static_cast<const cuComplex *>(alpha),
          static_cast<const cuComplex *>(A), lda, strideA, static_cast<const cuComplex *>(B), ldb,
          strideB, static_cast<const cuComplex *>(beta), static_cast<cuComplex *>(C), ldc, strideC,
          batchCount, true);
    }
  }
  using fn_t = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int64_t,
                                  int64_t, int64_t, const void *, const void *, cudaDataType_t,
                                  int64_t, long long int, const void *, cudaDataType_t, int64_t,
                                  long long int, const void *, void *, cudaDataType_t, int64_t,
                                  long long int, int64_t, cublasComputeType_t, cublasGemmAlgo_t);
  static fn_t fn = reinterpret_cast<fn_t>(real_cublas_symbol("cublasGemmStridedBatchedEx_64"));
  if (fn == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  return fn(handle, transa, transb, m, n, k, alpha, A, Atype, lda, strideA, B, Btype, ldb, strideB,
            beta, C, Ctype, ldc, strideC, batchCount, computeType, algo);
}
#undef CUMPSGEMM_NEG6

} // extern "C"

// ---------------------------------------------------------------- hijack_control
namespace cumpsgemm {
namespace hijack_control {

cuMpSGEMM_handle_t get_internal_global_handle() { return global_handle(); }

void set_compute_mode(const cuMpSGEMM_compute_mode_t mode) {
  if (mode == CUMPSGEMM_FP32_SIMT) {
    throw std::runtime_error("CUMPSGEMM_FP32_SIMT mode is currently not supported.");
  }
  g_static_mode = mode;
  g_hijack_mode = HijackMode::static_mode;
}
void unset_compute_mode() { g_hijack_mode = HijackMode::dynamic_mode; }

void enable_custom_gemm_Mx2x2() { g_mx2x2_enabled = true; }
void disable_custom_gemm_Mx2x2() { g_mx2x2_enabled = false; }

void reset_exp_stats_buffer_id() {
  cuMpSGEMM_handle_t h = global_handle();
  if (h != nullptr) cumpsgemm::reset_exp_stats_buffer_id(h);
}

void set_exp_stats_params(const float ignore_threshold, const float underflow_threshold,
                          const float underflow_tolerance_rate) {
  log_info("AUTO config: ignore_threshold=" + sci(ignore_threshold) + " @" + __func__);
  log_info("AUTO config: underflow_threshold=" + sci(underflow_threshold) + " @" + __func__);
  log_info("AUTO config: underflow_tolerance_rate=" + sci(underflow_tolerance_rate) + " @" +
           __func__);
  cuMpSGEMM_handle_t h = global_handle();
  if (h != nullptr)
    cumpsgemm::set_exp_stats_params(h, ignore_threshold, underflow_threshold,
                                    underflow_tolerance_rate);
}

// A and B are never modified by this implementation, so there is nothing to restore; the
// switch is kept (and logged) for source compatibility.
void enable_restoring_AB_after_scaling() {
  g_restore_ab = true;
  log_info(std::string("AUTO config: restore_AB_scaling=True @") + __func__);
}
void disable_restoring_AB_after_scaling() {
  g_restore_ab = false;
  log_info(std::string("AUTO config: restore_AB_scaling=False @") + __func__);
}

std::string get_last_called_function_str() {
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_last_called;
}
void set_last_called_function_str(const std::string func_str) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_last_called = func_str;
}
void clear_last_called_function_str() { set_last_called_function_str(""); }

bool is_library_loaded() { return true; }

void set_control_function(const control_function_t control_function) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_control_func = control_function;
}
void unset_control_function() {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_control_func = nullptr;
}

} // namespace hijack_control
} // namespace cumpsgemm
