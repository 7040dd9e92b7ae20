// Default compute-mode rule, built both into libcumpsgemm.so (fallback) and
// as libcumpsgemm_rule.so (the library users replace with their own rule).
//
// Behaviour follows the reference's src/default_cumpsgemm_rule.cu:6-49:
// any of m, n, k <= 1024 -> CUBLAS_SIMT; otherwise the value of
// CUMPSGEMM_COMPUTE_MODE selects the mode.  An unset variable selects
// CUMPSGEMM_CUBLAS quietly (the reference dereferences a null string there);
// an unknown value logs an error and selects CUMPSGEMM_CUBLAS.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cumpsgemm/cumpsgemm.h>

extern "C" cuMpSGEMM_compute_mode_t cuMpSGEMM_get_compute_mode(
    const char *const /*func_name*/, cublasHandle_t const /*cublas_handle*/,
    const cublasOperation_t /*op_A*/, const cublasOperation_t /*op_B*/, const unsigned m,
    const unsigned n, const unsigned k) {
  if (m <= 1024 || n <= 1024 || k <= 1024) return CUMPSGEMM_CUBLAS_SIMT;

  const char *env = std::getenv("CUMPSGEMM_COMPUTE_MODE");
  if (env == nullptr) return CUMPSGEMM_CUBLAS;

  static const struct {
    const char *name;
    cuMpSGEMM_compute_mode_t mode;
  } table[] = {
      {"FP16TCEC", CUMPSGEMM_FP16TCEC},
      {"TF32TCEC", CUMPSGEMM_TF32TCEC},
      {"FP16TC", CUMPSGEMM_FP16TC},
      {"TF32TC", CUMPSGEMM_TF32TC},
      {"CUBLAS_TF32TC", CUMPSGEMM_CUBLAS_TF32TC},
      {"CUBLAS_FP16TC", CUMPSGEMM_CUBLAS_FP16TC},
      {"CUBLAS_SIMT", CUMPSGEMM_CUBLAS_SIMT},
      {"CUBLAS", CUMPSGEMM_CUBLAS},
      {"DRY_RUN", CUMPSGEMM_DRY_RUN},
      {"AUTO", CUMPSGEMM_AUTO},
      {"FP16TCEC_SCALING", CUMPSGEMM_FP16TCEC_SCALING},
  };
  for (const auto &e : table) {
    if (std::strcmp(env, e.name) == 0) return e.mode;
  }
  const char *err_env = std::getenv("CUMPSGEMM_ERROR_LOG");
  if (err_env == nullptr || std::strcmp(err_env, "0") != 0) {
    std::fprintf(stdout, "[cuMpSGEMM ERROR] Unknown CUMPSGEMM_COMPUTE_MODE = %s. Ignored\n", env);
    std::fflush(stdout);
  }
  return CUMPSGEMM_CUBLAS;
}
