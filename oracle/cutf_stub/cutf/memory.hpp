// Stand-in for the parts of cutf's memory header the reference uses: the error-check macro,
// a typed copy with automatic direction (src/exp_stats.cu:679, src/dynamic_launch.cu:54) and
// a pinned host buffer that kernels may write (src/exp_stats.cu:618-626).
// TEST INFRASTRUCTURE ONLY, see math.hpp.
#pragma once
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <memory>

#include <cuda_runtime.h>

#ifndef CUTF_CHECK_ERROR
#define CUTF_CHECK_ERROR(call)                                                                   \
  do {                                                                                           \
    const cudaError_t cutf_stub_err = (call);                                                    \
    if (cutf_stub_err != cudaSuccess) {                                                          \
      std::fprintf(stderr, "[reference checker] %s failed: %s (%s:%d)\n", #call,                \
                   cudaGetErrorString(cutf_stub_err), __FILE__, __LINE__);                       \
      std::abort();                                                                              \
    }                                                                                            \
  } while (0)
#endif

namespace cutf {
namespace memory {
template <class T> inline void copy(T *dst, const T *src, const std::size_t count) {
  CUTF_CHECK_ERROR(cudaMemcpy(dst, src, sizeof(T) * count, cudaMemcpyDefault));
}

struct host_deleter {
  void operator()(void *p) const { cudaFreeHost(p); }
};
template <class T> using host_unique_ptr = std::unique_ptr<T, host_deleter>;

// Page-locked, device-visible host memory (kernels of the reference store into it).
template <class T> inline host_unique_ptr<T> get_host_unique_ptr(const std::size_t count) {
  T *p = nullptr;
  CUTF_CHECK_ERROR(cudaHostAlloc(reinterpret_cast<void **>(&p), sizeof(T) * count,
                                 cudaHostAllocMapped | cudaHostAllocPortable));
  return host_unique_ptr<T>(p);
}
} // namespace memory
} // namespace cutf
