// Stand-in for cutf's bit-reinterpretation helper (called at src/exp_stats.cu:161, :455).
// TEST INFRASTRUCTURE ONLY, see ../math.hpp.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace cutf {
namespace experimental {
namespace fp {
__host__ __device__ inline std::uint32_t reinterpret_as_uint(const float v) {
#ifdef __CUDA_ARCH__
  return __float_as_uint(v);
#else
  union {
    float f;
    std::uint32_t u;
  } c;
  c.f = v;
  return c.u;
#endif
}
} // namespace fp
} // namespace experimental
} // namespace cutf
