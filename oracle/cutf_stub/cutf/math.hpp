// Stand-in for the two functions of the third-party `cutf` library's math header that the
// reference's statistics kernels call (src/exp_stats.cu:32-44, :118-152).  TEST
// INFRASTRUCTURE ONLY: it exists so that the reference's own exp_stats.cu /
// dynamic_scaling.cu / dynamic_launch.cu compile unmodified into the checker library
// oracle/_ref/libref_stats.so.  The product never includes it.
#pragma once
#include <cuda_runtime.h>

namespace cutf {
namespace math {
__host__ __device__ inline float abs(const float a) { return fabsf(a); }
__host__ __device__ inline float max(const float a, const float b) { return fmaxf(a, b); }
} // namespace math
} // namespace cutf
