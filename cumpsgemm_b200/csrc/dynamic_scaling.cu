// Power-of-two operand scaling and the device-resident dynamic-launch flags.
//
// Semantics follow the reference:
//   src/dynamic_scaling.cu:15        target exponent 2^14
//   src/dynamic_scaling.cu:75-97     scale_A / scale_B:  X *= 2^14 / max_exp(X)   (gated by flag bit, skipped when max == 0)
//   src/dynamic_scaling.cu:99-126    scale_C:            C *= prod(max_exp / 2^14) over the operands whose bit is set
//   src/dynamic_scaling.cu:128-150   reset_scale_A / B:  X *= max_exp(X) / 2^14
//   src/dynamic_scaling.cu:364-385   flag word from the statistics decisions of A and B
//   src/dynamic_launch.cu:6-9        reserved slots: flag[0] = TF32TCEC, flag[1] = FP16TCEC | scaleA | scaleB
//   src/dynamic_launch.cu:36-70      ring ids, enable / disable
// One scalar per operand for the whole (batched) matrix, as in the reference.
// The kernels use 128-bit accesses in a persistent grid; 64-bit indices.
#include "internal.hpp"

namespace cumpsgemm_b200 {
namespace {

constexpr int THREADS = 256;
constexpr int CHUNK = 4096;

struct ScaleParams {
  float *ptr;
  uint64_t m, n, ld, stride; // floats
  uint32_t batch;
  uint64_t chunks_per_col, items;
  int vec_ok;
};

ScaleParams make_scale(void *ptr, uint64_t m, uint64_t n, uint64_t ld, uint32_t batch,
                       uint64_t stride, int fpe) {
  ScaleParams s;
  s.ptr = reinterpret_cast<float *>(ptr);
  s.m = m * fpe;
  s.n = n;
  s.ld = ld * fpe;
  s.stride = stride * fpe;
  s.batch = (stride == 0) ? 1u : batch;
  if (s.ld == s.m) {
    s.m *= s.n;
    s.n = 1;
    s.ld = s.m;
    if (s.batch > 1 && s.stride == s.m) {
      s.m *= s.batch;
      s.ld = s.m;
      s.batch = 1;
    }
  }
  s.chunks_per_col = (s.m + CHUNK - 1) / CHUNK;
  s.items = static_cast<uint64_t>(s.batch) * s.n * s.chunks_per_col;
  s.vec_ok = ((reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) && (s.ld % 4 == 0) &&
             (s.stride % 4 == 0);
  return s;
}

__device__ __forceinline__ void scale_items(const ScaleParams &s, float coef) {
  for (uint64_t item = blockIdx.x; item < s.items; item += gridDim.x) {
    const uint64_t chunk = item % s.chunks_per_col;
    const uint64_t col_id = item / s.chunks_per_col;
    const uint64_t col = col_id % s.n;
    const uint64_t b = col_id / s.n;
    float *p = s.ptr + b * s.stride + col * s.ld;
    const uint64_t begin = chunk * CHUNK;
    const uint64_t end = min(s.m, begin + CHUNK);
    if (s.vec_ok) {
      const uint64_t vec_end = begin + ((end - begin) & ~3ull);
      for (uint64_t i = begin + threadIdx.x * 4ull; i < vec_end; i += THREADS * 4ull) {
        float4 v = *reinterpret_cast<float4 *>(p + i);
        v.x *= coef;
        v.y *= coef;
        v.z *= coef;
        v.w *= coef;
        *reinterpret_cast<float4 *>(p + i) = v;
      }
      for (uint64_t i = vec_end + threadIdx.x; i < end; i += THREADS) p[i] *= coef;
    } else {
      for (uint64_t i = begin + threadIdx.x; i < end; i += THREADS) p[i] *= coef;
    }
  }
}

// which: 0 = operand A, 1 = operand B.  inverse = false: X *= 2^14 / max; true: X *= max / 2^14.
__global__ void __launch_bounds__(THREADS)
    scale_ab_kernel(const ScaleParams s, const int *flag, const float *max_slot, int which,
                    int inverse) {
  if (flag != nullptr) {
    const int f = *flag;
    if (which == 0 && !flag_scale_a(f)) return;
    if (which == 1 && !flag_scale_b(f)) return;
  }
  const float mx = *max_slot;
  if (mx == 0.f) return;
  const float coef = inverse ? (mx / kHalfExpMax) : (kHalfExpMax / mx);
  scale_items(s, coef);
}

__global__ void __launch_bounds__(THREADS)
    scale_c_kernel(const ScaleParams s, const int *flag, const float *max_a, const float *max_b) {
  const float ma = *max_a, mb = *max_b;
  if (ma == 0.f || mb == 0.f) return;
  float coef = 1.f;
  if (flag != nullptr) {
    const int f = *flag;
    if (!flag_scale_a(f) && !flag_scale_b(f)) return;
    if (flag_scale_a(f)) coef *= ma / kHalfExpMax;
    if (flag_scale_b(f)) coef *= mb / kHalfExpMax;
  } else {
    coef = (ma * mb) / (kHalfExpMax * kHalfExpMax);
  }
  scale_items(s, coef);
}

__global__ void flag_from_stats_kernel(int *flag, const int *mode_a, const int *mode_b) {
  const int pa = *mode_a, pb = *mode_b;
  if (pa == CUMPSGEMM_TF32TCEC || pb == CUMPSGEMM_TF32TCEC) {
    *flag = CUMPSGEMM_TF32TCEC;
    return;
  }
  int f = CUMPSGEMM_FP16TCEC;
  if (pa == CUMPSGEMM_FP16TCEC_SCALING) f |= kFlagScaleA;
  if (pb == CUMPSGEMM_FP16TCEC_SCALING) f |= kFlagScaleB;
  *flag = f;
}

__global__ void init_flag_buffer_kernel(int *flag) {
  flag[0] = CUMPSGEMM_TF32TCEC;
  flag[1] = CUMPSGEMM_FP16TCEC | kFlagScaleA | kFlagScaleB;
}

// Constants of the fused path.  An operand is scaled iff its flag bit is set
// and its max exponent is non-zero; the product is un-scaled by exactly the
// inverse of what was applied.
__global__ void dyn_params_kernel(DynParams *out, const int *flag, const float *max_a,
                                  const float *max_b) {
  CUMPSGEMM_CHAINED_KERNEL_ENTRY();
  const int f = *flag;
  const float ma = *max_a, mb = *max_b;
  const bool sa = flag_scale_a(f) && ma != 0.f;
  const bool sb = flag_scale_b(f) && mb != 0.f;
  out->scale_a = sa ? kHalfExpMax / ma : 1.f;
  out->scale_b = sb ? kHalfExpMax / mb : 1.f;
  out->unscale_c = (sa ? ma / kHalfExpMax : 1.f) * (sb ? mb / kHalfExpMax : 1.f);
  const int mode = flag_gemm_mode(f);
  out->gemm_mode = (mode == CUMPSGEMM_TF32TCEC) ? CUMPSGEMM_TF32TCEC : CUMPSGEMM_FP16TCEC;
}

// flag_from_stats_kernel and dyn_params_kernel in one launch (the AUTO path of a GEMM call).
__global__ void flag_and_dyn_params_kernel(DynParams *out, int *flag, const int *mode_a,
                                           const int *mode_b, const float *max_a,
                                           const float *max_b) {
  CUMPSGEMM_CHAINED_KERNEL_ENTRY();
  const int pa = *mode_a, pb = *mode_b;
  int f;
  if (pa == CUMPSGEMM_TF32TCEC || pb == CUMPSGEMM_TF32TCEC) {
    f = CUMPSGEMM_TF32TCEC;
  } else {
    f = CUMPSGEMM_FP16TCEC;
    if (pa == CUMPSGEMM_FP16TCEC_SCALING) f |= kFlagScaleA;
    if (pb == CUMPSGEMM_FP16TCEC_SCALING) f |= kFlagScaleB;
  }
  *flag = f;
  const float ma = *max_a, mb = *max_b;
  const bool sa = flag_scale_a(f) && ma != 0.f;
  const bool sb = flag_scale_b(f) && mb != 0.f;
  out->scale_a = sa ? kHalfExpMax / ma : 1.f;
  out->scale_b = sb ? kHalfExpMax / mb : 1.f;
  out->unscale_c = (sa ? ma / kHalfExpMax : 1.f) * (sb ? mb / kHalfExpMax : 1.f);
  const int mode = flag_gemm_mode(f);
  out->gemm_mode = (mode == CUMPSGEMM_TF32TCEC) ? CUMPSGEMM_TF32TCEC : CUMPSGEMM_FP16TCEC;
}

unsigned scale_grid(const cuMpSGEMM_handle *h, const ScaleParams &s) {
  const uint64_t cap = static_cast<uint64_t>(h->num_sms) * 8;
  return static_cast<unsigned>(s.items < cap ? (s.items ? s.items : 1) : cap);
}

} // namespace

unsigned next_dyn_launch_id(cuMpSGEMM_handle *h) {
  const unsigned next = ++(h->dyn_launch.current_buffer_id);
  if (next < h->dyn_launch.flag_buffer_length) return next;
  // wrap the ring back to the first non-reserved slot
  h->dyn_launch.current_buffer_id = 2;
  return 2;
}

void init_flag_buffer(cuMpSGEMM_handle *h) {
  init_flag_buffer_kernel<<<1, 1, 0, h->cuda_stream>>>(h->dyn_launch.flag_buffer);
}

template <class T>
void launch_scaling(cuMpSGEMM_handle *h, ScaleOp op, unsigned m, unsigned n, T *ptr, unsigned ld,
                    unsigned batch, unsigned stride, unsigned stats_id_a, unsigned stats_id_b,
                    unsigned flag_id) {
  DeviceGuard guard(h->device);
  const ScaleParams s = make_scale(ptr, m, n, ld, batch, stride, sizeof(T) / sizeof(float));
  const int *flag = h->dyn_launch.flag_buffer + flag_id;
  const unsigned grid = scale_grid(h, s);
  const bool prof = h->exp_stats.profiling_enabled;
  switch (op) {
  case ScaleOp::scale_a:
  case ScaleOp::scale_b:
    if (prof) h->exp_stats.profiler.start("scaling_AB", h->cuda_stream);
    scale_ab_kernel<<<grid, THREADS, 0, h->cuda_stream>>>(
        s, flag, h->exp_stats.dev_max + stats_id_a, op == ScaleOp::scale_a ? 0 : 1, 0);
    if (prof) h->exp_stats.profiler.stop("scaling_AB", h->cuda_stream);
    break;
  case ScaleOp::reset_a:
  case ScaleOp::reset_b:
    scale_ab_kernel<<<grid, THREADS, 0, h->cuda_stream>>>(
        s, flag, h->exp_stats.dev_max + stats_id_a, op == ScaleOp::reset_a ? 0 : 1, 1);
    break;
  case ScaleOp::scale_c:
    if (prof) h->exp_stats.profiler.start("scaling_C", h->cuda_stream);
    scale_c_kernel<<<grid, THREADS, 0, h->cuda_stream>>>(s, flag, h->exp_stats.dev_max + stats_id_a,
                                                         h->exp_stats.dev_max + stats_id_b);
    if (prof) h->exp_stats.profiler.stop("scaling_C", h->cuda_stream);
    break;
  }
}
template void launch_scaling<float>(cuMpSGEMM_handle *, ScaleOp, unsigned, unsigned, float *,
                                    unsigned, unsigned, unsigned, unsigned, unsigned, unsigned);
template void launch_scaling<cuComplex>(cuMpSGEMM_handle *, ScaleOp, unsigned, unsigned,
                                        cuComplex *, unsigned, unsigned, unsigned, unsigned,
                                        unsigned, unsigned);

DynParams *prepare_dyn_params(cuMpSGEMM_handle *h, unsigned flag_id, unsigned stats_id_a,
                              unsigned stats_id_b) {
  DynParams *slot = h->dev_dyn_params + h->dyn_params_next;
  h->dyn_params_next = (h->dyn_params_next + 1) % h->dyn_params_length;
  launch_chained(dyn_params_kernel, 1, 1, 0, h->cuda_stream, slot,
                 static_cast<const int *>(h->dyn_launch.flag_buffer + flag_id),
                 static_cast<const float *>(h->exp_stats.dev_max + stats_id_a),
                 static_cast<const float *>(h->exp_stats.dev_max + stats_id_b));
  return slot;
}

DynParams *prepare_dyn_params_from_stats(cuMpSGEMM_handle *h, unsigned flag_id,
                                         unsigned stats_id_a, unsigned stats_id_b) {
  DynParams *slot = h->dev_dyn_params + h->dyn_params_next;
  h->dyn_params_next = (h->dyn_params_next + 1) % h->dyn_params_length;
  launch_chained(flag_and_dyn_params_kernel, 1, 1, 0, h->cuda_stream, slot,
                 h->dyn_launch.flag_buffer + flag_id,
                 static_cast<const int *>(h->exp_stats.dev_mode + stats_id_a),
                 static_cast<const int *>(h->exp_stats.dev_mode + stats_id_b),
                 static_cast<const float *>(h->exp_stats.dev_max + stats_id_a),
                 static_cast<const float *>(h->exp_stats.dev_max + stats_id_b));
  return slot;
}

} // namespace cumpsgemm_b200

// ---------------------------------------------------------------- public C++ API
namespace cumpsgemm {
using namespace cumpsgemm_b200;

template <class T>
void scale_A(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
             const unsigned dynamic_launch_flag_buffer_id, const unsigned m, const unsigned n,
             T *const ptr, const unsigned ld, const unsigned batch_size, const unsigned stride) {
  launch_scaling<T>(handle, ScaleOp::scale_a, m, n, ptr, ld, batch_size, stride,
                    exp_stats_buffer_id, 0, dynamic_launch_flag_buffer_id);
}
template <class T>
void scale_B(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
             const unsigned dynamic_launch_flag_buffer_id, const unsigned m, const unsigned n,
             T *const ptr, const unsigned ld, const unsigned batch_size, const unsigned stride) {
  launch_scaling<T>(handle, ScaleOp::scale_b, m, n, ptr, ld, batch_size, stride,
                    exp_stats_buffer_id, 0, dynamic_launch_flag_buffer_id);
}
template <class T>
void scale_C(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_A_id,
             const unsigned exp_stats_buffer_B_id, const unsigned dynamic_launch_flag_buffer_id,
             const unsigned m, const unsigned n, T *const ptr, const unsigned ld,
             const unsigned batch_size, const unsigned stride) {
  launch_scaling<T>(handle, ScaleOp::scale_c, m, n, ptr, ld, batch_size, stride,
                    exp_stats_buffer_A_id, exp_stats_buffer_B_id, dynamic_launch_flag_buffer_id);
}
template <class T>
void reset_scale_A(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
                   const unsigned dynamic_launch_flag_buffer_id, const unsigned m,
                   const unsigned n, T *const ptr, const unsigned ld, const unsigned batch_size,
                   const unsigned stride) {
  launch_scaling<T>(handle, ScaleOp::reset_a, m, n, ptr, ld, batch_size, stride,
                    exp_stats_buffer_id, 0, dynamic_launch_flag_buffer_id);
}
template <class T>
void reset_scale_B(cuMpSGEMM_handle_t handle, const unsigned exp_stats_buffer_id,
                   const unsigned dynamic_launch_flag_buffer_id, const unsigned m,
                   const unsigned n, T *const ptr, const unsigned ld, const unsigned batch_size,
                   const unsigned stride) {
  launch_scaling<T>(handle, ScaleOp::reset_b, m, n, ptr, ld, batch_size, stride,
                    exp_stats_buffer_id, 0, dynamic_launch_flag_buffer_id);
}

#define INSTANTIATE(T)                                                                          \
  template void scale_A<T>(cuMpSGEMM_handle_t, const unsigned, const unsigned, const unsigned,  \
                           const unsigned, T *const, const unsigned, const unsigned,            \
                           const unsigned);                                                     \
  template void scale_B<T>(cuMpSGEMM_handle_t, const unsigned, const unsigned, const unsigned,  \
                           const unsigned, T *const, const unsigned, const unsigned,            \
                           const unsigned);                                                     \
  template void scale_C<T>(cuMpSGEMM_handle_t, const unsigned, const unsigned, const unsigned,  \
                           const unsigned, const unsigned, T *const, const unsigned,            \
                           const unsigned, const unsigned);                                     \
  template void reset_scale_A<T>(cuMpSGEMM_handle_t, const unsigned, const unsigned,            \
                                 const unsigned, const unsigned, T *const, const unsigned,      \
                                 const unsigned, const unsigned);                               \
  template void reset_scale_B<T>(cuMpSGEMM_handle_t, const unsigned, const unsigned,            \
                                 const unsigned, const unsigned, T *const, const unsigned,      \
                                 const unsigned, const unsigned);
INSTANTIATE(float)
INSTANTIATE(cuComplex)
#undef INSTANTIATE

unsigned get_current_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle) {
  return handle->dyn_launch.current_buffer_id;
}
unsigned get_next_dynamic_launch_buffer_id(cuMpSGEMM_handle_t handle) {
  return next_dyn_launch_id(handle);
}

static int read_flag(cuMpSGEMM_handle_t handle, unsigned id) {
  DeviceGuard guard(handle->device);
  int f = 0;
  cudaMemcpyAsync(&f, handle->dyn_launch.flag_buffer + id, sizeof(int), cudaMemcpyDeviceToHost,
                  handle->cuda_stream);
  cudaStreamSynchronize(handle->cuda_stream);
  return f;
}

cuMpSGEMM_compute_mode_t get_dynamic_launch_gemm_compute_mode(cuMpSGEMM_handle_t handle,
                                                              const unsigned buffer_id) {
  return static_cast<cuMpSGEMM_compute_mode_t>(flag_gemm_mode(read_flag(handle, buffer_id)));
}

std::pair<int, int> get_dynamic_launch_scaling_mode_AB(cuMpSGEMM_handle_t handle,
                                                       const unsigned buffer_id) {
  const int f = read_flag(handle, buffer_id);
  return std::pair<int, int>{flag_scale_a(f) ? 1 : 0, flag_scale_b(f) ? 1 : 0};
}

void set_dynamic_launch_buffer_by_exp_stats(cuMpSGEMM_handle *handle,
                                            const unsigned dynamic_launch_buffer_id,
                                            const unsigned A_exp_stats_buffer_id,
                                            const unsigned B_exp_stats_buffer_id) {
  DeviceGuard guard(handle->device);
  flag_from_stats_kernel<<<1, 1, 0, handle->cuda_stream>>>(
      handle->dyn_launch.flag_buffer + dynamic_launch_buffer_id,
      handle->exp_stats.dev_mode + A_exp_stats_buffer_id,
      handle->exp_stats.dev_mode + B_exp_stats_buffer_id);
}
} // namespace cumpsgemm
