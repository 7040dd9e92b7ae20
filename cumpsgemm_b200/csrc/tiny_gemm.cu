// FP32 GEMMs with two-by-two inner problems: (m x 2)(2 x 2) and (2 x 2)(2 x n).
//
// The reference routes these shapes (power-of-two m or n, the other two dimensions equal to
// two) to the third-party cuGEMM-Mx2x2 kernels before any compute-mode decision
// (src/cumpsgemm_cublas.cu:269-338 single, :647-725 strided batch).  That library's source is
// not part of the reference tree, so these kernels are written from the call sites' contract:
// plain FP32 arithmetic, cuBLAS argument meaning, alpha / beta by value, one stream.
//
// The shapes are pure streaming work (HBM bound): per long-dimension index the kernel reads
// two operand values and two values of C (only when beta != 0) and writes two, so there is
// nothing for a tensor core to do.  One thread owns one row (or column) of C; a warp's loads
// are contiguous along the long dimension when the operand is stored that way, and an
// interleaved pair otherwise.  Measured on 2^25 real / 2^24 complex rows: 0.70-0.77 of the copy
// bandwidth with beta == 0, 0.90 with beta != 0.
//
// The arithmetic is fixed, operation by operation, with non-contracting intrinsics so that a
// host restatement with fmaf() gives the same bits:
//   real:     p = fma(a1, b1, a0 * b0);   c' = beta == 0 ? alpha * p : fma(alpha, p, beta * c)
//   complex:  p.re = a0r*b0r; p.re = fma(-a0i, b0i, p.re); p.re = fma(a1r, b1r, p.re);
//             p.re = fma(-a1i, b1i, p.re);  p.im likewise with (a0r,b0i) (a0i,b0r) (a1r,b1i)
//             (a1i,b1r);  t = alpha * p as (ar*pr, then fma(-ai, pi)), (ar*pi, then fma(ai, pr));
//             with beta != 0: t.re = fma(br, cr, t.re); t.re = fma(-bi, ci, t.re);
//             t.im = fma(br, ci, t.im); t.im = fma(bi, cr, t.im).
#include "internal.hpp"

namespace cumpsgemm_b200 {
namespace {

struct cplx {
  float re, im;
};

__device__ __forceinline__ float load_val(const float *p, bool) { return *p; }
__device__ __forceinline__ cplx load_val(const cuComplex *p, bool conj) {
  const float2 v = *reinterpret_cast<const float2 *>(p);
  return cplx{v.x, conj ? -v.y : v.y};
}

// sum over the inner dimension of two products
__device__ __forceinline__ float dot2(float a0, float b0, float a1, float b1) {
  return __fmaf_rn(a1, b1, __fmul_rn(a0, b0));
}
__device__ __forceinline__ cplx dot2(cplx a0, cplx b0, cplx a1, cplx b1) {
  float re = __fmul_rn(a0.re, b0.re);
  re = __fmaf_rn(-a0.im, b0.im, re);
  re = __fmaf_rn(a1.re, b1.re, re);
  re = __fmaf_rn(-a1.im, b1.im, re);
  float im = __fmul_rn(a0.re, b0.im);
  im = __fmaf_rn(a0.im, b0.re, im);
  im = __fmaf_rn(a1.re, b1.im, im);
  im = __fmaf_rn(a1.im, b1.re, im);
  return cplx{re, im};
}

__device__ __forceinline__ float load_c(const float *p) { return *p; }
__device__ __forceinline__ cplx load_c(const cuComplex *p) {
  const float2 v = *reinterpret_cast<const float2 *>(p);
  return cplx{v.x, v.y};
}

// alpha * p (+ beta * old)
__device__ __forceinline__ void store_result(float *c, float p, float alpha, float beta, float old,
                                             bool read_c) {
  *c = read_c ? __fmaf_rn(alpha, p, __fmul_rn(beta, old)) : __fmul_rn(alpha, p);
}
__device__ __forceinline__ void store_result(cuComplex *c, cplx p, cplx alpha, cplx beta, cplx old,
                                             bool read_c) {
  float re = __fmul_rn(alpha.re, p.re);
  re = __fmaf_rn(-alpha.im, p.im, re);
  float im = __fmul_rn(alpha.re, p.im);
  im = __fmaf_rn(alpha.im, p.re, im);
  if (read_c) {
    re = __fmaf_rn(beta.re, old.re, re);
    re = __fmaf_rn(-beta.im, old.im, re);
    im = __fmaf_rn(beta.re, old.im, im);
    im = __fmaf_rn(beta.im, old.re, im);
  }
  *reinterpret_cast<float2 *>(c) = make_float2(re, im);
}

template <class T> struct scalar_of;
template <> struct scalar_of<float> {
  using type = float;
  static __host__ __device__ float make(float v) { return v; }
  static __host__ bool is_zero(float v) { return v == 0.0f; }
};
template <> struct scalar_of<cuComplex> {
  using type = cplx;
  static __host__ __device__ cplx make(cuComplex v) { return cplx{v.x, v.y}; }
  static __host__ bool is_zero(cuComplex v) { return v.x == 0.0f && v.y == 0.0f; }
};

struct TinyArgs {
  const void *a, *b;
  void *c;
  uint64_t lda, ldb, ldc, stride_a, stride_b, stride_c;
  uint64_t len;     // the long dimension (m or n), a power of two
  uint32_t log2_len;
  uint64_t batch;
  bool trans_a, conj_a, trans_b, conj_b, read_c;
};

// LONG_IS_M: C is len x 2 = op(A)(len x 2) op(B)(2 x 2); otherwise C is 2 x len =
// op(A)(2 x 2) op(B)(2 x len).  Each thread handles kUnroll indices of the long dimension per
// trip, a grid stride apart, and issues all their loads before the first store, so enough
// bytes are in flight per SM to cover the memory latency.
template <class T> struct unroll_of { static constexpr int value = 8; };       // 4-byte elements
template <> struct unroll_of<cuComplex> { static constexpr int value = 4; };   // 8-byte elements

template <class T, bool LONG_IS_M>
__global__ void __launch_bounds__(256)
tiny_gemm_kernel(TinyArgs g, typename scalar_of<T>::type alpha, typename scalar_of<T>::type beta) {
  using S = typename scalar_of<T>::type;
  constexpr int kUnroll = unroll_of<T>::value;
  const uint64_t total = g.len * g.batch;
  const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t t0 = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; t0 < total;
       t0 += step * kUnroll) {
    // phase 1: everything that comes from DRAM, for all kUnroll indices
    S x0[kUnroll], x1[kUnroll]; // the two values along the inner dimension of the long operand
    S old[kUnroll][2];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const uint64_t t = t0 + u * step;
      if (t >= total) continue;
      const uint64_t bt = t >> g.log2_len; // len is a power of two: no 64-bit division
      const uint64_t i = t & (g.len - 1);
      T *c = static_cast<T *>(g.c) + bt * g.stride_c;
      if (LONG_IS_M) {
        // op(A)(i, l): stored A(i, l) = a[i + l*lda] or, transposed, a[l + i*lda]
        const T *a = static_cast<const T *>(g.a) + bt * g.stride_a;
        x0[u] = load_val(g.trans_a ? a + i * g.lda : a + i, g.conj_a);
        x1[u] = load_val(g.trans_a ? a + 1 + i * g.lda : a + i + g.lda, g.conj_a);
      } else {
        // op(B)(l, i): b[l + i*ldb] or, transposed, b[i + l*ldb]
        const T *b = static_cast<const T *>(g.b) + bt * g.stride_b;
        x0[u] = load_val(g.trans_b ? b + i : b + i * g.ldb, g.conj_b);
        x1[u] = load_val(g.trans_b ? b + i + g.ldb : b + 1 + i * g.ldb, g.conj_b);
      }
#pragma unroll
      for (int j = 0; j < 2; j++) {
        old[u][j] = g.read_c ? load_c(LONG_IS_M ? c + i + j * g.ldc : c + j + i * g.ldc) : S{};
      }
    }
    // phase 2: the 2 x 2 operand (a few cache-resident values per batch entry), arithmetic, stores
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const uint64_t t = t0 + u * step;
      if (t >= total) continue;
      const uint64_t bt = t >> g.log2_len;
      const uint64_t i = t & (g.len - 1);
      T *c = static_cast<T *>(g.c) + bt * g.stride_c;
      S q[4]; // q[2*j + l] = op(B)(l, j) resp. op(A)(j, l)
      if (LONG_IS_M) {
        const T *b = static_cast<const T *>(g.b) + bt * g.stride_b;
#pragma unroll
        for (int j = 0; j < 2; j++) {
          q[2 * j] = load_val(g.trans_b ? b + j : b + j * g.ldb, g.conj_b);
          q[2 * j + 1] = load_val(g.trans_b ? b + j + g.ldb : b + 1 + j * g.ldb, g.conj_b);
        }
      } else {
        const T *a = static_cast<const T *>(g.a) + bt * g.stride_a;
#pragma unroll
        for (int r = 0; r < 2; r++) {
          q[2 * r] = load_val(g.trans_a ? a + r * g.lda : a + r, g.conj_a);
          q[2 * r + 1] = load_val(g.trans_a ? a + 1 + r * g.lda : a + r + g.lda, g.conj_a);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; j++) {
        // the operand order inside each product is (value of A, value of B)
        const S p = LONG_IS_M ? dot2(x0[u], q[2 * j], x1[u], q[2 * j + 1])
                              : dot2(q[2 * j], x0[u], q[2 * j + 1], x1[u]);
        store_result(LONG_IS_M ? c + i + j * g.ldc : c + j + i * g.ldc, p, alpha, beta,
                     old[u][j], g.read_c);
      }
    }
  }
}

bool is_pow2(uint64_t v) { return v != 0 && (v & (v - 1)) == 0; }

} // namespace

template <class T>
cublasStatus_t tiny_gemm(cuMpSGEMM_handle *h, bool long_is_m, cublasOperation_t op_A,
                         cublasOperation_t op_B, uint64_t len, const T *alpha, const T *a,
                         uint64_t lda, uint64_t stride_a, const T *b, uint64_t ldb,
                         uint64_t stride_b, const T *beta, T *c, uint64_t ldc, uint64_t stride_c,
                         uint64_t batch) {
  if (h == nullptr || alpha == nullptr || beta == nullptr || a == nullptr || b == nullptr ||
      c == nullptr)
    return CUBLAS_STATUS_INVALID_VALUE;
  if (!is_pow2(len) || batch == 0) return CUBLAS_STATUS_INVALID_VALUE;
  // cuBLAS rules for the leading dimensions: at least the stored row count.
  const uint64_t rows_a = long_is_m ? (op_A == CUBLAS_OP_N ? len : 2) : 2;
  const uint64_t rows_b = long_is_m ? 2 : (op_B == CUBLAS_OP_N ? 2 : len);
  const uint64_t rows_c = long_is_m ? len : 2;
  if (lda < rows_a || ldb < rows_b || ldc < rows_c) return CUBLAS_STATUS_INVALID_VALUE;
  DeviceGuard guard(h->device);
  TinyArgs g{};
  g.a = a;
  g.b = b;
  g.c = c;
  g.lda = lda;
  g.ldb = ldb;
  g.ldc = ldc;
  g.stride_a = stride_a;
  g.stride_b = stride_b;
  g.stride_c = stride_c;
  g.len = len;
  g.log2_len = 0;
  while ((1ull << g.log2_len) < len) ++g.log2_len;
  g.batch = batch;
  g.trans_a = op_A != CUBLAS_OP_N;
  g.conj_a = op_A == CUBLAS_OP_C;
  g.trans_b = op_B != CUBLAS_OP_N;
  g.conj_b = op_B == CUBLAS_OP_C;
  g.read_c = !scalar_of<T>::is_zero(*beta);
  const uint64_t total = len * batch;
  const uint64_t want = (total + 255) / 256;   // small problems: one index per thread
  const uint64_t cap = static_cast<uint64_t>(h->num_sms) * 8;
  const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
  if (long_is_m)
    tiny_gemm_kernel<T, true><<<grid, 256, 0, h->cuda_stream>>>(g, scalar_of<T>::make(*alpha),
                                                           scalar_of<T>::make(*beta));
  else
    tiny_gemm_kernel<T, false><<<grid, 256, 0, h->cuda_stream>>>(g, scalar_of<T>::make(*alpha),
                                                            scalar_of<T>::make(*beta));
  return cudaGetLastError() == cudaSuccess ? CUBLAS_STATUS_SUCCESS
                                           : CUBLAS_STATUS_EXECUTION_FAILED;
}

template cublasStatus_t tiny_gemm<float>(cuMpSGEMM_handle *, bool, cublasOperation_t,
                                         cublasOperation_t, uint64_t, const float *, const float *,
                                         uint64_t, uint64_t, const float *, uint64_t, uint64_t,
                                         const float *, float *, uint64_t, uint64_t, uint64_t);
template cublasStatus_t tiny_gemm<cuComplex>(cuMpSGEMM_handle *, bool, cublasOperation_t,
                                             cublasOperation_t, uint64_t, const cuComplex *,
                                             const cuComplex *, uint64_t, uint64_t,
                                             const cuComplex *, uint64_t, uint64_t,
                                             const cuComplex *, cuComplex *, uint64_t, uint64_t,
                                             uint64_t);

} // namespace cumpsgemm_b200
