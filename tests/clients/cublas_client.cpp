// Minimal cuBLAS application used by the interception tests: it knows nothing about
// cuMpSGEMM and is run with and without LD_PRELOAD=libcumpsgemm.so.
//   cublas_client <s|c|sb|ex> <m> <n> <k>
// Prints "RESIDUAL <relative Frobenius residual vs FP64 host GEMM>" and "STATUS <n>".
#include <cmath>
#include <complex>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <vector>

static float frand(unsigned &s) {
  s = s * 1664525u + 1013904223u;
  return ((s >> 8) & 0xffffff) / 8388608.0f - 1.0f;
}

int main(int argc, char **argv) {
  if (argc < 5) return 2;
  const char *kind = argv[1];
  const int m = atoi(argv[2]), n = atoi(argv[3]), k = atoi(argv[4]);
  cublasHandle_t h;
  if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) return 3;
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  cublasSetStream(h, stream);
  unsigned seed = 12345;
  cublasStatus_t st = CUBLAS_STATUS_SUCCESS;
  double base = 0, diff = 0;
  if (!strcmp(kind, "c")) {
    std::vector<std::complex<float>> a((size_t)m * k), b((size_t)k * n), c((size_t)m * n);
    for (auto &x : a) x = {frand(seed), frand(seed)};
    for (auto &x : b) x = {frand(seed), frand(seed)};
    cuComplex *da, *db, *dc;
    cudaMalloc(&da, a.size() * 8); cudaMalloc(&db, b.size() * 8); cudaMalloc(&dc, c.size() * 8);
    cudaMemcpy(da, a.data(), a.size() * 8, cudaMemcpyHostToDevice);
    cudaMemcpy(db, b.data(), b.size() * 8, cudaMemcpyHostToDevice);
    const cuComplex alpha = {1.f, 0.f}, beta = {0.f, 0.f};
    st = cublasCgemm(h, CUBLAS_OP_N, CUBLAS_OP_N, m, n, k, &alpha, da, m, db, k, &beta, dc, m);
    cudaStreamSynchronize(stream);
    cudaMemcpy(c.data(), dc, c.size() * 8, cudaMemcpyDeviceToHost);
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < m; ++i) {
        std::complex<double> s = 0;
        for (int l = 0; l < k; ++l)
          s += std::complex<double>(a[i + (size_t)l * m]) * std::complex<double>(b[l + (size_t)j * k]);
        base += std::norm(s);
        diff += std::norm(s - std::complex<double>(c[i + (size_t)j * m]));
      }
  } else {
    const int batch = !strcmp(kind, "sb") ? 3 : 1;
    std::vector<float> a((size_t)m * k * batch), b((size_t)k * n * batch), c((size_t)m * n * batch);
    for (auto &x : a) x = frand(seed);
    for (auto &x : b) x = frand(seed);
    float *da, *db, *dc;
    cudaMalloc(&da, a.size() * 4); cudaMalloc(&db, b.size() * 4); cudaMalloc(&dc, c.size() * 4);
    cudaMemcpy(da, a.data(), a.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(db, b.data(), b.size() * 4, cudaMemcpyHostToDevice);
    const float alpha = 1.f, beta = 0.f;
    if (!strcmp(kind, "s")) {
      st = cublasSgemm(h, CUBLAS_OP_N, CUBLAS_OP_N, m, n, k, &alpha, da, m, db, k, &beta, dc, m);
    } else if (!strcmp(kind, "sb")) {
      st = cublasSgemmStridedBatched(h, CUBLAS_OP_N, CUBLAS_OP_N, m, n, k, &alpha, da, m,
                                     (long long)m * k, db, k, (long long)k * n, &beta, dc, m,
                                     (long long)m * n, batch);
    } else {
      st = cublasGemmEx(h, CUBLAS_OP_N, CUBLAS_OP_N, m, n, k, &alpha, da, CUDA_R_32F, m, db,
                        CUDA_R_32F, k, &beta, dc, CUDA_R_32F, m, CUBLAS_COMPUTE_32F,
                        CUBLAS_GEMM_DEFAULT);
    }
    cudaStreamSynchronize(stream);
    cudaMemcpy(c.data(), dc, c.size() * 4, cudaMemcpyDeviceToHost);
    for (int bi = 0; bi < batch; ++bi)
      for (int j = 0; j < n; j += 7)       // sampled columns keep the host check short
        for (int i = 0; i < m; ++i) {
          double s = 0;
          for (int l = 0; l < k; ++l)
            s += (double)a[(size_t)bi * m * k + i + (size_t)l * m] *
                 (double)b[(size_t)bi * k * n + l + (size_t)j * k];
          const double d = s - (double)c[(size_t)bi * m * n + i + (size_t)j * m];
          base += s * s;
          diff += d * d;
        }
  }
  printf("STATUS %d\n", (int)st);
  printf("RESIDUAL %.6e\n", std::sqrt(diff / base));
  cublasDestroy(h);
  return 0;
}
