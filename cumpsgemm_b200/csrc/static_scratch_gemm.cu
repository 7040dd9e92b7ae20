// cuMpSGEMM_sgemm_static_scratch: the FP32 TCEC GEMM for callers that must not allocate.
//
// Some users of this library run where device allocation is off the table: a service that
// hands its whole memory budget to its own pool at start-up and forbids later cudaMalloc
// calls, a latency-critical loop that cannot afford the implicit device synchronisation of
// cudaMalloc/cudaFree, or a process that does not even own a cuMpSGEMM handle (creating one
// allocates the statistics rings).  The regular entry points keep the split hi/lo operand
// panels in a workspace they grow with cudaMalloc.  This one keeps the panels in a fixed
// array that is part of the library image instead, so a call consists of kernel launches
// only: no handle, no cudaMalloc, no cudaFree, no allocating library routine.
//
// Limits and rules for the caller:
//   * The array is kStaticScratchBytes (32 MiB) per GPU, resident from library load to
//     process exit on every GPU that loads the library.  The panels of a call need
//     2 * (round_up(m, tile_m) + round_up(n, tile_n)) * round_up(k,64) * elem bytes
//     (elem = 2 for FP16TCEC, 4 for TF32TCEC; tile_m x tile_n is the tile the library's one
//     tile rule picks for the shape: 256 x 256 when the CTA-pair kernel runs, else 128 x
//     256 / 128 / 64; the environment overrides CUMPSGEMM_TILE_N and CUMPSGEMM_PAIR apply
//     here as everywhere).  The bound that holds for every tile choice is
//     2 * (round_up(m,256) + round_up(n,256)) * round_up(k,64) * elem <= 32 MiB; e.g.
//     FP16TCEC m=n=k=2048 fits exactly.  Larger problems are rejected with
//     CUBLAS_STATUS_INVALID_VALUE and an error line; nothing is launched.
//   * The first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress) and sets the kernels' shared-memory attribute.  Make that first
//     call before starting any stream capture on that device.
//   * All calls on one GPU share the one array.  Every call rewrites the whole region it
//     uses, padding included, so nothing stale is ever read and nothing needs clearing; but
//     two calls that overlap in time on the same GPU (different streams, different threads)
//     race on it.  Serialise them on one stream.
#include "gemm_common.cuh"

#include <cumpsgemm/cumpsgemm_ext.h>
#include <mutex>

namespace {

constexpr std::size_t kStaticScratchBytes = 32ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
  bool ready = false;
  void *scratch = nullptr; // device address of g_static_scratch on this device
  int num_sms = 0;
};
PerDevice g_per_device[kMaxDevices];
std::mutex g_setup_mutex;

inline std::uint64_t round_up(std::uint64_t x, std::uint64_t a) { return (x + a - 1) / a * a; }

// Once per device, with that device current: the name g_static_scratch is only a host-side
// stand-in for the symbol, so ask the runtime for the address kernels can use.
cudaError_t setup_device(int dev, PerDevice **out) {
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  PerDevice &pd = g_per_device[dev];
  if (!pd.ready) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    pd.scratch = ptr;
    pd.num_sms = sms;
    pd.ready = true;
  }
  *out = &pd;
  return cudaSuccess;
}

} // namespace

using namespace cumpsgemm_b200;

extern "C" cublasStatus_t cuMpSGEMM_sgemm_static_scratch(
    cudaStream_t stream, cublasOperation_t op_A, cublasOperation_t op_B, uint64_t m, uint64_t n,
    uint64_t k, const float *alpha, const float *a, uint64_t lda, const float *b, uint64_t ldb,
    const float *beta, float *c, uint64_t ldc, cuMpSGEMM_compute_mode_t compute_mode) {
  if (compute_mode != CUMPSGEMM_FP16TCEC && compute_mode != CUMPSGEMM_TF32TCEC) {
    log_error("cuMpSGEMM_sgemm_static_scratch computes FP16TCEC and TF32TCEC only");
    return CUBLAS_STATUS_NOT_SUPPORTED;
  }
  if (op_A == CUBLAS_OP_C || op_B == CUBLAS_OP_C) return CUBLAS_STATUS_INVALID_VALUE;
  if (m == 0 || n == 0 || k == 0 || alpha == nullptr || beta == nullptr || a == nullptr ||
      b == nullptr || c == nullptr)
    return CUBLAS_STATUS_INVALID_VALUE;
  const bool a_n = (op_A == CUBLAS_OP_N), b_n = (op_B == CUBLAS_OP_N);
  if (lda < (a_n ? m : k) || ldb < (b_n ? k : n) || ldc < m) return CUBLAS_STATUS_INVALID_VALUE;
  if (m > 0x3fffffffull || n > 0x3fffffffull || k > 0x3fffffffull)
    return CUBLAS_STATUS_INVALID_VALUE;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CUBLAS_STATUS_NOT_INITIALIZED;
  PerDevice *pd = nullptr;
  const cudaError_t se = setup_device(dev, &pd);
  if (se != cudaSuccess) {
    log_error(std::string("cuMpSGEMM_sgemm_static_scratch: device set-up failed: ") +
              cudaGetErrorString(se));
    return CUBLAS_STATUS_NOT_INITIALIZED;
  }

  const SplitKind kind = (compute_mode == CUMPSGEMM_FP16TCEC) ? SplitKind::fp16 : SplitKind::tf32;
  const std::size_t es = (kind == SplitKind::fp16) ? 2 : 4;
  // the tile rule of the regular entry points, so that both run the same kernels
  const Tuning tuning = read_tuning_env(); // no handle to cache them in
  const TileChoice choice = pick_tile(tuning, static_cast<unsigned>(pd->num_sms), m, n, 1, true);
  const int tile_n = choice.tile_n;
  const bool use_pair = choice.pair;
  const std::uint64_t rows_pad_a = round_up(m, use_pair ? 256 : 128);
  const std::uint64_t rows_pad_b = round_up(n, tile_n);
  const std::uint64_t k_pad = round_up(k, 64);
  // Each factor is below 2^31, so the row sum times k_pad stays below 2^63 / 8 only after this
  // first test; the byte counts are formed afterwards and cannot wrap.
  const std::uint64_t max_elems = kStaticScratchBytes / (2 * es);
  const bool fits = (rows_pad_a + rows_pad_b) <= max_elems && k_pad <= max_elems &&
                    (rows_pad_a + rows_pad_b) * k_pad <= max_elems;
  const std::uint64_t bytes_a = fits ? 2 * rows_pad_a * k_pad * es : 0;
  const std::uint64_t bytes_b = fits ? 2 * rows_pad_b * k_pad * es : 0;
  if (!fits) {
    log_error("cuMpSGEMM_sgemm_static_scratch: m=" + std::to_string(m) + " n=" +
              std::to_string(n) + " k=" + std::to_string(k) + " needs 2 * (" +
              std::to_string(rows_pad_a) + " + " + std::to_string(rows_pad_b) + ") * " +
              std::to_string(k_pad) + " * " + std::to_string(es) +
              " bytes of operand panels; the built-in scratch array holds " +
              std::to_string(kStaticScratchBytes) + " bytes. Use cuMpSGEMM_sgemm for this size.");
    return CUBLAS_STATUS_INVALID_VALUE;
  }
  unsigned char *panel_a = static_cast<unsigned char *>(pd->scratch);
  unsigned char *panel_b = panel_a + bytes_a; // bytes_a is a multiple of 16 KiB

  SplitArgs sa;
  sa.kind = kind;
  sa.operand = Operand::A;
  sa.is_complex = false;
  sa.conjugate = false;
  sa.src_k_contig = !a_n;
  sa.rows = m;
  sa.k = k;
  sa.src = a;
  sa.ld = lda;
  sa.stride = 0;
  sa.batch = 1;
  sa.panel = panel_a;
  sa.rows_pad = static_cast<std::uint32_t>(rows_pad_a);
  sa.k_pad = static_cast<std::uint32_t>(k_pad);
  sa.with_lo = true;
  sa.dyn = nullptr;
  cudaError_t err;
  {
    SplitArgs sb = sa;
    sb.operand = Operand::B;
    sb.src_k_contig = b_n;
    sb.rows = n;
    sb.src = b;
    sb.ld = ldb;
    sb.panel = panel_b;
    sb.rows_pad = static_cast<std::uint32_t>(rows_pad_b);
    err = launch_split_pair(sa, sb, stream);
  }
  if (err == cudaSuccess) {
    TcecGemmArgs g;
    g.kind = kind;
    g.error_correction = true;
    g.m = static_cast<std::uint32_t>(m);
    g.n = static_cast<std::uint32_t>(n);
    g.k_pad = static_cast<std::uint32_t>(k_pad);
    g.rows_pad_a = static_cast<std::uint32_t>(rows_pad_a);
    g.rows_pad_b = static_cast<std::uint32_t>(rows_pad_b);
    g.batch = 1;
    g.panel_a = panel_a;
    g.panel_b = panel_b;
    g.c = c;
    g.ldc = ldc;
    g.stride_c = 0;
    g.alpha_r = *alpha;
    g.alpha_i = 0.f;
    g.beta_r = *beta;
    g.beta_i = 0.f;
    g.is_complex = false;
    g.dyn = nullptr;
    g.tile_n = tile_n;
    g.dev_status = nullptr; // no handle, hence no status word; waits stay bounded
    g.tuning = tuning;
    err = use_pair ? launch_tcec_gemm_pair(g, stream) : launch_tcec_gemm(g, stream);
  }
  if (err != cudaSuccess) {
    log_error(std::string("cuMpSGEMM_sgemm_static_scratch: launch failed: ") +
              cudaGetErrorString(err));
    return CUBLAS_STATUS_EXECUTION_FAILED;
  }
  return CUBLAS_STATUS_SUCCESS;
}
