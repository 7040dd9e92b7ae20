// Host dispatch of the TCEC GEMM and the C ABI around it.
//
// Reference counterparts: cumpsgemm::gemm<T> (src/cumpsgemm.cu:228-419),
// cumpsgemm::gemm_stridedBatch<T> (:421-547), the extern "C" wrappers
// (:549-605) and the AUTO / FP16TCEC_SCALING orchestration of the
// interception layer (src/cumpsgemm_cublas.cu:445-577, :829-961).
//
// One call = split op(A) -> split op(B) -> tcgen05 GEMM, all on the handle's
// stream.  The reference's module table (364 instantiations per arch,
// src/instance_sm80.cu) collapses to three tile widths because op N/T/C,
// leading dimensions and edges are absorbed by the split pass.
#include "gemm_common.cuh"

#include <algorithm>
#include <type_traits>

namespace cumpsgemm_b200 {
namespace {

constexpr std::size_t kDefaultWorkspaceLimit = 8ull << 30;

inline std::uint64_t round_up(std::uint64_t x, std::uint64_t a) { return (x + a - 1) / a * a; }

bool ensure_workspace(cuMpSGEMM_handle *h, std::size_t bytes) {
  if (h->workspace_bytes >= bytes) return true;
  // cudaFree waits for work that may still read the old buffer.
  if (h->workspace != nullptr) cudaFree(h->workspace);
  h->workspace = nullptr;
  h->workspace_bytes = 0;
  if (cudaMalloc(&h->workspace, bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  h->workspace_bytes = bytes;
  return true;
}

__global__ void dyn_params_from_flag_kernel(DynParams *out, const int *flag) {
  out->scale_a = 1.f;
  out->scale_b = 1.f;
  out->unscale_c = 1.f;
  const int mode = flag_gemm_mode(*flag);
  out->gemm_mode = (mode == CUMPSGEMM_TF32TCEC) ? CUMPSGEMM_TF32TCEC : CUMPSGEMM_FP16TCEC;
}

template <class T> struct Scalar;
template <> struct Scalar<float> {
  static float re(const float *p) { return *p; }
  static float im(const float *) { return 0.f; }
};
template <> struct Scalar<cuComplex> {
  static float re(const cuComplex *p) { return p->x; }
  static float im(const cuComplex *p) { return p->y; }
};

// Tile for a problem: width 256 / 128 / 64 of the single-CTA kernel (128 rows), or the CTA-pair
// kernel's 256 x 256 tile (error-corrected modes only).  CUMPSGEMM_TILE_N forces the width,
// CUMPSGEMM_PAIR=0/1 the kernel.  Measured on B200 (GEMM kernel only, us, FP16TCEC, beta=0.5,
// 30 calls back to back):
//   m=n=k   128x64   128x128   128x256   pairs 256x256
//   1024     22.0     24.4      32.4       37.0      (16 pair tiles)
//   1536     50.4     31.3      40.8       46.7      (36)
//   2048    121       76.3      56.7       65.9      (64 pair tiles on 74 pair slots)
//   3072      -      198       155        154        (144)
//   4096      -      449       384        362        (256)
// The pair kernel wins once there is more than one wave of pair tiles; below that the widest
// single-CTA tile that still gives about two thirds of the SMs a tile is fastest: narrower
// tiles move the same operand bytes for fewer MMAs.
} // namespace

TileChoice pick_tile(const Tuning &tuning, unsigned num_sms, std::uint64_t m_exp, std::uint64_t n,
                     std::uint64_t batch, bool ec) {
  const bool pair_off = tuning.pair == 0;
  const bool pair_on = tuning.pair == 1;
  if (tuning.tile_n == 256) return {256, ec && !pair_off};
  if (tuning.tile_n == 128 || tuning.tile_n == 64) return {tuning.tile_n, false};
  const std::uint64_t sms = static_cast<std::uint64_t>(num_sms);
  const std::uint64_t pair_tiles = ((m_exp + 255) / 256) * ((n + 255) / 256) * batch;
  const std::uint64_t tiles_256 = ((m_exp + 127) / 128) * ((n + 255) / 256) * batch;
  const std::uint64_t tiles_128 = ((m_exp + 127) / 128) * ((n + 127) / 128) * batch;
  if (ec && !pair_off && (pair_on || pair_tiles > sms / 2)) return {256, true};
  if (3 * tiles_256 >= 2 * sms) return {256, false};
  if (3 * tiles_128 >= 2 * sms) return {128, false};
  return {64, false};
}

namespace {

// The kernel that splits operands on the fly handles FP16TCEC (with or without fused scaling)
// on 16-byte aligned strided operands in the layouts its converters know; see
// tcec_gemm_fused.cu.  Returns false when the call has to take the pre-split path.
template <class T>
bool fused_args(const cuMpSGEMM_handle *h, cublasOperation_t op_A, cublasOperation_t op_B,
                std::uint64_t m, std::uint64_t n, std::uint64_t k, const T *a, std::uint64_t lda,
                std::uint64_t stridea, const T *b, std::uint64_t ldb, std::uint64_t strideb,
                std::uint64_t batch, FusedGemmArgs *out) {
  constexpr bool is_complex = std::is_same<T, cuComplex>::value;
  constexpr std::uint64_t fpe = is_complex ? 2 : 1;
  if (h->tuning.fused == 0) return false;
  if (batch > 0x7fffffffull) return false;
  if (is_complex && (op_A != CUBLAS_OP_N || op_B != CUBLAS_OP_N)) return false;
  const std::uint64_t lda_f = lda * fpe, ldb_f = ldb * fpe;
  const std::uint64_t sa_f = (batch > 1 ? stridea : 0) * fpe, sb_f = (batch > 1 ? strideb : 0) * fpe;
  const bool aligned = (reinterpret_cast<std::uintptr_t>(a) % 16 == 0) &&
                       (reinterpret_cast<std::uintptr_t>(b) % 16 == 0) && lda_f % 4 == 0 &&
                       ldb_f % 4 == 0 && sa_f % 4 == 0 && sb_f % 4 == 0;
  if (!aligned) return false;
  const std::uint64_t m_exp = m * fpe, k_exp = k * fpe;
  if (h->tuning.fused != 1) {
    // Measured crossover (B200, FP16TCEC, one call, ms; pre-split path / this kernel):
    //   512 x complex 256^3      0.51 / 0.43      2048 x real 128^3        0.38 / 0.09
    //   512 x real 256^3         0.20 / 0.15      64 x real 1024^3         0.53 / 0.87
    //   real 4096 x 4096 x 512   0.086 / 0.113    real 8192 x 8192 x 256   0.17 / 0.24
    //   real 1024^3              0.025 / 0.036    real 4096^3              0.37 / 0.81
    // The on-the-fly split wins for strided batches of small matrices, where the split pass,
    // its workspace traffic and a second launch weigh as much as the products; a single
    // matrix, large tiles counts or a long K loop are better off pre-split (every operand
    // element is converted once per tile that uses it).
    // A handful of tiles and a very long K loop: this kernel with its K loop cut over the SMs
    // (split-K below) against the pre-split split-K path, ms per call, NN:
    //   256 x 256 x 65536   0.068 / 0.085     128 x 128 x 131072   0.054 / 0.080
    //   384 x 384 x 32768   0.070 / 0.079     256 x 256 x 8192     0.021 / 0.025
    //   512 x 512 x 16384   0.064 / 0.056 (sixteen tiles: the pre-split path wins again)
    // There the split pass alone moves twice the operand bytes the products need.
    const std::uint64_t tiles = ((m_exp + 127) / 128) * ((n + 127) / 128) * batch;
    const bool few_long = h->tuning.split_k != 0 && h->tuning.pair != 1 &&
                          h->tuning.tile_n != 256 && tiles <= 9 && k_exp >= 8192;
    if (!few_long && (batch < 8 || m_exp > 512 || n > 512 || k_exp > 1024)) return false;
  }
  out->a = reinterpret_cast<const float *>(a);
  out->b = reinterpret_cast<const float *>(b);
  out->lda = lda_f;
  out->ldb = ldb_f;
  out->stride_a = sa_f;
  out->stride_b = sb_f;
  if (is_complex) {
    out->layout_a = 2;
    out->layout_b = 0;
  } else {
    out->layout_a = (op_A == CUBLAS_OP_N) ? 1 : 0;
    out->layout_b = (op_B == CUBLAS_OP_N) ? 0 : 1;
  }
  out->m = static_cast<std::uint32_t>(m_exp);
  out->n = static_cast<std::uint32_t>(n);
  out->k = static_cast<std::uint32_t>(k_exp);
  out->batch = static_cast<std::uint32_t>(batch);
  out->is_complex = is_complex;
  out->tile_n = (h->tuning.tile_n == 64 || n <= 64) ? 64 : 128;
  out->tuning = h->tuning;
  // split-K when the tiles leave at least half of the SMs idle and K is long: as many slices
  // as fill the GPU, each at least four stages (256 k values) long
  out->k_slices = 1;
  out->partial = nullptr;
  {
    const std::uint64_t tiles =
        ((m_exp + 127) / 128) * ((n + out->tile_n - 1) / out->tile_n) * batch;
    const std::uint64_t stages = (k_exp + 63) / 64;
    if (h->tuning.split_k != 0 && 2 * tiles <= h->num_sms && stages >= 8) {
      std::uint64_t want = h->num_sms / tiles;
      if (h->tuning.split_k > 1) want = static_cast<std::uint64_t>(h->tuning.split_k);
      want = std::min<std::uint64_t>(want, stages / 4);
      if (want > 1) {
        const std::uint64_t per = (stages + want - 1) / want;
        out->k_slices = static_cast<std::uint32_t>((stages + per - 1) / per);
      }
    }
  }
  return true;
}

} // namespace

template <class T>
cublasStatus_t gemm_dispatch(cuMpSGEMM_handle *h, cublasOperation_t op_A, cublasOperation_t op_B,
                             std::uint64_t m, std::uint64_t n, std::uint64_t k, const T *alpha,
                             const T *a, std::uint64_t lda, std::uint64_t stridea, const T *b,
                             std::uint64_t ldb, std::uint64_t strideb, const T *beta, T *c,
                             std::uint64_t ldc, std::uint64_t stridec, std::uint64_t batch,
                             cuMpSGEMM_compute_mode_t mode, const DynParams *dyn,
                             unsigned *used_kernel_module_id, const T *const *a_array,
                             const T *const *b_array, T *const *c_array) {
  constexpr bool is_complex = std::is_same<T, cuComplex>::value;
  if (h == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  if (mode == CUMPSGEMM_DRY_RUN) return CUBLAS_STATUS_SUCCESS;
  const bool ptr_arrays = (a_array != nullptr) || (b_array != nullptr) || (c_array != nullptr);
  if (ptr_arrays && (a_array == nullptr || b_array == nullptr || c_array == nullptr))
    return CUBLAS_STATUS_INVALID_VALUE;
  if (m == 0 || n == 0 || k == 0 || batch == 0 || alpha == nullptr || beta == nullptr ||
      (!ptr_arrays && (a == nullptr || b == nullptr || c == nullptr)))
    return CUBLAS_STATUS_INVALID_VALUE;
  const bool a_n = (op_A == CUBLAS_OP_N), b_n = (op_B == CUBLAS_OP_N);
  if (lda < (a_n ? m : k) || ldb < (b_n ? k : n) || ldc < m) return CUBLAS_STATUS_INVALID_VALUE;
  if (m > 0x3fffffffull || n > 0x7fffffffull || k > 0x3fffffffull || batch > 0x3fffffffull)
    return CUBLAS_STATUS_INVALID_VALUE;

  bool want_fp16 = false, want_tf32 = false, ec = true;
  switch (mode) {
  case CUMPSGEMM_FP16TCEC:
    want_fp16 = true;
    break;
  case CUMPSGEMM_TF32TCEC:
    want_tf32 = true;
    break;
  case CUMPSGEMM_FP16TC:
    want_fp16 = true;
    ec = false;
    break;
  case CUMPSGEMM_TF32TC:
    want_tf32 = true;
    ec = false;
    break;
  case CUMPSGEMM_AUTO:
    want_fp16 = want_tf32 = true; // both launched, gated on the device-side decision
    break;
  default:
    log_error(std::string("compute mode ") + cuMpSGEMM_get_compute_mode_string(mode) +
              " is not computed by cuMpSGEMM kernels");
    return CUBLAS_STATUS_NOT_SUPPORTED;
  }

  DeviceGuard guard(h->device);
  if (mode == CUMPSGEMM_AUTO && dyn == nullptr) {
    // Direct API use: the caller enabled a flag slot (or none: slot 0 = TF32TCEC).
    DynParams *slot = h->dev_dyn_params + h->dyn_params_next;
    h->dyn_params_next = (h->dyn_params_next + 1) % h->dyn_params_length;
    const unsigned id = h->dyn_launch.enabled ? h->dyn_launch.enabled_id : 0u;
    dyn_params_from_flag_kernel<<<1, 1, 0, h->cuda_stream>>>(slot, h->dyn_launch.flag_buffer + id);
    dyn = slot;
  }

  const std::uint64_t fpe = is_complex ? 2 : 1;
  const std::uint64_t m_exp = m * fpe; // rows of the expanded real problem
  const std::uint64_t k_exp = k * fpe;

  // ---- one launch, no workspace: operands split inside the GEMM kernel
  FusedGemmArgs fa;
  if (mode == CUMPSGEMM_FP16TCEC && !ptr_arrays &&
      fused_args<T>(h, op_A, op_B, m, n, k, a, lda, stridea, b, ldb, strideb, batch, &fa)) {
    fa.c = reinterpret_cast<float *>(c);
    fa.ldc = ldc * fpe;
    fa.stride_c = stridec * fpe;
    fa.alpha_r = Scalar<T>::re(alpha);
    fa.alpha_i = Scalar<T>::im(alpha);
    fa.beta_r = Scalar<T>::re(beta);
    fa.beta_i = Scalar<T>::im(beta);
    fa.dyn = dyn;
    fa.dev_status = h->dev_status;
    if (fa.k_slices > 1) {
      const std::size_t bytes = static_cast<std::size_t>(fa.k_slices) * fa.m * fa.n * fa.batch *
                                sizeof(float);
      const std::size_t limit =
          h->workspace_limit_bytes ? h->workspace_limit_bytes : kDefaultWorkspaceLimit;
      if (bytes > limit || !ensure_workspace(h, bytes)) fa.k_slices = 1; // no room: no split
      else fa.partial = reinterpret_cast<float *>(h->workspace);
    }
    if (used_kernel_module_id != nullptr)
      *used_kernel_module_id = (fa.k_slices > 1) ? 100u : (fa.tile_n == 128) ? 1u : 2u;
    const bool prof = h->exp_stats.profiling_enabled;
    if (prof) h->exp_stats.profiler.start("gemm_kernel", h->cuda_stream);
    cuMpSGEMM_handle::TimingTriple tt{};
    if (h->kernel_timing) {
      for (auto &e : tt.e) cudaEventCreate(&e);
      cudaEventRecord(tt.e[0], h->cuda_stream);
      cudaEventRecord(tt.e[1], h->cuda_stream);
    }
    cudaError_t ferr = launch_tcec_gemm_fused(fa, h->cuda_stream);
    if (ferr == cudaSuccess && fa.k_slices > 1) {
      TcecGemmArgs r = {};
      r.m = fa.m;
      r.n = fa.n;
      r.batch = fa.batch;
      r.c = fa.c;
      r.ldc = fa.ldc;
      r.stride_c = fa.stride_c;
      r.alpha_r = fa.alpha_r;
      r.alpha_i = fa.alpha_i;
      r.beta_r = fa.beta_r;
      r.beta_i = fa.beta_i;
      r.is_complex = fa.is_complex;
      r.dyn = fa.dyn;
      r.k_slices = fa.k_slices;
      r.partial = fa.partial;
      ferr = launch_splitk_reduce(r, h->cuda_stream);
    }
    if (h->kernel_timing) {
      cudaEventRecord(tt.e[2], h->cuda_stream);
      h->timing_events.push_back(tt);
    }
    if (prof) h->exp_stats.profiler.stop("gemm_kernel", h->cuda_stream);
    mark_stream_work(h);
    if (ferr != cudaSuccess) {
      log_error(std::string("kernel launch failed: ") + cudaGetErrorString(ferr));
      return CUBLAS_STATUS_EXECUTION_FAILED;
    }
    return CUBLAS_STATUS_SUCCESS;
  }

  TileChoice choice = pick_tile(h->tuning, h->num_sms, m_exp, n, batch, ec);
  // Few tiles and a long K loop (the shapes the reference hands to its atomic split-K kernel,
  // src/cumpsgemm.cu:272-304): cut K into slices, one CTA each, so that the tiles fill the
  // GPU; the slices' partial sums are added in a fixed order by a second kernel.  The widest
  // tile the problem fills is taken (fewest operand bytes per product), and each slice keeps
  // at least 256 k values.
  std::uint32_t k_slices = 1;
  {
    const std::uint32_t k_pad64 = static_cast<std::uint32_t>(round_up(k_exp, 64));
    int wide = (n > 128) ? 256 : (n > 64 ? 128 : 64);
    if (h->tuning.tile_n != 0) wide = h->tuning.tile_n;
    const std::uint64_t tiles = ((m_exp + 127) / 128) * ((n + wide - 1) / wide) * batch;
    const bool forced = h->tuning.split_k > 1;
    if (!ptr_arrays && h->tuning.split_k != 0 && h->tuning.pair != 1 &&
        (forced || (k_pad64 >= 2048 && 2 * tiles <= h->num_sms))) {
      std::uint32_t wanted = static_cast<std::uint32_t>(h->num_sms / tiles);
      wanted = std::min<std::uint32_t>(wanted, k_pad64 / 256);
      if (forced) wanted = static_cast<std::uint32_t>(h->tuning.split_k);
      k_slices = split_k_slices(k_pad64, wanted);
      if (k_slices > 1) choice = TileChoice{wide, false};
    }
  }
  const int tile_n = choice.tile_n;
  const bool use_pair = choice.pair;
  // tile class, or 100 for the split-K path as in the reference (src/cumpsgemm.cu:283-285)
  if (used_kernel_module_id != nullptr)
    *used_kernel_module_id =
        (k_slices > 1) ? 100u : (tile_n == 256) ? 0u : (tile_n == 128 ? 1u : 2u);

  const std::uint32_t rows_pad_a =
      static_cast<std::uint32_t>(round_up(m_exp, use_pair ? 256 : 128));
  const std::uint32_t rows_pad_b = static_cast<std::uint32_t>(round_up(n, tile_n));
  const std::uint32_t k_pad = static_cast<std::uint32_t>(round_up(k_exp, 64));
  const std::size_t es_max = want_tf32 ? 4 : 2;
  const std::size_t planes = ec ? 2 : 1;
  const std::size_t bytes_a_1 = planes * rows_pad_a * static_cast<std::size_t>(k_pad) * es_max;
  const std::size_t bytes_b_1 = planes * rows_pad_b * static_cast<std::size_t>(k_pad) * es_max;
  const std::size_t limit =
      h->workspace_limit_bytes ? h->workspace_limit_bytes : kDefaultWorkspaceLimit;
  // split-K partial sums: k_slices blocks of m x n floats per batch entry, behind the panels
  const std::size_t bytes_p_1 =
      (k_slices > 1) ? static_cast<std::size_t>(k_slices) * m_exp * n * sizeof(float) : 0;
  // scratch of the pair kernel's tail split (once per call, behind everything else)
  const std::size_t bytes_tail = use_pair ? pair_tail_scratch_bytes(h->num_sms) : 0;
  std::uint64_t chunk = std::max<std::uint64_t>(1, limit / (bytes_a_1 + bytes_b_1 + bytes_p_1));
  chunk = std::min<std::uint64_t>(chunk, batch);
  chunk = std::min<std::uint64_t>(chunk, 32768); // planes of a tensor map, tiles of a launch
  if (!ensure_workspace(h, chunk * (bytes_a_1 + bytes_b_1 + bytes_p_1) + bytes_tail)) {
    log_error("failed to allocate the operand workspace");
    return CUBLAS_STATUS_ALLOC_FAILED;
  }
  char *ws_a = reinterpret_cast<char *>(h->workspace);
  char *ws_b = ws_a + chunk * bytes_a_1;
  float *ws_p = reinterpret_cast<float *>(ws_b + chunk * bytes_b_1);
  float *ws_t = reinterpret_cast<float *>(reinterpret_cast<char *>(ws_p) + chunk * bytes_p_1);

  const bool prof = h->exp_stats.profiling_enabled;
  if (prof) h->exp_stats.profiler.start("gemm_kernel", h->cuda_stream);
  cudaError_t err = cudaSuccess;
  for (std::uint64_t b0 = 0; b0 < batch && err == cudaSuccess; b0 += chunk) {
    const std::uint32_t nb = static_cast<std::uint32_t>(std::min<std::uint64_t>(chunk, batch - b0));
    // AUTO: one split launch and one GEMM launch whose kernels read the device-side decision
    // and run the FP16 or the TF32 pipeline; every other mode: the one kind it names.
    const bool auto_kind = want_fp16 && want_tf32;
    const SplitKind kind = want_fp16 ? SplitKind::fp16 : SplitKind::tf32;
    SplitArgs sa;
    sa.kind = kind;
    sa.operand = Operand::A;
    sa.is_complex = is_complex;
    sa.conjugate = is_complex && op_A == CUBLAS_OP_C;
    sa.src_k_contig = !a_n;
    sa.rows = m;
    sa.k = k;
    sa.src = ptr_arrays ? nullptr : a + b0 * stridea;
    sa.src_array = ptr_arrays ? reinterpret_cast<const void *const *>(a_array + b0) : nullptr;
    sa.ld = lda;
    sa.stride = stridea;
    sa.batch = nb;
    sa.panel = ws_a;
    sa.rows_pad = rows_pad_a;
    sa.k_pad = k_pad;
    sa.with_lo = ec;
    sa.dyn = dyn;
    cuMpSGEMM_handle::TimingTriple tt{};
    if (h->kernel_timing) {
      for (auto &e : tt.e) cudaEventCreate(&e);
      cudaEventRecord(tt.e[0], h->cuda_stream);
    }
    SplitArgs sb = sa;
    sb.operand = Operand::B;
    sb.conjugate = is_complex && op_B == CUBLAS_OP_C;
    sb.src_k_contig = b_n;
    sb.rows = n;
    sb.src = ptr_arrays ? nullptr : b + b0 * strideb;
    sb.src_array = ptr_arrays ? reinterpret_cast<const void *const *>(b_array + b0) : nullptr;
    sb.ld = ldb;
    sb.stride = strideb;
    sb.panel = ws_b;
    sb.rows_pad = rows_pad_b;
    err = auto_kind ? launch_split_pair_auto(sa, sb, h->cuda_stream)
                    : launch_split_pair(sa, sb, h->cuda_stream);
    if (err != cudaSuccess) break;
    if (h->kernel_timing) cudaEventRecord(tt.e[1], h->cuda_stream);

    TcecGemmArgs g;
    g.kind = kind;
    g.error_correction = ec;
    g.m = static_cast<std::uint32_t>(m_exp);
    g.n = static_cast<std::uint32_t>(n);
    g.k_pad = k_pad;
    g.rows_pad_a = rows_pad_a;
    g.rows_pad_b = rows_pad_b;
    g.batch = nb;
    g.panel_a = ws_a;
    g.panel_b = ws_b;
    g.c = ptr_arrays ? nullptr : reinterpret_cast<float *>(c + b0 * stridec);
    g.c_array = ptr_arrays ? reinterpret_cast<float *const *>(c_array + b0) : nullptr;
    g.ldc = ldc * fpe;
    g.stride_c = stridec * fpe;
    g.alpha_r = Scalar<T>::re(alpha);
    g.alpha_i = Scalar<T>::im(alpha);
    g.beta_r = Scalar<T>::re(beta);
    g.beta_i = Scalar<T>::im(beta);
    g.is_complex = is_complex;
    g.dyn = dyn;
    g.tile_n = tile_n;
    g.dev_status = h->dev_status;
    g.wave_counter = reinterpret_cast<unsigned int *>(h->dev_status + 1);
    g.debug = h->debug_buffer;
    g.tuning = h->tuning;
    g.k_slices = k_slices;
    g.partial = (k_slices > 1) ? ws_p : nullptr;
    g.tail_partial = use_pair ? ws_t : nullptr;
    if (auto_kind)
      err = use_pair ? launch_tcec_gemm_pair_auto(g, h->cuda_stream)
                     : launch_tcec_gemm_auto(g, h->cuda_stream);
    else
      err = use_pair ? launch_tcec_gemm_pair(g, h->cuda_stream)
                     : launch_tcec_gemm(g, h->cuda_stream);
    if (err == cudaSuccess && k_slices > 1) err = launch_splitk_reduce(g, h->cuda_stream);
    if (h->kernel_timing) {
      cudaEventRecord(tt.e[2], h->cuda_stream);
      h->timing_events.push_back(tt);
    }
  }
  if (prof) h->exp_stats.profiler.stop("gemm_kernel", h->cuda_stream);
  mark_stream_work(h);
  if (err != cudaSuccess) {
    log_error(std::string("kernel launch failed: ") + cudaGetErrorString(err));
    return CUBLAS_STATUS_EXECUTION_FAILED;
  }
  return CUBLAS_STATUS_SUCCESS;
}

template <class T>
cublasStatus_t gemm_with_statistics(cuMpSGEMM_handle *h, cublasOperation_t op_A,
                                    cublasOperation_t op_B, std::uint64_t m, std::uint64_t n,
                                    std::uint64_t k, const T *alpha, const T *a, std::uint64_t lda,
                                    std::uint64_t stridea, const T *b, std::uint64_t ldb,
                                    std::uint64_t strideb, const T *beta, T *c, std::uint64_t ldc,
                                    std::uint64_t stridec, std::uint64_t batch,
                                    cuMpSGEMM_compute_mode_t mode, unsigned *stats_id_a_out,
                                    unsigned *stats_id_b_out, unsigned *flag_id_out) {
  if (h == nullptr) return CUBLAS_STATUS_NOT_INITIALIZED;
  if (mode != CUMPSGEMM_AUTO && mode != CUMPSGEMM_FP16TCEC_SCALING)
    return CUBLAS_STATUS_INVALID_VALUE;
  if (m == 0 || n == 0 || k == 0 || batch == 0 || a == nullptr || b == nullptr)
    return CUBLAS_STATUS_INVALID_VALUE;
  if (m > 0xffffffffull || n > 0xffffffffull || k > 0xffffffffull || lda > 0xffffffffull ||
      ldb > 0xffffffffull || stridea > 0xffffffffull || strideb > 0xffffffffull ||
      batch > 0xffffffffull)
    return CUBLAS_STATUS_INVALID_VALUE;
  DeviceGuard guard(h->device);
  // stored extents of A and B (before op)
  const unsigned am = static_cast<unsigned>(op_A == CUBLAS_OP_N ? m : k);
  const unsigned an = static_cast<unsigned>(op_A == CUBLAS_OP_N ? k : m);
  const unsigned bm = static_cast<unsigned>(op_B == CUBLAS_OP_N ? k : n);
  const unsigned bn = static_cast<unsigned>(op_B == CUBLAS_OP_N ? n : k);
  // A batch of one is a single matrix whatever the stride says.
  const unsigned sa = batch > 1 ? static_cast<unsigned>(stridea) : 0u;
  const unsigned sb = batch > 1 ? static_cast<unsigned>(strideb) : 0u;
  unsigned id_a, id_b, flag_id;
  cuMpSGEMM_compute_mode_t gemm_mode;
  const DynParams *dyn;
  const bool fused_scans = !h->exp_stats.profiling_enabled;
  if (fused_scans) {
    // both operands share the scan launches; the slot ids are taken in the usual order
    id_a = next_exp_stats_id(h);
    id_b = next_exp_stats_id(h);
    exp_stats_pair<T>(h, mode == CUMPSGEMM_AUTO, id_a, am, an, a, static_cast<unsigned>(lda), sa,
                      id_b, bm, bn, b, static_cast<unsigned>(ldb), sb,
                      static_cast<unsigned>(batch));
  }
  if (mode == CUMPSGEMM_AUTO) {
    if (!fused_scans) {
      id_a = cumpsgemm::exp_stats_ext<T>(h, am, an, a, static_cast<unsigned>(lda),
                                         static_cast<unsigned>(batch), sa);
      id_b = cumpsgemm::exp_stats_ext<T>(h, bm, bn, b, static_cast<unsigned>(ldb),
                                         static_cast<unsigned>(batch), sb);
    }
    flag_id = next_dyn_launch_id(h);
    dyn = prepare_dyn_params_from_stats(h, flag_id, id_a, id_b);
    gemm_mode = CUMPSGEMM_AUTO;
  } else {
    if (!fused_scans) {
      id_a = cumpsgemm::exp_max_ext<T>(h, am, an, a, static_cast<unsigned>(lda),
                                       static_cast<unsigned>(batch), sa);
      id_b = cumpsgemm::exp_max_ext<T>(h, bm, bn, b, static_cast<unsigned>(ldb),
                                       static_cast<unsigned>(batch), sb);
    }
    flag_id = 1; // reserved slot: FP16TCEC with both scale bits
    dyn = prepare_dyn_params(h, flag_id, id_a, id_b);
    gemm_mode = CUMPSGEMM_FP16TCEC;
  }
  if (stats_id_a_out) *stats_id_a_out = id_a;
  if (stats_id_b_out) *stats_id_b_out = id_b;
  if (flag_id_out) *flag_id_out = flag_id;
  return gemm_dispatch<T>(h, op_A, op_B, m, n, k, alpha, a, lda, stridea, b, ldb, strideb, beta, c,
                          ldc, stridec, batch, gemm_mode, dyn, nullptr);
}

#define INSTANTIATE(T)                                                                            \
  template cublasStatus_t gemm_dispatch<T>(                                                       \
      cuMpSGEMM_handle *, cublasOperation_t, cublasOperation_t, std::uint64_t, std::uint64_t,     \
      std::uint64_t, const T *, const T *, std::uint64_t, std::uint64_t, const T *, std::uint64_t, \
      std::uint64_t, const T *, T *, std::uint64_t, std::uint64_t, std::uint64_t,                 \
      cuMpSGEMM_compute_mode_t, const DynParams *, unsigned *, const T *const *,                  \
      const T *const *, T *const *);                                                              \
  template cublasStatus_t gemm_with_statistics<T>(                                                \
      cuMpSGEMM_handle *, cublasOperation_t, cublasOperation_t, std::uint64_t, std::uint64_t,     \
      std::uint64_t, const T *, const T *, std::uint64_t, std::uint64_t, const T *, std::uint64_t, \
      std::uint64_t, const T *, T *, std::uint64_t, std::uint64_t, std::uint64_t,                 \
      cuMpSGEMM_compute_mode_t, unsigned *, unsigned *, unsigned *);
INSTANTIATE(float)
INSTANTIATE(cuComplex)
#undef INSTANTIATE

} // namespace cumpsgemm_b200

// ---------------------------------------------------------------- public C++ API
namespace cumpsgemm {
using namespace cumpsgemm_b200;

template <class T>
cublasStatus_t gemm(cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
                    const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
                    const uint64_t k, const T *alpha, const T *const a_dmem_ptr,
                    const uint64_t lda, const T *const b_dmem_ptr, const uint64_t ldb,
                    const T *beta, T *const c_dmem_ptr, const uint64_t ldc,
                    const cuMpSGEMM_compute_mode_t compute_mode,
                    unsigned *const used_kernel_module_id) {
  if (compute_mode == CUMPSGEMM_FP16TCEC_SCALING) {
    return gemm_with_statistics<T>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda, 0,
                                   b_dmem_ptr, ldb, 0, beta, c_dmem_ptr, ldc, 0, 1, compute_mode,
                                   nullptr, nullptr, nullptr);
  }
  return gemm_dispatch<T>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda, 0, b_dmem_ptr, ldb,
                          0, beta, c_dmem_ptr, ldc, 0, 1, compute_mode, nullptr,
                          used_kernel_module_id);
}

template <class T>
cublasStatus_t gemm_stridedBatch(cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
                                 const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
                                 const uint64_t k, const T *alpha, const T *const a_dmem_ptr,
                                 const uint64_t lda, const uint64_t stridea,
                                 const T *const b_dmem_ptr, const uint64_t ldb,
                                 const uint64_t strideb, const T *beta, T *const c_dmem_ptr,
                                 const uint64_t ldc, const uint64_t stridec,
                                 const uint64_t batch_count,
                                 const cuMpSGEMM_compute_mode_t compute_mode,
                                 unsigned *const used_kernel_module_id) {
  if (compute_mode == CUMPSGEMM_FP16TCEC_SCALING) {
    return gemm_with_statistics<T>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda, stridea,
                                   b_dmem_ptr, ldb, strideb, beta, c_dmem_ptr, ldc, stridec,
                                   batch_count, compute_mode, nullptr, nullptr, nullptr);
  }
  return gemm_dispatch<T>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda, stridea,
                          b_dmem_ptr, ldb, strideb, beta, c_dmem_ptr, ldc, stridec, batch_count,
                          compute_mode, nullptr, used_kernel_module_id);
}

#define INSTANTIATE(T)                                                                           \
  template cublasStatus_t gemm<T>(cuMpSGEMM_handle_t, const cublasOperation_t,                   \
                                  const cublasOperation_t, const uint64_t, const uint64_t,       \
                                  const uint64_t, const T *, const T *const, const uint64_t,     \
                                  const T *const, const uint64_t, const T *, T *const,           \
                                  const uint64_t, const cuMpSGEMM_compute_mode_t,                \
                                  unsigned *const);                                              \
  template cublasStatus_t gemm_stridedBatch<T>(                                                  \
      cuMpSGEMM_handle_t, const cublasOperation_t, const cublasOperation_t, const uint64_t,      \
      const uint64_t, const uint64_t, const T *, const T *const, const uint64_t, const uint64_t, \
      const T *const, const uint64_t, const uint64_t, const T *, T *const, const uint64_t,       \
      const uint64_t, const uint64_t, const cuMpSGEMM_compute_mode_t, unsigned *const);
INSTANTIATE(float)
INSTANTIATE(cuComplex)
#undef INSTANTIATE
} // namespace cumpsgemm

// ---------------------------------------------------------------- C ABI
extern "C" {

cublasStatus_t cuMpSGEMM_sgemm(cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
                               const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
                               const uint64_t k, const float *alpha, const float *const a_dmem_ptr,
                               const uint64_t lda, const float *const b_dmem_ptr,
                               const uint64_t ldb, const float *beta, float *const c_dmem_ptr,
                               const uint64_t ldc, const cuMpSGEMM_compute_mode_t compute_mode) {
  if (op_A == CUBLAS_OP_C || op_B == CUBLAS_OP_C) return CUBLAS_STATUS_INVALID_VALUE;
  return cumpsgemm::gemm<float>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda, b_dmem_ptr,
                                ldb, beta, c_dmem_ptr, ldc, compute_mode);
}

cublasStatus_t cuMpSGEMM_cgemm(cuMpSGEMM_handle_t handle, const cublasOperation_t op_A,
                               const cublasOperation_t op_B, const uint64_t m, const uint64_t n,
                               const uint64_t k, const cuComplex *alpha,
                               const cuComplex *const a_dmem_ptr, const uint64_t lda,
                               const cuComplex *const b_dmem_ptr, const uint64_t ldb,
                               const cuComplex *beta, cuComplex *const c_dmem_ptr,
                               const uint64_t ldc, const cuMpSGEMM_compute_mode_t compute_mode) {
  return cumpsgemm::gemm<cuComplex>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda,
                                    b_dmem_ptr, ldb, beta, c_dmem_ptr, ldc, compute_mode);
}

cublasStatus_t cuMpSGEMM_sgemm_strided_batch(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A, const cublasOperation_t op_B,
    const uint64_t m, const uint64_t n, const uint64_t k, const float *alpha,
    const float *const a_dmem_ptr, const uint64_t lda, const uint64_t stridea,
    const float *const b_dmem_ptr, const uint64_t ldb, const uint64_t strideb, const float *beta,
    float *const c_dmem_ptr, const uint64_t ldc, const uint64_t stridec,
    const uint64_t batch_count, const cuMpSGEMM_compute_mode_t compute_mode) {
  if (op_A == CUBLAS_OP_C || op_B == CUBLAS_OP_C) return CUBLAS_STATUS_INVALID_VALUE;
  return cumpsgemm::gemm_stridedBatch<float>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr, lda,
                                             stridea, b_dmem_ptr, ldb, strideb, beta, c_dmem_ptr,
                                             ldc, stridec, batch_count, compute_mode);
}

cublasStatus_t cuMpSGEMM_cgemm_strided_batch(
    cuMpSGEMM_handle_t handle, const cublasOperation_t op_A, const cublasOperation_t op_B,
    const uint64_t m, const uint64_t n, const uint64_t k, const cuComplex *alpha,
    const cuComplex *const a_dmem_ptr, const uint64_t lda, const uint64_t stridea,
    const cuComplex *const b_dmem_ptr, const uint64_t ldb, const uint64_t strideb,
    const cuComplex *beta, cuComplex *const c_dmem_ptr, const uint64_t ldc,
    const uint64_t stridec, const uint64_t batch_count,
    const cuMpSGEMM_compute_mode_t compute_mode) {
  return cumpsgemm::gemm_stridedBatch<cuComplex>(handle, op_A, op_B, m, n, k, alpha, a_dmem_ptr,
                                                 lda, stridea, b_dmem_ptr, ldb, strideb, beta,
                                                 c_dmem_ptr, ldc, stridec, batch_count,
                                                 compute_mode);
}

} // extern "C"
