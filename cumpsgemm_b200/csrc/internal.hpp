// Internal declarations shared by the translation units of libcumpsgemm.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include <cuComplex.h>
#include <cuda_runtime.h>
#include <cumpsgemm/cumpsgemm.hpp>

namespace cumpsgemm_b200 {

// ---------------------------------------------------------------- logging
// Same grammar and environment switches as the reference's src/utils.hpp:5-42:
// "[cuMpSGEMM LOG] ..." when CUMPSGEMM_INFO is set and not "0";
// "[cuMpSGEMM ERROR] ..." unless CUMPSGEMM_ERROR_LOG=0;
// "[cuMpSGEMM WARNING] ..." only when CUMPSGEMM_ERROR_LOG is set and not "0".
bool env_flag(const char *name, bool default_value);
void log_info(const std::string &s);
void log_error(const std::string &s);
void log_warning(const std::string &s);

// ---------------------------------------------------------------- flag word
// Dynamic-launch flag word: bits [0,5) GEMM mode, bit 5 "scale B", bit 6
// "scale A" (reference: src/dynamic_launch_utils.hpp:7-41).
constexpr int kFlagModeMask = 0x1f;
constexpr int kFlagScaleB = 0x20;
constexpr int kFlagScaleA = 0x40;
__host__ __device__ inline int flag_gemm_mode(int flag) { return flag & kFlagModeMask; }
__host__ __device__ inline bool flag_scale_a(int flag) { return (flag & kFlagScaleA) != 0; }
__host__ __device__ inline bool flag_scale_b(int flag) { return (flag & kFlagScaleB) != 0; }

// Scaling target: operands are scaled so that their largest exponent becomes
// 2^14 (reference: src/dynamic_scaling.cu:15).
constexpr float kHalfExpMax = 16384.0f;

// Per-call constants of the fused AUTO / FP16TCEC_SCALING pipeline, computed
// on the device from a flag word and two statistics slots so that the host
// never synchronises.
struct DynParams {
  float scale_a;   // multiply op(A) by this (exact power of two) before splitting
  float scale_b;   // same for op(B)
  float unscale_c; // multiply the product by this in the GEMM epilogue
  int gemm_mode;   // CUMPSGEMM_FP16TCEC or CUMPSGEMM_TF32TCEC
};

// ---------------------------------------------------------------- profiler
// Named accumulating timers (reference uses cutf's time_breakdown profiler:
// src/exp_stats.cu:309-378).  start/stop synchronise the stream.
struct Profiler {
  struct Entry {
    double sum_s = 0;
    std::uint64_t n = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
  };
  std::unordered_map<std::string, Entry> entries;
  void start(const std::string &name, cudaStream_t s);
  void stop(const std::string &name, cudaStream_t s);
  void clear();
  ~Profiler();
};

// Tuning switches read from the environment.  A handle reads them once, when it is created
// (cuMpSGEMM_reload_tuning_env reads them again); entry points without a handle read them per
// call.  CUMPSGEMM_TILE_N = 256 / 128 / 64 forces the tile width, CUMPSGEMM_PAIR = 0 / 1 the
// CTA-pair kernel off / on, CUMPSGEMM_DRAIN_CHUNK and CUMPSGEMM_FIRST_CHUNK the number of
// K stages per accumulator drain (pair kernel), CUMPSGEMM_PACE = 0 the wave pacing off,
// CUMPSGEMM_FUSED = 0 / 1 the kernel that splits operands on the fly off / on wherever it is
// applicable, CUMPSGEMM_SPLIT_K = 0 / n the K-slicing of problems with few tiles off / to n
// slices.
struct Tuning {
  int tile_n = 0;      // 0 = by rule
  int pair = -1;       // -1 = by rule
  int drain_chunk = 0; // 0 = default
  int first_chunk = 0; // 0 = default
  int pace = 1;
  int fused = -1;      // -1 = by rule
  int split_k = -1;    // CUMPSGEMM_SPLIT_K: 0 = never, -1 = by rule, n > 1 = that many slices
  int tail_split = -1; // CUMPSGEMM_TAIL_SPLIT: 0 = never, -1 = by rule, n > 1 = at most n slices
};
Tuning read_tuning_env();

struct ExpStatsState {
  bool enabled = false;
  unsigned long long *dev_total = nullptr;
  unsigned long long *dev_underflow = nullptr;
  int *dev_mode = nullptr;
  float *dev_max = nullptr;
  float ignore_threshold = 0.f;
  float underflow_threshold = 1.f / 32768.f;
  float underflow_tolerance_rate = 0.f;
  std::uint32_t buffer_length = 10000;
  std::uint32_t current_buffer_id = 1;
  Profiler profiler;
  bool profiling_enabled = false;
  // Compatibility switch: also count the zeros the reference's 4-wide counting loop appends
  // to a matrix whose element count is not a multiple of 4 (src/exp_stats.cu:101-116).
  bool count_tail_padding = false;
  // Scratch of the one-launch-per-stage scans: for each of two operands one 24-byte record per
  // CTA (num_sms * 8 of them), then two ticket counters, which every launch leaves at zero.
  void *dev_scan_scratch = nullptr;
};

struct DynLaunchState {
  unsigned flag_buffer_length = 10000;
  unsigned current_buffer_id = 1;
  int *flag_buffer = nullptr;
  bool enabled = false;
  unsigned enabled_id = 0;
};

} // namespace cumpsgemm_b200

// The public opaque handle (reference: src/handle.hpp:7-29).
struct cuMpSGEMM_handle {
  int device = 0;
  unsigned num_sms = 0;
  cudaStream_t cuda_stream = 0;
  cumpsgemm_b200::ExpStatsState exp_stats;
  cumpsgemm_b200::DynLaunchState dyn_launch;

  // Ring of DynParams records for fused scaling calls.
  cumpsgemm_b200::DynParams *dev_dyn_params = nullptr;
  unsigned dyn_params_length = 1024;
  unsigned dyn_params_next = 0;

  // Operand workspace: hi/lo panels of op(A) and op(B) in the K-major tile
  // format the GEMM kernel reads through TMA.  Grown on demand.
  void *workspace = nullptr;
  std::size_t workspace_bytes = 0;
  std::size_t workspace_limit_bytes = 0; // 0 = derive from free memory

  cumpsgemm_b200::Tuning tuning;

  // Device status word the GEMM kernel writes when a bounded wait gives up.
  int *dev_status = nullptr; // [0] kernel status word, [1] wave counter of the pair kernel

  // Optional per-launch timing: events recorded on the launching stream before the split
  // pass, between split pass and GEMM kernel, and after the GEMM kernel.
  struct TimingTriple {
    cudaEvent_t e[3];
  };
  bool kernel_timing = false;
  unsigned long long *debug_buffer = nullptr; // caller-owned, see cuMpSGEMM_set_debug_buffer

  // The workspace, the DynParams ring, the statistics scratch and the wave counter are shared by
  // all calls on the handle.  Calls on one stream are ordered by the stream; when the handle is
  // moved to another stream (cuMpSGEMM_set_stream; the interception layer does it for every
  // caller's cuBLAS stream) the new stream first waits for `order_event`, which every call that
  // touches the shared buffers records behind its last launch.
  cudaEvent_t order_event = nullptr;
  bool order_event_recorded = false;
  // Held by the interception layer from set_stream to the last launch of a call, so that host
  // threads sharing the per-device handle cannot interleave inside a call.  Users of the handle
  // API use one handle per thread (or their own lock), as with cuBLAS handles.
  std::mutex call_mutex;
  std::vector<TimingTriple> timing_events;
};

namespace cumpsgemm_b200 {

// Record the handle's ordering event behind the work just enqueued (see cuMpSGEMM_handle).
// Skipped while the stream is being captured into a graph: a captured event cannot order
// work outside the capture, and a graph replays as one unit of its launch stream anyway.
inline void mark_stream_work(cuMpSGEMM_handle *h) {
  if (h->order_event == nullptr) return;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(h->cuda_stream, &cap) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  if (cap != cudaStreamCaptureStatusNone) return;
  if (cudaEventRecord(h->order_event, h->cuda_stream) == cudaSuccess)
    h->order_event_recorded = true;
  else
    cudaGetLastError();
}

// RAII: make the handle's device current for the duration of a call.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) {
      cudaSetDevice(dev);
      changed = true;
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

// ---------------------------------------------------------------- operand split
enum class SplitKind : int { fp16 = 0, tf32 = 1 };
enum class Operand : int { A = 0, B = 1 };

struct SplitArgs {
  SplitKind kind;
  Operand operand;
  bool is_complex;
  bool conjugate;      // op == C on complex input
  bool src_k_contig;   // true: source element (r, kk) at [kk + r*ld]; false: [r + kk*ld]
  std::uint64_t rows;  // logical rows of op(X): m for A, n for B (complex: complex elements)
  std::uint64_t k;     // logical K (complex: complex elements)
  const void *src;
  const void *const *src_array = nullptr; // device array of per-batch pointers (or null)
  std::uint64_t ld;     // in elements of the source type
  std::uint64_t stride; // batch stride in elements of the source type
  std::uint32_t batch;
  void *panel;             // destination
  std::uint32_t rows_pad;  // padded expanded rows (multiple of 64)
  std::uint32_t k_pad;     // padded expanded K (multiple of 64)
  bool with_lo;            // also write the lo panel
  const DynParams *dyn;    // nullable: scale factor and gating
};
// Splits op(A) and op(B) of one GEMM in a single launch.
cudaError_t launch_split_pair(const SplitArgs &a, const SplitArgs &b, cudaStream_t stream);
// Same, with the kind taken on the device from dyn->gemm_mode (`kind` of the arguments is
// ignored; dyn must be set and the panels sized for TF32).
cudaError_t launch_split_pair_auto(const SplitArgs &a, const SplitArgs &b, cudaStream_t stream);

// ---------------------------------------------------------------- TCEC GEMM
// Launch behind the previous kernel of the stream with programmatic stream serialization: the
// new grid may be scheduled while that kernel drains (which hides the launch latency of the short
// kernels an AUTO / FP16TCEC_SCALING call chains: statistics -> constants -> split -> GEMM).
// Every kernel launched this way executes griddepcontrol.wait before it reads or writes global
// memory and only then griddepcontrol.launch_dependents, so completion stays transitive along
// the chain and nothing runs ahead of data it depends on.
#ifdef __CUDACC__
template <class Kernel, class... Args>
inline cudaError_t launch_chained(Kernel kernel, unsigned grid, unsigned block, std::size_t smem,
                                  cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
// First statements of a kernel that is launched with launch_chained (harmless otherwise).
#define CUMPSGEMM_CHAINED_KERNEL_ENTRY()                          \
  asm volatile("griddepcontrol.wait;" ::: "memory");             \
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
// First statement of a kernel that heads a chain (ordinary launch).
#define CUMPSGEMM_CHAIN_HEAD_ENTRY() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#endif

struct TcecGemmArgs {
  SplitKind kind;
  bool error_correction;
  std::uint32_t m, n;  // C extent in floats (complex: m counts re/im rows separately)
  std::uint32_t k_pad;
  std::uint32_t rows_pad_a, rows_pad_b;
  std::uint32_t batch;
  const void *panel_a;
  const void *panel_b;
  float *c;
  float *const *c_array = nullptr; // device array of per-batch C pointers (or null)
  std::uint64_t ldc;      // in floats
  std::uint64_t stride_c; // in floats
  float alpha_r, alpha_i, beta_r, beta_i;
  bool is_complex;
  const DynParams *dyn; // nullable
  int tile_n;           // 256, 128 or 64
  int *dev_status;
  unsigned long long *debug = nullptr; // optional stall breakdown buffer (8 x u64)
  // Optional device word the persistent pair kernel uses to keep its clusters in step
  // (zeroed by the launcher before every launch); null switches the pacing off.
  unsigned int *wave_counter = nullptr;
  Tuning tuning;
  // Split-K (single-CTA kernel only): k_slices > 1 cuts the K loop into that many CTAs per tile,
  // which write plain partial sums to `partial` (k_slices * batch * m * n floats); the caller
  // then runs launch_splitk_reduce.  split_k_slices() gives the slice count that makes every
  // slice the same whole number of 64-k-value units (0 or 1: no split).
  std::uint32_t k_slices = 1;
  float *partial = nullptr;
  // Pair kernel only: scratch for the K-split of the last, partly filled wave of tiles
  // (pair_tail_scratch_bytes() bytes) and kPairTailCounters zeroed device words behind
  // `wave_counter`; null switches the tail split off.
  float *tail_partial = nullptr;
};
// Device words the pair kernel's tail split needs behind the wave counter (two per tail tile).
constexpr int kPairTailCounters = 256;
// Bytes of `tail_partial` on a device with num_sms SMs: one 256 x 256 FP32 tile per CTA pair.
inline std::size_t pair_tail_scratch_bytes(int num_sms) {
  return static_cast<std::size_t>(num_sms / 2) * 256u * 256u * sizeof(float);
}
// Slices actually used when `wanted` are asked for a K loop of k_pad values.
std::uint32_t split_k_slices(std::uint32_t k_pad, std::uint32_t wanted);
// C = alpha * unscale * sum_s partial[s] + beta * C with the slices added in ascending order
// (run-to-run bit-identical, unlike the reference's atomic accumulation,
// src/cumpsgemm.cu:272-304 and src/dmem_accessor.hpp:352-395).  Sizes as in TcecGemmArgs.
cudaError_t launch_splitk_reduce(const TcecGemmArgs &a, cudaStream_t stream);
cudaError_t launch_tcec_gemm(const TcecGemmArgs &a, cudaStream_t stream);
// AUTO: one launch that reads dyn->gemm_mode and runs the FP16 or the TF32 pipeline
// (error-corrected kinds only).  `a` describes the problem; its `kind` is ignored.
cudaError_t launch_tcec_gemm_auto(const TcecGemmArgs &a, cudaStream_t stream);
// GEMM that splits its operands on the fly (tcec_gemm_fused.cu): no workspace, FP16 kinds with
// error correction only.  Sizes are those of the real problem (complex operands expanded:
// m = 2 * rows of C, k = 2 * K); leading dimensions and strides are in floats.
struct FusedGemmArgs {
  const float *a, *b;
  std::uint64_t lda, ldb;           // floats between consecutive columns of the stored operand
  std::uint64_t stride_a, stride_b; // floats between batch entries
  int layout_a, layout_b;           // 0 = K contiguous, 1 = row contiguous, 2 = complex A, op N
  std::uint32_t m, n, k;
  std::uint32_t batch;
  float *c;
  std::uint64_t ldc, stride_c; // floats
  float alpha_r, alpha_i, beta_r, beta_i;
  bool is_complex;
  const DynParams *dyn; // nullable: scale factors and the un-scaling of C
  int *dev_status;
  int tile_n; // 128 or 64
  Tuning tuning;
  // Split-K: k_slices > 1 cuts every tile's K loop into that many CTAs, which write plain
  // partial sums to `partial` (k_slices * batch * m * n floats, [slice][batch][column][row]);
  // the caller then runs launch_splitk_reduce, which applies alpha, beta and the un-scaling.
  std::uint32_t k_slices = 1;
  float *partial = nullptr;
};
cudaError_t launch_tcec_gemm_fused(const FusedGemmArgs &a, cudaStream_t stream);
// Self-test of the bounded mbarrier wait (see cuMpSGEMM_selftest_bounded_wait).
cudaError_t launch_bounded_wait_selftest(int *dev_status, unsigned long long limit_ns,
                                         unsigned long long *dev_waited_ns, cudaStream_t stream);
// Dynamic shared memory and stage count of a tile configuration (for tests/docs).
int tcec_gemm_stages(int tile_n, bool error_correction);

// ---------------------------------------------------------------- statistics & scaling
// Stage-wise entry points so that a multi-GPU caller can all-reduce the slot
// between stages; exp_stats_ext() below chains them.
void exp_stats_init_slot(cuMpSGEMM_handle *h, unsigned id);
template <class T>
void exp_stats_stage1(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                      unsigned ld, unsigned batch, unsigned stride);
void exp_stats_decide1(cuMpSGEMM_handle *h, unsigned id);
template <class T>
void exp_stats_stage2(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                      unsigned ld, unsigned batch, unsigned stride);
void exp_stats_decide2(cuMpSGEMM_handle *h, unsigned id);
template <class T>
void exp_max_only(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                  unsigned ld, unsigned batch, unsigned stride);
// Statistics (full) or maximum exponent only of both operands of a GEMM in shared launches;
// the slots receive what two separate exp_stats_ext / exp_max_ext calls would leave.
template <class T>
void exp_stats_pair(cuMpSGEMM_handle *h, bool full, unsigned id_a, unsigned am, unsigned an,
                    const T *a, unsigned lda, unsigned stride_a, unsigned id_b, unsigned bm,
                    unsigned bn, const T *b, unsigned ldb, unsigned stride_b, unsigned batch);
unsigned next_exp_stats_id(cuMpSGEMM_handle *h);
unsigned next_dyn_launch_id(cuMpSGEMM_handle *h);

enum class ScaleOp : int { scale_a, scale_b, scale_c, reset_a, reset_b };
template <class T>
void launch_scaling(cuMpSGEMM_handle *h, ScaleOp op, unsigned m, unsigned n, T *ptr, unsigned ld,
                    unsigned batch, unsigned stride, unsigned stats_id_a, unsigned stats_id_b,
                    unsigned flag_id);

// Fill the next DynParams record from a flag slot and two statistics slots.
DynParams *prepare_dyn_params(cuMpSGEMM_handle *h, unsigned flag_id, unsigned stats_id_a,
                              unsigned stats_id_b);
// Same, but first derives the flag slot from the two statistics slots' decisions (what
// set_dynamic_launch_buffer_by_exp_stats does) in the same launch.
DynParams *prepare_dyn_params_from_stats(cuMpSGEMM_handle *h, unsigned flag_id,
                                         unsigned stats_id_a, unsigned stats_id_b);

// FP32 GEMMs whose two short dimensions are 2 (tiny_gemm.cu).  long_is_m: C = op(A)(len x 2)
// op(B)(2 x 2); otherwise C = op(A)(2 x 2) op(B)(2 x len).  len must be a power of two.
template <class T>
cublasStatus_t tiny_gemm(cuMpSGEMM_handle *h, bool long_is_m, cublasOperation_t op_A,
                         cublasOperation_t op_B, std::uint64_t len, const T *alpha, const T *a,
                         std::uint64_t lda, std::uint64_t stride_a, const T *b, std::uint64_t ldb,
                         std::uint64_t stride_b, const T *beta, T *c, std::uint64_t ldc,
                         std::uint64_t stride_c, std::uint64_t batch);

// ---------------------------------------------------------------- GEMM dispatch
// Tile for a problem: width 256 / 128 / 64 of the single-CTA kernel (128 rows), or the CTA-pair
// kernel's 256 x 256 tile (error-corrected modes only).  m_exp = rows of the real problem
// (twice m for complex).  The one rule every entry point uses.
struct TileChoice {
  int tile_n;
  bool pair;
};
TileChoice pick_tile(const Tuning &tuning, unsigned num_sms, std::uint64_t m_exp, std::uint64_t n,
                     std::uint64_t batch, bool error_correction);

// Shared implementation behind gemm<T> / gemm_stridedBatch<T>.
// `dyn` != nullptr selects the fused scaling path (scale in the split pass,
// un-scale in the epilogue); `gate_by_flag` launches both kinds gated on
// dyn->gemm_mode.
template <class T>
cublasStatus_t gemm_dispatch(cuMpSGEMM_handle *h, cublasOperation_t op_A, cublasOperation_t op_B,
                             std::uint64_t m, std::uint64_t n, std::uint64_t k, const T *alpha,
                             const T *a, std::uint64_t lda, std::uint64_t stridea, const T *b,
                             std::uint64_t ldb, std::uint64_t strideb, const T *beta, T *c,
                             std::uint64_t ldc, std::uint64_t stridec, std::uint64_t batch,
                             cuMpSGEMM_compute_mode_t mode, const DynParams *dyn,
                             unsigned *used_kernel_module_id, const T *const *a_array = nullptr,
                             const T *const *b_array = nullptr, T *const *c_array = nullptr);
// a_array / b_array / c_array (device arrays of `batch` device pointers, all three or none)
// select pointer-array batches; a, b, c and the strides are then ignored.

// Full AUTO / FP16TCEC_SCALING pipeline (statistics -> flag -> fused GEMM).
// Does not modify A or B.
template <class T>
cublasStatus_t gemm_with_statistics(cuMpSGEMM_handle *h, cublasOperation_t op_A,
                                    cublasOperation_t op_B, std::uint64_t m, std::uint64_t n,
                                    std::uint64_t k, const T *alpha, const T *a, std::uint64_t lda,
                                    std::uint64_t stridea, const T *b, std::uint64_t ldb,
                                    std::uint64_t strideb, const T *beta, T *c, std::uint64_t ldc,
                                    std::uint64_t stridec, std::uint64_t batch,
                                    cuMpSGEMM_compute_mode_t mode, unsigned *stats_id_a_out,
                                    unsigned *stats_id_b_out, unsigned *flag_id_out);

} // namespace cumpsgemm_b200
