// Exponent statistics: max |x| exponent and the (total, underflow) counts
// that drive the AUTO decision.
//
// Semantics follow the reference's src/exp_stats.cu:
//   counting rule            :40-62   (|x| >= ignore -> total++; and |x| < uf -> underflow++;
//                                      complex counts re and im as two values)
//   stage 1 + max exponent   :74-167  (max slot = bits(max|x|) & 0x7f800000)
//   decision 1               :169-184
//   stage 2 (relative thr.)  :187-275 (thresholds (t/2) * 2^e_max, only when undecided)
//   decision 2               :277-293
//   exp_max only             :386-459
//   ring ids                 :12-29, 566-568
//   readback                 :607-629
// Differences, all deliberate: the matrix is read with 128-bit loads in a
// persistent grid sized to the SM count; per-CTA partial counts stay integers
// (the reference stages them through float shared memory); index arithmetic is
// 64-bit throughout; the zero padding the reference's 4-wide loop appends (and
// counts) when m*n is not a multiple of 4 (:101-116, :222-238) is counted only
// when the handle asks for it (cuMpSGEMM_set_count_tail_padding or
// CUMPSGEMM_COUNT_TAIL_PADDING=1), because it is a defect of the counting loop:
// the default counts exactly the matrix elements.
#include "internal.hpp"

namespace cumpsgemm_b200 {
namespace {

constexpr int THREADS = 256;
constexpr int CHUNK = 16384; // floats of one column handled per work item

struct ScanParams {
  const float *ptr;   // complex input viewed as floats
  uint64_t m;         // floats per column
  uint64_t n;         // columns per matrix
  uint64_t ld;        // floats
  uint64_t stride;    // floats
  uint32_t batch;
  uint64_t chunks_per_col;
  uint64_t items;     // batch * n * chunks_per_col
  int vec_ok;         // pointer, ld and stride allow aligned float4 access
  // Zero values the reference's stage kernels append to the tail of every matrix when m*n is
  // not a multiple of 4 and then count like data (0 unless the compatibility switch is on).
  unsigned long long pad_values;
};

// Collapse contiguous storage into one long column so that small matrices still vectorise.
ScanParams make_scan(const void *ptr, uint64_t m, uint64_t n, uint64_t ld, uint32_t batch,
                     uint64_t stride, int floats_per_elem, bool count_tail_padding = false) {
  ScanParams s;
  s.pad_values = 0;
  if (count_tail_padding) {
    const uint64_t matrices = (stride == 0) ? 1u : batch;
    s.pad_values = ((4 - (m * n) % 4) % 4) * static_cast<uint64_t>(floats_per_elem) * matrices;
  }
  s.ptr = reinterpret_cast<const float *>(ptr);
  s.m = m * floats_per_elem;
  s.n = n;
  s.ld = ld * floats_per_elem;
  s.stride = stride * floats_per_elem;
  s.batch = (stride == 0) ? 1u : batch; // reference: stride 0 means a single matrix
  if (s.ld == s.m) {
    s.m = s.m * s.n;
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

// Per-thread partial results.  32-bit counters are enough: one thread visits fewer than
// 2^32 values; they are widened before the cross-thread reduction.
struct Acc {
  float max_abs;
  unsigned int total, underflow;
};

template <bool COUNT, bool MAXV>
__device__ __forceinline__ void visit(float x, Acc &a, float ignore_thr, float uf_thr) {
  const float ax = fabsf(x);
  if (MAXV) a.max_abs = fmaxf(a.max_abs, ax);
  if (COUNT) {
    if (ax >= ignore_thr) {
      a.total++;
      if (ax < uf_thr) a.underflow++;
    }
  }
}

// `bid` of `nblocks` CTAs share the work items of one operand (a launch may serve two operands,
// each with its own range of CTAs).
template <bool COUNT, bool MAXV>
__device__ __forceinline__ void scan_items(const ScanParams &s, Acc &a, float ignore_thr,
                                           float uf_thr, unsigned int bid = blockIdx.x,
                                           unsigned int nblocks = gridDim.x) {
  for (uint64_t item = bid; item < s.items; item += nblocks) {
    const uint64_t chunk = item % s.chunks_per_col;
    const uint64_t col_id = item / s.chunks_per_col;
    const uint64_t col = col_id % s.n;
    const uint64_t b = col_id / s.n;
    const float *p = s.ptr + b * s.stride + col * s.ld;
    const uint64_t begin = chunk * CHUNK;
    const uint64_t end = min(s.m, begin + CHUNK);
    if (s.vec_ok) {
      // begin is a multiple of 4 and the column start is 16-byte aligned
      const uint64_t vec_end = begin + ((end - begin) & ~3ull);
      uint64_t i = begin + threadIdx.x * 4ull;
      // four independent 16-byte loads in flight per thread
      for (; i + 3ull * THREADS * 4ull < vec_end; i += 4ull * THREADS * 4ull) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[u] = *reinterpret_cast<const float4 *>(p + i + static_cast<uint64_t>(u) * THREADS * 4ull);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          visit<COUNT, MAXV>(v[u].x, a, ignore_thr, uf_thr);
          visit<COUNT, MAXV>(v[u].y, a, ignore_thr, uf_thr);
          visit<COUNT, MAXV>(v[u].z, a, ignore_thr, uf_thr);
          visit<COUNT, MAXV>(v[u].w, a, ignore_thr, uf_thr);
        }
      }
      for (; i < vec_end; i += THREADS * 4ull) {
        const float4 v = *reinterpret_cast<const float4 *>(p + i);
        visit<COUNT, MAXV>(v.x, a, ignore_thr, uf_thr);
        visit<COUNT, MAXV>(v.y, a, ignore_thr, uf_thr);
        visit<COUNT, MAXV>(v.z, a, ignore_thr, uf_thr);
        visit<COUNT, MAXV>(v.w, a, ignore_thr, uf_thr);
      }
      for (uint64_t i = vec_end + threadIdx.x; i < end; i += THREADS)
        visit<COUNT, MAXV>(p[i], a, ignore_thr, uf_thr);
    } else {
      for (uint64_t i = begin + threadIdx.x; i < end; i += THREADS)
        visit<COUNT, MAXV>(p[i], a, ignore_thr, uf_thr);
    }
  }
}

// The padded zeros of the compatibility mode, counted once per operand (by thread 0 of its
// first CTA) under the stage's thresholds: |0| >= ignore -> total, and 0 < underflow
// threshold -> underflow.
struct PadCounts {
  unsigned long long total, underflow;
};
__device__ __forceinline__ PadCounts pad_counts(const ScanParams &s, unsigned int bid,
                                                float ignore_thr, float uf_thr) {
  PadCounts p{0ull, 0ull};
  if (s.pad_values != 0 && bid == 0 && threadIdx.x == 0 && 0.f >= ignore_thr) {
    p.total = s.pad_values;
    if (0.f < uf_thr) p.underflow = s.pad_values;
  }
  return p;
}

template <bool COUNT, bool MAXV>
__device__ __forceinline__ void reduce_and_publish(Acc acc, float *max_slot,
                                                   unsigned long long *total_slot,
                                                   unsigned long long *uf_slot,
                                                   PadCounts pad = PadCounts{0ull, 0ull}) {
  struct {
    float max_abs;
    unsigned long long total, underflow;
  } a{acc.max_abs, acc.total + pad.total, acc.underflow + pad.underflow};
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (MAXV) a.max_abs = fmaxf(a.max_abs, __shfl_xor_sync(0xffffffffu, a.max_abs, off));
    if (COUNT) {
      a.total += __shfl_xor_sync(0xffffffffu, a.total, off);
      a.underflow += __shfl_xor_sync(0xffffffffu, a.underflow, off);
    }
  }
  __shared__ float s_max[THREADS / 32];
  __shared__ unsigned long long s_total[THREADS / 32];
  __shared__ unsigned long long s_uf[THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_max[warp] = a.max_abs;
    s_total[warp] = a.total;
    s_uf[warp] = a.underflow;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = 0.f;
    unsigned long long t = 0, u = 0;
    for (int w = 0; w < THREADS / 32; ++w) {
      mx = fmaxf(mx, s_max[w]);
      t += s_total[w];
      u += s_uf[w];
    }
    if (MAXV) {
      // keep only the exponent field: 2^floor(log2 max|x|) as a float
      atomicMax(reinterpret_cast<unsigned int *>(max_slot), __float_as_uint(mx) & 0x7f800000u);
    }
    if (COUNT) {
      if (t) atomicAdd(total_slot, t);
      if (u) atomicAdd(uf_slot, u);
    }
  }
}

__global__ void init_slot_kernel(float *max_slot, unsigned long long *total_slot,
                                 unsigned long long *uf_slot) {
  *max_slot = 0.f;
  if (total_slot != nullptr) *total_slot = 0;
  if (uf_slot != nullptr) *uf_slot = 0;
}

__global__ void __launch_bounds__(THREADS)
    stage1_kernel(const ScanParams s, float *max_slot, unsigned long long *total_slot,
                  unsigned long long *uf_slot, float ignore_thr, float uf_thr) {
  Acc a{0.f, 0u, 0u};
  scan_items<true, true>(s, a, ignore_thr, uf_thr);
  reduce_and_publish<true, true>(a, max_slot, total_slot, uf_slot,
                                 pad_counts(s, blockIdx.x, ignore_thr, uf_thr));
}

__global__ void decide1_kernel(int *mode, const float *max_slot, unsigned long long *total_slot,
                               unsigned long long *uf_slot, float tolerance) {
  // the comparison is carried out in float, as in the reference
  if ((static_cast<float>(*uf_slot) > static_cast<float>(*total_slot) * tolerance) ||
      (*max_slot > 0.f && *total_slot == 0)) {
    *mode = CUMPSGEMM_UNDEFINED;
    *total_slot = 0;
    *uf_slot = 0;
  } else {
    *mode = CUMPSGEMM_FP16TCEC;
  }
}

__global__ void __launch_bounds__(THREADS)
    stage2_kernel(const ScanParams s, const int *mode, const float *max_slot,
                  unsigned long long *total_slot, unsigned long long *uf_slot,
                  float half_ignore_thr, float half_uf_thr) {
  if (*mode != CUMPSGEMM_UNDEFINED) return; // launch-and-exit
  const float mx = *max_slot;
  Acc a{0.f, 0u, 0u};
  scan_items<true, false>(s, a, half_ignore_thr * mx, half_uf_thr * mx);
  reduce_and_publish<true, false>(a, nullptr, total_slot, uf_slot,
                                  pad_counts(s, blockIdx.x, half_ignore_thr * mx, half_uf_thr * mx));
}

__global__ void decide2_kernel(int *mode, const unsigned long long *total_slot,
                               const unsigned long long *uf_slot, float tolerance) {
  if (*mode != CUMPSGEMM_UNDEFINED) return;
  if (static_cast<float>(*uf_slot) <= static_cast<float>(*total_slot) * tolerance) {
    *mode = CUMPSGEMM_FP16TCEC_SCALING;
  } else {
    *mode = CUMPSGEMM_TF32TCEC;
  }
}

__global__ void __launch_bounds__(THREADS) max_only_kernel(const ScanParams s, float *max_slot) {
  Acc a{0.f, 0u, 0u};
  scan_items<false, true>(s, a, 0.f, 0.f);
  reduce_and_publish<false, true>(a, max_slot, nullptr, nullptr);
}

// ---------------------------------------------------------------- fused variants
// exp_stats_ext / exp_max_ext outside the profiler use these: slot initialisation, scan and
// decision in one launch per stage (two launches instead of five, one instead of two), which
// is what an AUTO GEMM on a small matrix spends most of its time on otherwise.  Every CTA
// writes its partial result to its own scratch record and takes a ticket; the CTA that draws
// the last ticket adds the records up, writes the slot and takes the decision, then puts the
// ticket counter back to zero for the next launch.  Sums of integers and a maximum do not
// depend on the order, so the slot receives the same bits as on the five-launch path.
struct ScanPartial {
  unsigned long long total, underflow;
  unsigned int max_bits, pad;
};

struct ScanTotals {
  float max_abs;
  unsigned long long total, underflow;
};

// Block-wide reduction of (max, total, underflow); the result is valid in thread 0.
__device__ __forceinline__ ScanTotals block_reduce(ScanTotals a) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    a.max_abs = fmaxf(a.max_abs, __shfl_xor_sync(0xffffffffu, a.max_abs, off));
    a.total += __shfl_xor_sync(0xffffffffu, a.total, off);
    a.underflow += __shfl_xor_sync(0xffffffffu, a.underflow, off);
  }
  __shared__ float s_max[THREADS / 32];
  __shared__ unsigned long long s_total[THREADS / 32];
  __shared__ unsigned long long s_uf[THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads(); // the arrays may still be read from an earlier call
  if (lane == 0) {
    s_max[warp] = a.max_abs;
    s_total[warp] = a.total;
    s_uf[warp] = a.underflow;
  }
  __syncthreads();
  ScanTotals r{0.f, 0ull, 0ull};
  if (threadIdx.x == 0) {
    for (int w = 0; w < THREADS / 32; ++w) {
      r.max_abs = fmaxf(r.max_abs, s_max[w]);
      r.total += s_total[w];
      r.underflow += s_uf[w];
    }
  }
  return r;
}

// Returns true in thread 0 of the CTA that drew the last ticket, with the grid-wide totals in
// *out; false everywhere else.
__device__ __forceinline__ bool grid_reduce(Acc acc, ScanPartial *partials, unsigned int *ticket,
                                            ScanTotals *out, unsigned int bid = blockIdx.x,
                                            unsigned int nblocks = gridDim.x,
                                            PadCounts pad = PadCounts{0ull, 0ull}) {
  const ScanTotals mine = block_reduce(
      ScanTotals{acc.max_abs, acc.total + pad.total, acc.underflow + pad.underflow});
  __shared__ bool s_last;
  if (threadIdx.x == 0) {
    ScanPartial rec;
    rec.total = mine.total;
    rec.underflow = mine.underflow;
    rec.max_bits = __float_as_uint(mine.max_abs);
    rec.pad = 0;
    partials[bid] = rec;
    __threadfence();
    s_last = (atomicAdd(ticket, 1u) == nblocks - 1);
  }
  __syncthreads();
  if (!s_last) return false;
  __threadfence();
  ScanTotals sum{0.f, 0ull, 0ull};
  for (unsigned int i = threadIdx.x; i < nblocks; i += THREADS) {
    const volatile ScanPartial *r = partials + i;
    sum.max_abs = fmaxf(sum.max_abs, __uint_as_float(r->max_bits));
    sum.total += r->total;
    sum.underflow += r->underflow;
  }
  *out = block_reduce(sum);
  if (threadIdx.x == 0) *ticket = 0;
  return threadIdx.x == 0;
}

// Where one operand's results go.
struct StatSlots {
  int *mode;
  float *max_slot;
  unsigned long long *total_slot, *uf_slot;
};

__device__ __forceinline__ void fused_stage1_body(const ScanParams &s, const StatSlots &o,
                                                  float ignore_thr, float uf_thr, float tolerance,
                                                  ScanPartial *partials, unsigned int *ticket,
                                                  unsigned int bid, unsigned int nblocks) {
  Acc a{0.f, 0u, 0u};
  scan_items<true, true>(s, a, ignore_thr, uf_thr, bid, nblocks);
  ScanTotals t;
  if (!grid_reduce(a, partials, ticket, &t, bid, nblocks, pad_counts(s, bid, ignore_thr, uf_thr)))
    return;
  // keep only the exponent field: 2^floor(log2 max|x|) as a float
  const float mx = __uint_as_float(__float_as_uint(t.max_abs) & 0x7f800000u);
  *o.max_slot = mx;
  // the comparison is carried out in float, as in the reference
  if ((static_cast<float>(t.underflow) > static_cast<float>(t.total) * tolerance) ||
      (mx > 0.f && t.total == 0)) {
    *o.mode = CUMPSGEMM_UNDEFINED;
    *o.total_slot = 0;
    *o.uf_slot = 0;
  } else {
    *o.mode = CUMPSGEMM_FP16TCEC;
    *o.total_slot = t.total;
    *o.uf_slot = t.underflow;
  }
}

__device__ __forceinline__ void fused_stage2_body(const ScanParams &s, const StatSlots &o,
                                                  float half_ignore_thr, float half_uf_thr,
                                                  float tolerance, ScanPartial *partials,
                                                  unsigned int *ticket, unsigned int bid,
                                                  unsigned int nblocks) {
  if (*o.mode != CUMPSGEMM_UNDEFINED) return; // launch-and-exit, uniform over the operand's CTAs
  const float mx = *o.max_slot;
  Acc a{0.f, 0u, 0u};
  scan_items<true, false>(s, a, half_ignore_thr * mx, half_uf_thr * mx, bid, nblocks);
  ScanTotals t;
  if (!grid_reduce(a, partials, ticket, &t, bid, nblocks,
                   pad_counts(s, bid, half_ignore_thr * mx, half_uf_thr * mx)))
    return;
  *o.total_slot = t.total;
  *o.uf_slot = t.underflow;
  *o.mode = (static_cast<float>(t.underflow) <= static_cast<float>(t.total) * tolerance)
                ? CUMPSGEMM_FP16TCEC_SCALING
                : CUMPSGEMM_TF32TCEC;
}

__device__ __forceinline__ void fused_max_body(const ScanParams &s, float *max_slot,
                                               ScanPartial *partials, unsigned int *ticket,
                                               unsigned int bid, unsigned int nblocks) {
  Acc a{0.f, 0u, 0u};
  scan_items<false, true>(s, a, 0.f, 0.f, bid, nblocks);
  ScanTotals t;
  if (!grid_reduce(a, partials, ticket, &t, bid, nblocks)) return;
  *max_slot = __uint_as_float(__float_as_uint(t.max_abs) & 0x7f800000u);
}

__global__ void __launch_bounds__(THREADS, 8)
    fused_stage1_kernel(const ScanParams s, const StatSlots o, float ignore_thr, float uf_thr,
                        float tolerance, ScanPartial *partials, unsigned int *ticket) {
  fused_stage1_body(s, o, ignore_thr, uf_thr, tolerance, partials, ticket, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(THREADS, 8)
    fused_stage2_kernel(const ScanParams s, const StatSlots o, float half_ignore_thr,
                        float half_uf_thr, float tolerance, ScanPartial *partials,
                        unsigned int *ticket) {
  fused_stage2_body(s, o, half_ignore_thr, half_uf_thr, tolerance, partials, ticket, blockIdx.x,
                    gridDim.x);
}

__global__ void __launch_bounds__(THREADS, 8)
    fused_max_only_kernel(const ScanParams s, float *max_slot, ScanPartial *partials,
                          unsigned int *ticket) {
  fused_max_body(s, max_slot, partials, ticket, blockIdx.x, gridDim.x);
}

// Two operands in one launch (the A and B of a GEMM): CTAs [0, grid_a) scan the first, the
// rest the second; each operand has its own records (second half of `partials`) and ticket.
struct DualScan {
  ScanParams s[2];
  StatSlots o[2];
  unsigned int grid_a;
  unsigned int records_per_operand;
};

__global__ void __launch_bounds__(THREADS, 8)
    fused_stage1_dual_kernel(const DualScan d, float ignore_thr, float uf_thr, float tolerance,
                             ScanPartial *partials, unsigned int *tickets) {
  CUMPSGEMM_CHAIN_HEAD_ENTRY(); // stage 2 may be scheduled while this grid drains
  const unsigned int w = blockIdx.x >= d.grid_a ? 1u : 0u;
  const unsigned int bid = w ? blockIdx.x - d.grid_a : blockIdx.x;
  const unsigned int nb = w ? gridDim.x - d.grid_a : d.grid_a;
  fused_stage1_body(d.s[w], d.o[w], ignore_thr, uf_thr, tolerance,
                    partials + w * d.records_per_operand, tickets + w, bid, nb);
}

__global__ void __launch_bounds__(THREADS, 8)
    fused_stage2_dual_kernel(const DualScan d, float half_ignore_thr, float half_uf_thr,
                             float tolerance, ScanPartial *partials, unsigned int *tickets) {
  CUMPSGEMM_CHAINED_KERNEL_ENTRY(); // launched behind stage 1: its results are complete after this
  const unsigned int w = blockIdx.x >= d.grid_a ? 1u : 0u;
  const unsigned int bid = w ? blockIdx.x - d.grid_a : blockIdx.x;
  const unsigned int nb = w ? gridDim.x - d.grid_a : d.grid_a;
  fused_stage2_body(d.s[w], d.o[w], half_ignore_thr, half_uf_thr, tolerance,
                    partials + w * d.records_per_operand, tickets + w, bid, nb);
}

__global__ void __launch_bounds__(THREADS, 8)
    fused_max_dual_kernel(const DualScan d, ScanPartial *partials, unsigned int *tickets) {
  CUMPSGEMM_CHAIN_HEAD_ENTRY();
  const unsigned int w = blockIdx.x >= d.grid_a ? 1u : 0u;
  const unsigned int bid = w ? blockIdx.x - d.grid_a : blockIdx.x;
  const unsigned int nb = w ? gridDim.x - d.grid_a : d.grid_a;
  fused_max_body(d.s[w], d.o[w].max_slot, partials + w * d.records_per_operand, tickets + w, bid,
                 nb);
}

__global__ void configure_mode_buffer_kernel(int *mode_buffer) {
  mode_buffer[0] = CUMPSGEMM_TF32TCEC;
  mode_buffer[1] = CUMPSGEMM_FP16TCEC;
}

unsigned scan_grid(const cuMpSGEMM_handle *h, const ScanParams &s) {
  const uint64_t cap = static_cast<uint64_t>(h->num_sms) * 8; // 8 CTAs of 256 threads per SM
  return static_cast<unsigned>(s.items < cap ? (s.items ? s.items : 1) : cap);
}

template <class T> constexpr int floats_per_elem() { return sizeof(T) / sizeof(float); }

struct ScopedTimer {
  cuMpSGEMM_handle *h;
  const char *name;
  ScopedTimer(cuMpSGEMM_handle *h_, const char *n) : h(h_), name(n) {
    if (h->exp_stats.profiling_enabled) h->exp_stats.profiler.start(name, h->cuda_stream);
  }
  ~ScopedTimer() {
    if (h->exp_stats.profiling_enabled) h->exp_stats.profiler.stop(name, h->cuda_stream);
  }
};

} // namespace

// ---------------------------------------------------------------- profiler
void Profiler::start(const std::string &name, cudaStream_t s) {
  Entry &e = entries[name];
  if (e.e0 == nullptr) {
    cudaEventCreate(&e.e0);
    cudaEventCreate(&e.e1);
  }
  cudaStreamSynchronize(s);
  cudaEventRecord(e.e0, s);
}
void Profiler::stop(const std::string &name, cudaStream_t s) {
  auto it = entries.find(name);
  if (it == entries.end() || it->second.e0 == nullptr) return;
  Entry &e = it->second;
  cudaEventRecord(e.e1, s);
  cudaEventSynchronize(e.e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e.e0, e.e1);
  e.sum_s += static_cast<double>(ms) * 1e-3;
  e.n += 1;
}
void Profiler::clear() {
  for (auto &kv : entries) {
    kv.second.sum_s = 0;
    kv.second.n = 0;
  }
}
Profiler::~Profiler() {
  for (auto &kv : entries) {
    if (kv.second.e0) cudaEventDestroy(kv.second.e0);
    if (kv.second.e1) cudaEventDestroy(kv.second.e1);
  }
}

// ---------------------------------------------------------------- ring ids
// ids 0 and 1 are reserved; the ring runs 2 .. buffer_length-1 and wraps to 2.
unsigned next_exp_stats_id(cuMpSGEMM_handle *h) {
  h->exp_stats.current_buffer_id++;
  if (h->exp_stats.current_buffer_id < h->exp_stats.buffer_length)
    return h->exp_stats.current_buffer_id;
  h->exp_stats.current_buffer_id = 2;
  return 2;
}

// ---------------------------------------------------------------- stages
void exp_stats_init_slot(cuMpSGEMM_handle *h, unsigned id) {
  init_slot_kernel<<<1, 1, 0, h->cuda_stream>>>(h->exp_stats.dev_max + id,
                                                h->exp_stats.dev_total + id,
                                                h->exp_stats.dev_underflow + id);
}

template <class T>
void exp_stats_stage1(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                      unsigned ld, unsigned batch, unsigned stride) {
  const ScanParams s = make_scan(ptr, m, n, ld, batch, stride, floats_per_elem<T>(),
                                 h->exp_stats.count_tail_padding);
  stage1_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(
      s, h->exp_stats.dev_max + id, h->exp_stats.dev_total + id, h->exp_stats.dev_underflow + id,
      h->exp_stats.ignore_threshold, h->exp_stats.underflow_threshold);
}

void exp_stats_decide1(cuMpSGEMM_handle *h, unsigned id) {
  decide1_kernel<<<1, 1, 0, h->cuda_stream>>>(
      h->exp_stats.dev_mode + id, h->exp_stats.dev_max + id, h->exp_stats.dev_total + id,
      h->exp_stats.dev_underflow + id, h->exp_stats.underflow_tolerance_rate);
}

template <class T>
void exp_stats_stage2(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                      unsigned ld, unsigned batch, unsigned stride) {
  const ScanParams s = make_scan(ptr, m, n, ld, batch, stride, floats_per_elem<T>(),
                                 h->exp_stats.count_tail_padding);
  stage2_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(
      s, h->exp_stats.dev_mode + id, h->exp_stats.dev_max + id, h->exp_stats.dev_total + id,
      h->exp_stats.dev_underflow + id, h->exp_stats.ignore_threshold / 2,
      h->exp_stats.underflow_threshold / 2);
}

void exp_stats_decide2(cuMpSGEMM_handle *h, unsigned id) {
  decide2_kernel<<<1, 1, 0, h->cuda_stream>>>(h->exp_stats.dev_mode + id,
                                              h->exp_stats.dev_total + id,
                                              h->exp_stats.dev_underflow + id,
                                              h->exp_stats.underflow_tolerance_rate);
}

template <class T>
void exp_max_only(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                  unsigned ld, unsigned batch, unsigned stride) {
  {
    ScopedTimer t(h, "exp_max_init");
    init_slot_kernel<<<1, 1, 0, h->cuda_stream>>>(h->exp_stats.dev_max + id, nullptr, nullptr);
  }
  ScopedTimer t(h, "exp_max");
  const ScanParams s = make_scan(ptr, m, n, ld, batch, stride, floats_per_elem<T>());
  max_only_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(s, h->exp_stats.dev_max + id);
}

// One launch per stage (see the fused kernels above).  Scratch layout: two operands' records
// (num_sms * 8 each), then two tickets.
inline unsigned int scan_records(const cuMpSGEMM_handle *h) { return h->num_sms * 8u; }
inline ScanPartial *scan_partials(cuMpSGEMM_handle *h) {
  return reinterpret_cast<ScanPartial *>(h->exp_stats.dev_scan_scratch);
}
inline unsigned int *scan_tickets(cuMpSGEMM_handle *h) {
  return reinterpret_cast<unsigned int *>(scan_partials(h) + 2u * scan_records(h));
}
inline StatSlots stat_slots(cuMpSGEMM_handle *h, unsigned id) {
  auto &es = h->exp_stats;
  return StatSlots{es.dev_mode + id, es.dev_max + id, es.dev_total + id, es.dev_underflow + id};
}

template <class T>
void exp_stats_fused(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                     unsigned ld, unsigned batch, unsigned stride) {
  const ScanParams s = make_scan(ptr, m, n, ld, batch, stride, floats_per_elem<T>(),
                                 h->exp_stats.count_tail_padding);
  auto &es = h->exp_stats;
  fused_stage1_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(
      s, stat_slots(h, id), es.ignore_threshold, es.underflow_threshold,
      es.underflow_tolerance_rate, scan_partials(h), scan_tickets(h));
  fused_stage2_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(
      s, stat_slots(h, id), es.ignore_threshold / 2, es.underflow_threshold / 2,
      es.underflow_tolerance_rate, scan_partials(h), scan_tickets(h));
}

template <class T>
void exp_max_fused(cuMpSGEMM_handle *h, unsigned id, unsigned m, unsigned n, const T *ptr,
                   unsigned ld, unsigned batch, unsigned stride) {
  const ScanParams s = make_scan(ptr, m, n, ld, batch, stride, floats_per_elem<T>());
  fused_max_only_kernel<<<scan_grid(h, s), THREADS, 0, h->cuda_stream>>>(
      s, h->exp_stats.dev_max + id, scan_partials(h), scan_tickets(h));
}

// Statistics (full = true) or maximum exponent only of the two operands of a GEMM, two slots,
// in two launches resp. one.  Same slot contents as two separate calls.
template <class T>
void exp_stats_pair(cuMpSGEMM_handle *h, bool full, unsigned id_a, unsigned am, unsigned an,
                    const T *a, unsigned lda, unsigned stride_a, unsigned id_b, unsigned bm,
                    unsigned bn, const T *b, unsigned ldb, unsigned stride_b, unsigned batch) {
  DualScan d;
  const bool pad = full && h->exp_stats.count_tail_padding;
  d.s[0] = make_scan(a, am, an, lda, batch, stride_a, floats_per_elem<T>(), pad);
  d.s[1] = make_scan(b, bm, bn, ldb, batch, stride_b, floats_per_elem<T>(), pad);
  d.o[0] = stat_slots(h, id_a);
  d.o[1] = stat_slots(h, id_b);
  d.grid_a = scan_grid(h, d.s[0]);
  d.records_per_operand = scan_records(h);
  const unsigned grid = d.grid_a + scan_grid(h, d.s[1]);
  auto &es = h->exp_stats;
  if (!full) {
    fused_max_dual_kernel<<<grid, THREADS, 0, h->cuda_stream>>>(d, scan_partials(h),
                                                                scan_tickets(h));
    return;
  }
  fused_stage1_dual_kernel<<<grid, THREADS, 0, h->cuda_stream>>>(
      d, es.ignore_threshold, es.underflow_threshold, es.underflow_tolerance_rate,
      scan_partials(h), scan_tickets(h));
  launch_chained(fused_stage2_dual_kernel, grid, THREADS, 0, h->cuda_stream, d,
                 es.ignore_threshold / 2, es.underflow_threshold / 2, es.underflow_tolerance_rate,
                 scan_partials(h), scan_tickets(h));
}

#define INSTANTIATE(T)                                                                           \
  template void exp_stats_stage1<T>(cuMpSGEMM_handle *, unsigned, unsigned, unsigned, const T *, \
                                    unsigned, unsigned, unsigned);                               \
  template void exp_stats_stage2<T>(cuMpSGEMM_handle *, unsigned, unsigned, unsigned, const T *, \
                                    unsigned, unsigned, unsigned);                               \
  template void exp_max_only<T>(cuMpSGEMM_handle *, unsigned, unsigned, unsigned, const T *,     \
                                unsigned, unsigned, unsigned);                                   \
  template void exp_stats_fused<T>(cuMpSGEMM_handle *, unsigned, unsigned, unsigned, const T *,  \
                                   unsigned, unsigned, unsigned);                                \
  template void exp_max_fused<T>(cuMpSGEMM_handle *, unsigned, unsigned, unsigned, const T *,    \
                                 unsigned, unsigned, unsigned);                                  \
  template void exp_stats_pair<T>(cuMpSGEMM_handle *, bool, unsigned, unsigned, unsigned,        \
                                  const T *, unsigned, unsigned, unsigned, unsigned, unsigned,   \
                                  const T *, unsigned, unsigned, unsigned);
INSTANTIATE(float)
INSTANTIATE(cuComplex)
#undef INSTANTIATE

void configure_mode_buffer(cuMpSGEMM_handle *h) {
  configure_mode_buffer_kernel<<<1, 1, 0, h->cuda_stream>>>(h->exp_stats.dev_mode);
}

} // namespace cumpsgemm_b200

// ---------------------------------------------------------------- public C++ API
namespace cumpsgemm {
using namespace cumpsgemm_b200;

template <class T>
unsigned exp_stats_ext(cuMpSGEMM_handle_t handle, const unsigned m, const unsigned n,
                       const T *const ptr, const unsigned ld, const unsigned batch_size,
                       const unsigned stride) {
  DeviceGuard guard(handle->device);
  const unsigned id = next_exp_stats_id(handle);
  if (!handle->exp_stats.profiling_enabled) {
    // two launches; the five separate ones below exist for the named timers of the profiler
    exp_stats_fused<T>(handle, id, m, n, ptr, ld, batch_size, stride);
    mark_stream_work(handle);
    return id;
  }
  {
    ScopedTimer t(handle, "exp_stats_init");
    exp_stats_init_slot(handle, id);
  }
  {
    ScopedTimer t(handle, "exp_stats_1");
    exp_stats_stage1<T>(handle, id, m, n, ptr, ld, batch_size, stride);
  }
  {
    ScopedTimer t(handle, "exp_stats_set_1");
    exp_stats_decide1(handle, id);
  }
  {
    ScopedTimer t(handle, "exp_stats_2");
    exp_stats_stage2<T>(handle, id, m, n, ptr, ld, batch_size, stride);
  }
  {
    ScopedTimer t(handle, "exp_stats_set_2");
    exp_stats_decide2(handle, id);
  }
  return id;
}
template unsigned exp_stats_ext<float>(cuMpSGEMM_handle_t, const unsigned, const unsigned,
                                       const float *const, const unsigned, const unsigned,
                                       const unsigned);
template unsigned exp_stats_ext<cuComplex>(cuMpSGEMM_handle_t, const unsigned, const unsigned,
                                           const cuComplex *const, const unsigned, const unsigned,
                                           const unsigned);

template <class T>
unsigned exp_max_ext(cuMpSGEMM_handle_t handle, const unsigned m, const unsigned n,
                     const T *const ptr, const unsigned ld, const unsigned batch_size,
                     const unsigned stride) {
  DeviceGuard guard(handle->device);
  const unsigned id = next_exp_stats_id(handle);
  if (!handle->exp_stats.profiling_enabled)
    exp_max_fused<T>(handle, id, m, n, ptr, ld, batch_size, stride);
  else
    exp_max_only<T>(handle, id, m, n, ptr, ld, batch_size, stride);
  mark_stream_work(handle);
  return id;
}
template unsigned exp_max_ext<float>(cuMpSGEMM_handle_t, const unsigned, const unsigned,
                                     const float *const, const unsigned, const unsigned,
                                     const unsigned);
template unsigned exp_max_ext<cuComplex>(cuMpSGEMM_handle_t, const unsigned, const unsigned,
                                         const cuComplex *const, const unsigned, const unsigned,
                                         const unsigned);

std::pair<std::size_t, std::size_t> get_exp_stats(cuMpSGEMM_handle_t handle,
                                                  const unsigned buffer_id) {
  DeviceGuard guard(handle->device);
  unsigned long long total = 0, uf = 0;
  cudaMemcpyAsync(&total, handle->exp_stats.dev_total + buffer_id, sizeof(total),
                  cudaMemcpyDeviceToHost, handle->cuda_stream);
  cudaMemcpyAsync(&uf, handle->exp_stats.dev_underflow + buffer_id, sizeof(uf),
                  cudaMemcpyDeviceToHost, handle->cuda_stream);
  cudaStreamSynchronize(handle->cuda_stream);
  return std::pair<std::size_t, std::size_t>{uf, total};
}

unsigned get_current_exp_stats_buffer_id(cuMpSGEMM_handle_t handle) {
  return handle->exp_stats.current_buffer_id;
}

void reset_exp_stats_buffer_id(cuMpSGEMM_handle_t handle) {
  handle->exp_stats.current_buffer_id = 1;
}

void set_exp_stats_params(cuMpSGEMM_handle_t handle, const float ignore_threshold,
                          const float underflow_threshold,
                          const float underflow_ratio_tolerance) {
  handle->exp_stats.ignore_threshold = ignore_threshold;
  handle->exp_stats.underflow_threshold = underflow_threshold;
  handle->exp_stats.underflow_tolerance_rate = underflow_ratio_tolerance;
}

void enable_exp_stats(cuMpSGEMM_handle_t handle) { handle->exp_stats.enabled = true; }
void disable_exp_stats(cuMpSGEMM_handle_t handle) { handle->exp_stats.enabled = false; }

float get_max_exp(cuMpSGEMM_handle_t handle, const unsigned buffer_id) {
  DeviceGuard guard(handle->device);
  float v = 0.f;
  cudaMemcpyAsync(&v, handle->exp_stats.dev_max + buffer_id, sizeof(float),
                  cudaMemcpyDeviceToHost, handle->cuda_stream);
  cudaStreamSynchronize(handle->cuda_stream);
  return v;
}

cuMpSGEMM_compute_mode_t get_exp_stats_compute_mode_level(cuMpSGEMM_handle_t handle,
                                                          const unsigned buffer_id) {
  DeviceGuard guard(handle->device);
  int mode = 0;
  cudaMemcpyAsync(&mode, handle->exp_stats.dev_mode + buffer_id, sizeof(int),
                  cudaMemcpyDeviceToHost, handle->cuda_stream);
  cudaStreamSynchronize(handle->cuda_stream);
  return static_cast<cuMpSGEMM_compute_mode_t>(mode);
}

void enable_exp_stats_profiling(cuMpSGEMM_handle *const handle) {
  handle->exp_stats.profiling_enabled = true;
}
void disable_exp_stats_profiling(cuMpSGEMM_handle *const handle) {
  handle->exp_stats.profiling_enabled = false;
}
void reset_exp_stats_profiling(cuMpSGEMM_handle *const handle) {
  handle->exp_stats.profiler.clear();
}
void print_exp_stats_profiling(cuMpSGEMM_handle *const handle, unsigned csv) {
  for (const auto &kv : handle->exp_stats.profiler.entries) {
    if (kv.second.n == 0) continue;
    if (csv) {
      std::printf("%s,%e,%lu\n", kv.first.c_str(), kv.second.sum_s,
                  static_cast<unsigned long>(kv.second.n));
    } else {
      std::printf("%20s : %e [s] (n = %lu)\n", kv.first.c_str(), kv.second.sum_s,
                  static_cast<unsigned long>(kv.second.n));
    }
  }
  std::fflush(stdout);
}

namespace debug {
std::unordered_map<std::string, stats_t>
get_exp_stats_profiling_result(cuMpSGEMM_handle *const handle) {
  std::unordered_map<std::string, stats_t> result;
  for (const auto &kv : handle->exp_stats.profiler.entries) {
    if (kv.second.n == 0) continue;
    result.insert(std::make_pair(kv.first, stats_t{kv.second.sum_s, kv.second.n}));
  }
  return result;
}
} // namespace debug
} // namespace cumpsgemm
