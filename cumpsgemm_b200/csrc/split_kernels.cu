// Operand split pass: FP32 / complex64 column-major operand -> K-major hi/lo panels.
//
// Restates, as one HBM-bound pass per operand, the FP32 -> (hi, lo) split the
// reference performs inside its fragment loads for every warp and every k-step
// (src/device_tcec_wrapper.hpp:72-80 calling mtk::wmma::tcec::load_matrix_sync),
// together with the operand addressing of its global->shared loaders
// (src/dmem_accessor.hpp:8-170: op N/T/C, leading dimension, edge zero fill,
// conjugation).
//
//   FP16:  hi = RN_fp16(v),  lo = RN_fp16((v - float(hi)) * 2^11)
//   TF32:  hi = RNA_tf32(v), lo = RNA_tf32(v - hi)
// where v = x * scale (scale is an exact power of two, 1 when no scaling).
//
// Panel layout (element type half or float), blocked along K in units of 128 bytes
// (KBE = 64 half or 32 float elements), z = 0 (hi), 1 (lo):
//   panel[(((b * planes + z) * (k_pad / KBE) + kk / KBE) * rows_pad + r) * KBE + kk % KBE]
// so the 128-byte K slices of consecutive rows are contiguous: the box one TMA load of the
// GEMM kernel fetches (128 rows x 128 bytes) is one 16 KiB run of memory instead of 128 lines
// a whole panel row apart.  rows_pad / k_pad are multiples of 64 and every padding element is
// written as zero on every call, so the GEMM kernel needs no edge handling.
//
// Complex operands are expanded to real ones so that the GEMM kernel is a real
// GEMM producing interleaved (re, im) rows of C:
//   A' (2m x 2k): rows (2i, 2i+1), cols (2l, 2l+1) = [[re, -im], [im, re]] of a(i,l)
//   B' (n x 2k):  row j, cols (2l, 2l+1) = (re, im) of b(l,j)
// (a, b after op; op C conjugates).
#include "internal.hpp"

#include <cuda_fp16.h>

namespace cumpsgemm_b200 {
namespace {

constexpr int TILE = 64;       // expanded rows and expanded K per CTA
constexpr int THREADS = 256;

__device__ __forceinline__ float to_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// Offset of element (r, kk) inside one plane of a panel (see the layout above).
template <int KIND>
__device__ __forceinline__ uint64_t panel_offset(uint64_t r, uint64_t kk, uint32_t rows_pad) {
  constexpr uint64_t KBE = (KIND == 0) ? 64 : 32;
  return ((kk / KBE) * rows_pad + r) * KBE + (kk % KBE);
}

struct SplitParams {
  const float *src; // complex sources are addressed as pairs of floats
  const float *const *src_array; // pointer-array batches: matrix b starts at src_array[b]
  uint64_t ld, stride;
  uint64_t rows, k; // logical source extent (complex elements for complex input)
  void *panel;
  uint32_t rows_pad, k_pad;
  uint32_t planes; // 1 or 2
  const DynParams *dyn;
  int operand; // 0 = A, 1 = B
  int conj;
  int src_k_contig;
};

// MODE: 0 = real, 1 = complex A', 2 = complex B'
template <int KIND, int MODE>
__device__ __forceinline__ void split_generic_body(const SplitParams &p, const uint3 bid,
                                                   float (*tile)[TILE + 1]) {
  constexpr int MY_MODE = (KIND == 0) ? CUMPSGEMM_FP16TCEC : CUMPSGEMM_TF32TCEC;
  float scale = 1.f;
  if (p.dyn != nullptr) {
    if (p.dyn->gemm_mode != MY_MODE) return;
    scale = (p.operand == 0) ? p.dyn->scale_a : p.dyn->scale_b;
  }

  // Source tile in source coordinates; complex tiles store (re, im) in adjacent columns.
  constexpr int SR = (MODE == 1) ? TILE / 2 : TILE; // source rows per tile
  constexpr int SK = (MODE == 0) ? TILE : TILE / 2; // source k per tile
  constexpr int ES = (MODE == 0) ? 1 : 2;           // floats per source element

  const uint32_t b = bid.z;
  const uint64_t r0 = static_cast<uint64_t>(bid.y) * SR;
  const uint64_t k0 = static_cast<uint64_t>(bid.x) * SK;
  const float *src = (p.src_array != nullptr)
                         ? p.src_array[b]
                         : p.src + static_cast<uint64_t>(b) * p.stride * ES;

  // ---- phase 1: coalesced read along the source-contiguous dimension
  if constexpr (ES == 2) {
    // Complex: a thread's 4 (A') or 8 (B') loads are all issued before the first
    // shared-memory store; with one load per store the kernel spent over half of its warp
    // cycles waiting for the load just issued.
    constexpr int PER = SR * SK / THREADS;
    float2 v[PER];
#pragma unroll
    for (int q = 0; q < PER; ++q) {
      const int idx = threadIdx.x + q * THREADS;
      const int r = p.src_k_contig ? idx / SK : idx % SR;
      const int kk = p.src_k_contig ? idx % SK : idx / SR;
      const uint64_t gr = r0 + r, gk = k0 + kk;
      v[q] = make_float2(0.f, 0.f);
      if (gr < p.rows && gk < p.k)
        v[q] = reinterpret_cast<const float2 *>(src)[p.src_k_contig ? (gk + gr * p.ld)
                                                                    : (gr + gk * p.ld)];
    }
#pragma unroll
    for (int q = 0; q < PER; ++q) {
      const int idx = threadIdx.x + q * THREADS;
      const int r = p.src_k_contig ? idx / SK : idx % SR;
      const int kk = p.src_k_contig ? idx % SK : idx / SR;
      tile[r][2 * kk] = v[q].x * scale;
      tile[r][2 * kk + 1] = (p.conj ? -v[q].y : v[q].y) * scale;
    }
  } else {
    for (int idx = threadIdx.x; idx < SR * SK; idx += THREADS) {
      int r, kk;
      if (p.src_k_contig) {
        kk = idx % SK;
        r = idx / SK;
      } else {
        r = idx % SR;
        kk = idx / SR;
      }
      const uint64_t gr = r0 + r, gk = k0 + kk;
      float re = 0.f;
      if (gr < p.rows && gk < p.k)
        re = src[p.src_k_contig ? (gk + gr * p.ld) : (gr + gk * p.ld)] * scale;
      tile[r][kk] = re;
    }
  }
  __syncthreads();

  // ---- phase 2: each thread converts 8 consecutive expanded-K values of one expanded row
  const uint64_t er0 = static_cast<uint64_t>(bid.y) * TILE; // expanded row origin
  const uint64_t ek0 = static_cast<uint64_t>(bid.x) * TILE; // expanded K origin
  const uint64_t plane_elems = static_cast<uint64_t>(p.rows_pad) * p.k_pad;
#pragma unroll
  for (int it = 0; it < TILE * TILE / (THREADS * 8); ++it) {
    const int er = (threadIdx.x >> 3) + it * (THREADS >> 3);
    const int ek = (threadIdx.x & 7) * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = ek + j;
      if constexpr (MODE == 0 || MODE == 2) {
        v[j] = tile[er][c];
      } else {
        const int sr = er >> 1;
        const bool im_row = (er & 1) != 0;
        const bool odd = (c & 1) != 0;
        // [[re, -im], [im, re]]
        const float x = tile[sr][(c & ~1) + ((im_row != odd) ? 1 : 0)];
        v[j] = (!im_row && odd) ? -x : x;
      }
    }
    const uint64_t out_off = panel_offset<KIND>(er0 + er, ek0 + ek, p.rows_pad);
    if constexpr (KIND == 0) {
      __align__(16) __half hi[8];
      __align__(16) __half lo[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hi[j] = __float2half_rn(v[j]);
        lo[j] = __float2half_rn((v[j] - __half2float(hi[j])) * 2048.f);
      }
      __half *ph = reinterpret_cast<__half *>(p.panel) +
                   static_cast<uint64_t>(b) * p.planes * plane_elems + out_off;
      *reinterpret_cast<uint4 *>(ph) = *reinterpret_cast<const uint4 *>(hi);
      if (p.planes == 2)
        *reinterpret_cast<uint4 *>(ph + plane_elems) = *reinterpret_cast<const uint4 *>(lo);
    } else {
      __align__(16) float hi[8];
      __align__(16) float lo[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hi[j] = to_tf32(v[j]);
        lo[j] = to_tf32(v[j] - hi[j]);
      }
      float *ph = reinterpret_cast<float *>(p.panel) +
                  static_cast<uint64_t>(b) * p.planes * plane_elems + out_off;
      reinterpret_cast<uint4 *>(ph)[0] = reinterpret_cast<const uint4 *>(hi)[0];
      reinterpret_cast<uint4 *>(ph)[1] = reinterpret_cast<const uint4 *>(hi)[1];
      if (p.planes == 2) {
        reinterpret_cast<uint4 *>(ph + plane_elems)[0] = reinterpret_cast<const uint4 *>(lo)[0];
        reinterpret_cast<uint4 *>(ph + plane_elems)[1] = reinterpret_cast<const uint4 *>(lo)[1];
      }
    }
  }
}

// ---------------------------------------------------------------- vectorised real paths
// Used when the source base address, leading dimension and batch stride are multiples of
// 16 bytes; anything else (and every complex operand) takes split_kernel above.

template <int KIND>
__device__ __forceinline__ void convert_store8(const float (&v)[8], void *panel, uint64_t off,
                                               uint64_t plane_elems, uint32_t planes) {
  if constexpr (KIND == 0) {
    __align__(16) __half hi[8];
    __align__(16) __half lo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      hi[j] = __float2half_rn(v[j]);
      lo[j] = __float2half_rn((v[j] - __half2float(hi[j])) * 2048.f);
    }
    __half *ph = reinterpret_cast<__half *>(panel) + off;
    *reinterpret_cast<uint4 *>(ph) = *reinterpret_cast<const uint4 *>(hi);
    if (planes == 2)
      *reinterpret_cast<uint4 *>(ph + plane_elems) = *reinterpret_cast<const uint4 *>(lo);
  } else {
    __align__(16) float hi[8];
    __align__(16) float lo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      hi[j] = to_tf32(v[j]);
      lo[j] = to_tf32(v[j] - hi[j]);
    }
    float *ph = reinterpret_cast<float *>(panel) + off;
    reinterpret_cast<uint4 *>(ph)[0] = reinterpret_cast<const uint4 *>(hi)[0];
    reinterpret_cast<uint4 *>(ph)[1] = reinterpret_cast<const uint4 *>(hi)[1];
    if (planes == 2) {
      reinterpret_cast<uint4 *>(ph + plane_elems)[0] = reinterpret_cast<const uint4 *>(lo)[0];
      reinterpret_cast<uint4 *>(ph + plane_elems)[1] = reinterpret_cast<const uint4 *>(lo)[1];
    }
  }
}

// float4 at p if the whole vector is inside [.., limit), element-wise with zero fill otherwise
__device__ __forceinline__ float4 load4_guarded(const float *p, uint64_t first, uint64_t limit,
                                                bool row_ok) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!row_ok) return v;
  if (first + 4 <= limit) return *reinterpret_cast<const float4 *>(p);
  if (first + 0 < limit) v.x = p[0];
  if (first + 1 < limit) v.y = p[1];
  if (first + 2 < limit) v.z = p[2];
  return v;
}

// Source is K-contiguous (element (r, kk) at [kk + r*ld]): no transpose, no shared memory.
// CTA = 128 rows x 64 k; thread = 4 rows x 8 consecutive k, all eight 16-byte loads first.
template <int KIND>
__device__ __forceinline__ void split_kcontig_body(const SplitParams &p, const uint3 bid) {
  constexpr int MY_MODE = (KIND == 0) ? CUMPSGEMM_FP16TCEC : CUMPSGEMM_TF32TCEC;
  float scale = 1.f;
  if (p.dyn != nullptr) {
    if (p.dyn->gemm_mode != MY_MODE) return;
    scale = (p.operand == 0) ? p.dyn->scale_a : p.dyn->scale_b;
  }
  const uint32_t b = bid.z;
  const float *src = p.src + static_cast<uint64_t>(b) * p.stride;
  const uint64_t k0 = static_cast<uint64_t>(bid.x) * 64 + (threadIdx.x & 7) * 8;
  const uint64_t r_base = static_cast<uint64_t>(bid.y) * 128 + (threadIdx.x >> 3);
  const uint64_t plane_elems = static_cast<uint64_t>(p.rows_pad) * p.k_pad;
  float4 x[4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint64_t r = r_base + i * 32;
    const bool row_ok = r < p.rows;
    const float *q = src + r * p.ld + k0;
    x[i][0] = load4_guarded(q, k0, p.k, row_ok);
    x[i][1] = load4_guarded(q + 4, k0 + 4, p.k, row_ok);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint64_t r = r_base + i * 32;
    if (r >= p.rows_pad) continue;
    const float v[8] = {x[i][0].x * scale, x[i][0].y * scale, x[i][0].z * scale, x[i][0].w * scale,
                        x[i][1].x * scale, x[i][1].y * scale, x[i][1].z * scale, x[i][1].w * scale};
    convert_store8<KIND>(v, p.panel,
                         static_cast<uint64_t>(b) * p.planes * plane_elems +
                             panel_offset<KIND>(r, k0, p.rows_pad),
                         plane_elems, p.planes);
  }
}

// Source is row-contiguous (element (r, kk) at [r + kk*ld]): 64 x 64 transpose through
// shared memory with 16-byte loads along r.
template <int KIND>
__device__ __forceinline__ void split_rcontig_body(const SplitParams &p, const uint3 bid,
                                                   float (*tile)[TILE + 1]) {
  constexpr int MY_MODE = (KIND == 0) ? CUMPSGEMM_FP16TCEC : CUMPSGEMM_TF32TCEC;
  float scale = 1.f;
  if (p.dyn != nullptr) {
    if (p.dyn->gemm_mode != MY_MODE) return;
    scale = (p.operand == 0) ? p.dyn->scale_a : p.dyn->scale_b;
  }
  const uint32_t b = bid.z;
  const float *src = p.src + static_cast<uint64_t>(b) * p.stride;
  const uint64_t r0 = static_cast<uint64_t>(bid.y) * TILE;
  const uint64_t k0 = static_cast<uint64_t>(bid.x) * TILE;
  const int r4 = (threadIdx.x & 15) * 4;
  const int kq = threadIdx.x >> 4; // 0..15
  float4 x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint64_t gk = k0 + kq + i * 16;
    x[i] = load4_guarded(src + gk * p.ld + r0 + r4, r0 + r4, p.rows, gk < p.k);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kk = kq + i * 16;
    tile[r4 + 0][kk] = x[i].x * scale;
    tile[r4 + 1][kk] = x[i].y * scale;
    tile[r4 + 2][kk] = x[i].z * scale;
    tile[r4 + 3][kk] = x[i].w * scale;
  }
  __syncthreads();
  const uint64_t plane_elems = static_cast<uint64_t>(p.rows_pad) * p.k_pad;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int er = (threadIdx.x >> 3) + it * 32;
    const int ek = (threadIdx.x & 7) * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = tile[er][ek + j];
    convert_store8<KIND>(v, p.panel,
                         static_cast<uint64_t>(b) * p.planes * plane_elems +
                             panel_offset<KIND>(r0 + er, k0 + ek, p.rows_pad),
                         plane_elems, p.planes);
  }
}

// Which body handles an operand.
enum SplitPath : int { kPathReal = 0, kPathComplexA = 1, kPathComplexB = 2, kPathKContig = 3, kPathRContig = 4 };

// VEC = false leaves the vectorised bodies out, which keeps the register count of the
// latency-bound generic bodies low (30 instead of 64: twice the resident blocks).
template <int KIND, bool VEC>
__device__ __forceinline__ void split_dispatch(const SplitParams &p, int path, const uint3 bid,
                                               float (*tile)[TILE + 1]) {
  if constexpr (!VEC) {
    if (path == kPathReal) split_generic_body<KIND, 0>(p, bid, tile);
    else if (path == kPathComplexA) split_generic_body<KIND, 1>(p, bid, tile);
    else split_generic_body<KIND, 2>(p, bid, tile);
    return;
  }
  // Both operands of a call are real or both complex, and complex ones never take a
  // vectorised body, so this instantiation leaves the complex bodies (and their registers) out.
  switch (path) {
  case kPathReal:
    split_generic_body<KIND, 0>(p, bid, tile);
    break;
  case kPathKContig:
    split_kcontig_body<KIND>(p, bid);
    break;
  default:
    split_rcontig_body<KIND>(p, bid, tile);
    break;
  }
}

// One launch splits both operands of a GEMM: the first blocks_a blocks work on op(A), the
// rest on op(B).  Saves a launch (and its gap) per GEMM call, which matters for small problems.
struct SplitJob {
  SplitParams p;
  int path;
  uint32_t gx, gy, gz;
};

template <int KIND, bool VEC>
__global__ void __launch_bounds__(THREADS, VEC ? 5 : 6) split_dual_kernel(const SplitJob a, const SplitJob b) {
  __shared__ float tile[TILE][TILE + 1]; // transposing staging tile shared by all paths
  // Chained behind the kernel that writes the scaling constants (AUTO / FP16TCEC_SCALING), and
  // the GEMM kernel that follows may be scheduled while this one drains: its prologue does not
  // depend on the panels, and its first panel load waits for this grid to complete.
  CUMPSGEMM_CHAINED_KERNEL_ENTRY();
  const uint32_t blocks_a = a.gx * a.gy * a.gz;
  uint32_t id = blockIdx.x;
  const SplitJob &j = (id < blocks_a) ? a : b;
  if (id >= blocks_a) id -= blocks_a;
  const uint3 bid = make_uint3(id % j.gx, (id / j.gx) % j.gy, id / (j.gx * j.gy));
  split_dispatch<KIND, VEC>(j.p, j.path, bid, tile);
}

// AUTO: the kind (FP16 or TF32 panels) is decided on the device.  Job geometry, source
// addressing and the workspace are the same for both kinds, so one launch reads the decision
// and runs the matching bodies (the reference launches the kernels of both kinds and lets the
// deselected one exit, src/cumpsgemm_kernel.cuh:478-489).
template <bool VEC>
__global__ void __launch_bounds__(THREADS, VEC ? 5 : 6)
    split_dual_auto_kernel(const SplitJob a, const SplitJob b) {
  __shared__ float tile[TILE][TILE + 1];
  CUMPSGEMM_CHAINED_KERNEL_ENTRY(); // see split_dual_kernel
  const uint32_t blocks_a = a.gx * a.gy * a.gz;
  uint32_t id = blockIdx.x;
  const SplitJob &j = (id < blocks_a) ? a : b;
  if (id >= blocks_a) id -= blocks_a;
  const uint3 bid = make_uint3(id % j.gx, (id / j.gx) % j.gy, id / (j.gx * j.gy));
  if (j.p.dyn->gemm_mode == CUMPSGEMM_TF32TCEC)
    split_dispatch<1, VEC>(j.p, j.path, bid, tile);
  else
    split_dispatch<0, VEC>(j.p, j.path, bid, tile);
}

bool make_job(const SplitArgs &a, SplitJob *job) {
  if ((a.rows_pad % TILE) != 0 || (a.k_pad % TILE) != 0) return false;
  SplitParams &p = job->p;
  p.src = reinterpret_cast<const float *>(a.src);
  p.src_array = reinterpret_cast<const float *const *>(a.src_array);
  p.ld = a.ld;
  p.stride = a.stride;
  p.rows = a.rows;
  p.k = a.k;
  p.panel = a.panel;
  p.rows_pad = a.rows_pad;
  p.k_pad = a.k_pad;
  p.planes = a.with_lo ? 2u : 1u;
  p.dyn = a.dyn;
  p.operand = static_cast<int>(a.operand);
  p.conj = a.conjugate ? 1 : 0;
  p.src_k_contig = a.src_k_contig ? 1 : 0;
  job->gx = a.k_pad / TILE;
  job->gy = a.rows_pad / TILE;
  job->gz = a.batch;
  if (a.is_complex) {
    job->path = (a.operand == Operand::A) ? kPathComplexA : kPathComplexB;
  } else {
    const bool aligned = ((reinterpret_cast<uintptr_t>(a.src) & 15u) == 0) && (a.ld % 4 == 0) &&
                         (a.stride % 4 == 0);
    if (!aligned || a.src_array != nullptr) { // per-matrix alignment is unknown on the host
      job->path = kPathReal;
    } else if (a.src_k_contig) {
      job->path = kPathKContig;
      job->gy = (a.rows_pad + 127) / 128;
    } else {
      job->path = kPathRContig;
    }
  }
  return static_cast<uint64_t>(job->gx) * job->gy * job->gz <= 0x3fffffffull;
}

} // namespace

cudaError_t launch_split_pair_auto(const SplitArgs &a, const SplitArgs &b, cudaStream_t stream) {
  if (a.dyn == nullptr || b.dyn != a.dyn) return cudaErrorInvalidValue;
  SplitJob ja, jb;
  if (!make_job(a, &ja) || !make_job(b, &jb)) return cudaErrorInvalidValue;
  const uint64_t blocks = static_cast<uint64_t>(ja.gx) * ja.gy * ja.gz +
                          static_cast<uint64_t>(jb.gx) * jb.gy * jb.gz;
  if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  const bool vec = (ja.path >= kPathKContig) || (jb.path >= kPathKContig);
  const unsigned grid = static_cast<unsigned>(blocks);
  if (vec) return launch_chained(split_dual_auto_kernel<true>, grid, THREADS, 0, stream, ja, jb);
  return launch_chained(split_dual_auto_kernel<false>, grid, THREADS, 0, stream, ja, jb);
}

cudaError_t launch_split_pair(const SplitArgs &a, const SplitArgs &b, cudaStream_t stream) {
  if (a.kind != b.kind) return cudaErrorInvalidValue;
  SplitJob ja, jb;
  if (!make_job(a, &ja) || !make_job(b, &jb)) return cudaErrorInvalidValue;
  const uint64_t blocks = static_cast<uint64_t>(ja.gx) * ja.gy * ja.gz +
                          static_cast<uint64_t>(jb.gx) * jb.gy * jb.gz;
  if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  const bool vec = (ja.path >= kPathKContig) || (jb.path >= kPathKContig);
  const unsigned grid = static_cast<unsigned>(blocks);
  if (a.kind == SplitKind::fp16) {
    if (vec) return launch_chained(split_dual_kernel<0, true>, grid, THREADS, 0, stream, ja, jb);
    return launch_chained(split_dual_kernel<0, false>, grid, THREADS, 0, stream, ja, jb);
  }
  if (vec) return launch_chained(split_dual_kernel<1, true>, grid, THREADS, 0, stream, ja, jb);
  return launch_chained(split_dual_kernel<1, false>, grid, THREADS, 0, stream, ja, jb);
}

} // namespace cumpsgemm_b200
