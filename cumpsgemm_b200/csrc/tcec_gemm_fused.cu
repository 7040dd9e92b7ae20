// Error-corrected tensor-core GEMM that splits its FP32 operands on the fly.
//
// The reference splits every FP32 value into (hi, lo) at fragment load, inside the GEMM kernel
// (src/device_tcec_wrapper.hpp:72-80 called from src/cumpsgemm_kernel.cuh:58-100), so a call
// reads A and B once and needs no workspace.  This kernel does the same for tcgen05: converter
// warps read FP32 / complex64 tiles of op(A) and op(B) straight from global memory, split them
// in registers (same arithmetic as split_kernels.cu, so both paths feed the tensor core the
// same bits) and write the FP16 hi / lo tiles into shared memory in the 128-byte-swizzled
// K-major layout a UMMA shared-memory descriptor reads.  Per stage the tensor core then forms
// the three products hi*hi, hi*lo and lo*hi; every chunk of stages the accumulators are
// drained and added to an FP32 running sum with round-to-nearest adds outside the tensor core
// (hi*hi as it is, the two corrections times 2^-11), and the alpha / beta epilogue is the one
// of tcec_gemm_pair.cu.
//
// It pays where the split pass of the two-kernel path costs as much as the GEMM: short K and
// many small problems (strided batches of a few hundred rows), where writing the panels to HBM
// and reading them back is most of the traffic.  It loses for long K on large matrices, where
// every operand element is converted once per tile that uses it (n / BN times for A, m / 128
// times for B) and the converter warps, not the tensor core, set the pace; the dispatch keeps
// the pre-split path there.  A second regime is a handful of tiles with a very long K loop:
// the launch's work items are then (tile, K slice) pairs, every slice writes plain partial
// sums, and splitk_reduce_kernel (tcec_gemm.cu) adds them in ascending order and applies alpha,
// beta and the un-scaling — the deterministic successor of the reference's atomic split-K
// kernel (src/cumpsgemm.cu:272-304) without a split pass in front.
//
// Roles (896 threads = 7 warpgroups): warps 0-3 and 12-23 = 16 converter warps (eight for the
// A tile, eight for the B tile of every stage), warps 4-11 = accumulator drain + epilogue
// (TMEM lane quarter = warp % 4), warp 24 = TMEM allocation + the single MMA-issuing thread
// (warps 25-27 idle).  Sixteen converter warps with eight 16-byte loads in flight per thread
// keep a whole stage (64 KiB) of operand data in flight per SM, which is what hides the L2 /
// HBM latency.  The kernel starts with 72 registers per thread; converters and the issuer's
// warpgroup give part of their share back (setmaxnreg.dec to 64 and 40) and the two epilogue
// warpgroups, which hold the FP32 running sum of the tile, take it (setmaxnreg.inc to 104):
// 512*64 + 128*40 + 256*104 = 64512 = the registers the CTA was launched with, so the inc can
// always be served.
// Barriers: full[s] (16 arrivals: one per converter warp, after fence.proxy.async), empty[s]
// (tcgen05.commit), d0_full[b] / d0_empty[b] for the two accumulator buffers that alternate
// per drain chunk (the epilogue warps drain one while the tensor core fills the other).  Every
// wait is bounded.  No TMA is used at all.
//
// What bounds it (cycle sums per role from a diagnostic build, 512 complex 256^3 products,
// 128 x 128 tiles): a stage takes about 3,350 cycles.  A converter warp spends 2,200-2,400 of
// them loading, converting and storing its share (about 900 are load latency, 600 the split
// arithmetic and the stores), 100 on the fence and the arrival and 1,000 waiting for the
// stage's shared memory: all sixteen warps work on the same stage, so latency and conversion
// add up instead of overlapping.  The issuing thread is busy for 800 cycles per stage (eight
// instructions, 770 cycles of tensor-core work) and waits for operands the rest of the time;
// the epilogue warps drain for 590 and store for 380.  A quarter of the tensor-core rate, which
// is why the dispatch uses this kernel only where the two-kernel path is bound by its HBM round
// trip.  Two converter teams taking the stages in turn (one team's latency under the other's
// conversion) were tried and measured slower (0.59 against 0.38 ms): three stages of 64 KiB
// are all that fit, and with two of them being converted a team always needs the stage the
// tensor core has only just received from the other team.  The two operands' warps converting
// in turns (loads issued before the wait for the turn) measured 0.66 ms: a warp's conversion is
// bound by its own instruction latency, not by issue slots, so taking turns only serialises it.
//
// Operand layouts the converters understand (anything else takes the pre-split path):
//   kcontig  element (r, kk) of the real operand at src[r * ld + kk]      (A with op T, B with
//            op N; complex B with op N is this with doubled ld and K: row j of B' is the
//            interleaved (re, im) column j of B)
//   rcontig  element (r, kk) at src[kk * ld + r]                          (A with op N, B with op T)
//   cplx_a   complex A with op N: a(i, l) at src[2 * (i + l * ld)], expanded on the fly to
//            rows (2i, 2i+1) x columns (2l, 2l+1) = [[re, -im], [im, re]]
// All need 16-byte aligned bases, leading dimensions and batch strides.
#include "gemm_common.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>
#include <mutex>

namespace cumpsgemm_b200 {
namespace {

constexpr int BM = 128;
constexpr int ROW_BYTES = kGemmRowBytes; // 64 FP16 k values per stage and row
constexpr int KS = ROW_BYTES / 2;        // k values per stage
constexpr int NUM_THREADS = 896;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_CVT_WARPS = 16; // 8 per operand
constexpr int CVT_PER_OPERAND = 8;
constexpr int FIRST_EPI_WARP = 4; // warps 4..11
constexpr int MMA_WARP = 24;
constexpr int LAUNCH_REGS = 72;
constexpr int REGS_CVT = 64, REGS_MMA = 40, REGS_EPI = 104;
static_assert(512 * REGS_CVT + 128 * REGS_MMA + 256 * REGS_EPI <= NUM_THREADS * LAUNCH_REGS,
              "register re-allocation must fit what the CTA was launched with");
constexpr int STAGES = 3;
constexpr uint32_t PREFETCH_STAGES = 2; // how far ahead of their use operand lines are pulled into L2

enum OperandLayout : int { kLayoutKContig = 0, kLayoutRContig = 1, kLayoutCplxA = 2 };

struct FusedOperand {
  const float *src;
  uint64_t ld;     // floats (complex: floats of one column = 2 * ld)
  uint64_t stride; // floats between batch entries
  uint32_t rows;   // rows of the real (expanded) operand
  int layout;
};

struct FusedParams {
  FusedOperand a, b;
  uint32_t k;      // K of the real (expanded) problem
  // Diagnostic builds only (-DCUMPSGEMM_FUSED_DIAG_BUILD, never the library): bit 0 = the
  // converters use constants instead of loading the operands, bit 1 = they skip the split
  // arithmetic and the stores (environment variable CUMPSGEMM_FUSED_DIAG).  Results are then
  // meaningless; the time that remains separates load latency, conversion work and the rest of
  // the pipeline.  In the library the switches are the constant 0 and compile away.
  int diag;
};
// Every kernel parameter stays at or under 128 bytes: a larger struct is read through a pointer
// (see GemmKernelParams), which is why the operands and the output side travel separately.
static_assert(sizeof(FusedParams) <= 128, "kernel parameter structs stay within 128 bytes");

template <int BN> struct FusedCfg {
  static constexpr int A_TILE = BM * ROW_BYTES;
  static constexpr int B_TILE = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = 2 * (A_TILE + B_TILE);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  // two accumulator buffers, alternating per drain chunk, of 2 * BN columns each:
  // [hi*hi | hi*lo + lo*hi]
  static constexpr uint32_t TMEM_COLS = 4u * BN;
};

// Byte offset of (row r, 16-byte chunk c) inside a K-major tile with 128-byte rows and the
// 128-byte swizzle: 8-row groups of 1 KiB, chunk index XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) {
  return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4);
}

// hi = RN_fp16(v), lo = RN_fp16((v - hi) * 2^11) for two values, packed (v0 in the low half)
__device__ __forceinline__ void split2(float v0, float v1, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(v0, v1);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn((v0 - hf.x) * 2048.f, (v1 - hf.y) * 2048.f);
  hi = *reinterpret_cast<const uint32_t *>(&h);
  lo = *reinterpret_cast<const uint32_t *>(&l);
}

__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z,
                                             uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z),
               "r"(w)
               : "memory");
}
// generic-proxy writes to shared memory become visible to the async proxy (the tensor core)
__device__ __forceinline__ void fence_proxy_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 4 floats at p, zero filled outside [.., limit) / when !ok
__device__ __forceinline__ float4 ld4(const float *p, uint64_t first, uint64_t limit, bool ok) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!ok || first >= limit) return v;
  if (first + 4 <= limit) return __ldg(reinterpret_cast<const float4 *>(p));
  v.x = __ldg(p);
  if (first + 1 < limit) v.y = __ldg(p + 1);
  if (first + 2 < limit) v.z = __ldg(p + 2);
  return v;
}

// ---------------------------------------------------------------- converters
// One stage of one operand: ROWS x 64 real k values starting at (row0, k0), written as hi / lo
// tiles at shared addresses hi_base / lo_base by the eight converter warps of the operand
// (cw = 0..7).  Every body issues all of a thread's loads (up to eight float4) before the
// first conversion, reads whole 128-byte lines per warp instruction, and stores without
// shared-memory bank conflicts.

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(x), "r"(y) : "memory");
}

// K-contiguous source.  One warp instruction covers 2 rows x 64 k: lanes 0-15 read the 256
// contiguous bytes of one row, lanes 16-31 those of the next.  A lane's four values are half
// of a 16-byte chunk; the 16 lanes of a row store one whole 128-byte row (all banks once).
template <int ROWS>
__device__ __forceinline__ void convert_kcontig(const FusedOperand &o, const float *src,
                                                uint32_t row0, uint32_t k0, uint32_t kmax,
                                                float scale, uint32_t hi_base, uint32_t lo_base,
                                                int cw, int lane, bool prefetch) {
  constexpr int STEPS = ROWS / (2 * CVT_PER_OPERAND);
  const uint32_t q = lane & 15, half = lane >> 4;
  const uint32_t kk = k0 + 4 * q;
  float4 x[STEPS];
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const uint32_t r = (cw * STEPS + s) * 2 + half;
    const uint64_t gr = static_cast<uint64_t>(row0) + r;
    const float *p = src + gr * o.ld + kk;
    const bool ok = gr < o.rows;
    x[s] = ld4(p, kk, kmax, ok);
    if (prefetch && ok && (q & 7) == 0 && kk + PREFETCH_STAGES * KS < kmax)
      ptx::prefetch_l2(p + PREFETCH_STAGES * KS);
  }
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const uint32_t r = (cw * STEPS + s) * 2 + half;
    uint32_t h0, l0, h1, l1;
    split2(x[s].x * scale, x[s].y * scale, h0, l0);
    split2(x[s].z * scale, x[s].w * scale, h1, l1);
    const uint32_t off = swz(r, q >> 1) + (q & 1) * 8;
    st_shared_v2(hi_base + off, h0, h1);
    st_shared_v2(lo_base + off, l0, l1);
  }
}

// Row-contiguous source (needs a transpose).  A warp owns 32 rows x 32 k: lane = gq*8 + cq*2 + h
// with gq = 8-row group, h = which half of the group (rows 4h .. 4h+3), cq = one of the four
// 16-byte chunks.  For each of the chunk's eight k values the lane loads a float4 along the
// rows: per instruction the lanes (gq, h) read the 128 contiguous bytes of 32 rows, for four
// columns.  The lane then owns four rows x one whole chunk and stores four 16-byte vectors
// per plane; within a quarter warp (h, cq vary) the chunk position (4*chi + cq) ^ (4h + j)
// takes eight different values, so the stores are conflict free.
template <int ROWS>
__device__ __forceinline__ void convert_rcontig(const FusedOperand &o, const float *src,
                                                uint32_t row0, uint32_t k0, uint32_t kmax,
                                                float scale, uint32_t hi_base, uint32_t lo_base,
                                                int cw, int lane, bool prefetch) {
  constexpr int JOBS = (ROWS / 32) * 2; // 32-row blocks x two 32-k halves
  const uint32_t h = lane & 1, cq = (lane >> 1) & 3, gq = lane >> 3;
#pragma unroll 1
  for (int job = cw; job < JOBS; job += CVT_PER_OPERAND) {
    const uint32_t blk = job >> 1, chi = job & 1;
    const uint32_t chunk = 4 * chi + cq;
    const uint32_t kk = k0 + 8 * chunk;
    const uint32_t r = blk * 32 + gq * 8 + 4 * h;
    const uint64_t gr = static_cast<uint64_t>(row0) + r;
    const float *p = src + static_cast<uint64_t>(kk) * o.ld + gr;
    float4 x[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = ld4(p + e * o.ld, gr, o.rows, kk + e < kmax);
    if (prefetch && (lane & 0x19) == 0) { // gq == 0, h == 0: one lane per column
      if (gr < o.rows) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (kk + e + PREFETCH_STAGES * KS < kmax)
            ptx::prefetch_l2(p + static_cast<uint64_t>(e + PREFETCH_STAGES * KS) * o.ld);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        v[e] = (j == 0 ? x[e].x : j == 1 ? x[e].y : j == 2 ? x[e].z : x[e].w) * scale;
      uint32_t hh[4], ll[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) split2(v[2 * t], v[2 * t + 1], hh[t], ll[t]);
      const uint32_t off = swz(r + j, chunk);
      st_shared_v4(hi_base + off, hh[0], hh[1], hh[2], hh[3]);
      st_shared_v4(lo_base + off, ll[0], ll[1], ll[2], ll[3]);
    }
  }
}

// Complex A with op N, expanded to [[re, -im], [im, re]].  Same lane layout as rcontig; a
// float4 holds two complex rows (re0, im0, re1, im1) of one complex k, i.e. the real k pair
// (2l, 2l+1) of four real rows, so four loads fill the lane's chunk.
template <int ROWS>
__device__ __forceinline__ void convert_cplx_a(const FusedOperand &o, const float *src,
                                               uint32_t row0, uint32_t k0, uint32_t kmax,
                                               float scale, uint32_t hi_base, uint32_t lo_base,
                                               int cw, int lane, bool prefetch) {
  constexpr int JOBS = (ROWS / 32) * 2;
  const uint32_t h = lane & 1, cq = (lane >> 1) & 3, gq = lane >> 3;
#pragma unroll 1
  for (int job = cw; job < JOBS; job += CVT_PER_OPERAND) {
    const uint32_t blk = job >> 1, chi = job & 1;
    const uint32_t chunk = 4 * chi + cq;
    const uint32_t kk = k0 + 8 * chunk; // real k of the chunk's first value (multiple of 8)
    const uint32_t r = blk * 32 + gq * 8 + 4 * h;
    const uint64_t gr = static_cast<uint64_t>(row0) + r;
    // complex element (i, l) = floats 2i, 2i+1 of column l; o.ld = floats per column
    const float *p = src + static_cast<uint64_t>(kk >> 1) * o.ld + gr;
    float4 x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = ld4(p + e * o.ld, gr, o.rows, kk + 2 * e < kmax);
    if (prefetch && (lane & 0x19) == 0 && gr < o.rows) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (kk + 2 * e + PREFETCH_STAGES * KS < kmax)
          ptx::prefetch_l2(p + static_cast<uint64_t>(e + PREFETCH_STAGES * KS / 2) * o.ld);
    }
    uint32_t hh[4][4], ll[4][4]; // [row j][k pair e]
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float re0 = x[e].x * scale, im0 = x[e].y * scale;
      const float re1 = x[e].z * scale, im1 = x[e].w * scale;
      split2(re0, -im0, hh[0][e], ll[0][e]); // row 2i   : (re, -im)
      split2(im0, re0, hh[1][e], ll[1][e]);  // row 2i+1 : (im,  re)
      split2(re1, -im1, hh[2][e], ll[2][e]);
      split2(im1, re1, hh[3][e], ll[3][e]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t off = swz(r + j, chunk);
      st_shared_v4(hi_base + off, hh[j][0], hh[j][1], hh[j][2], hh[j][3]);
      st_shared_v4(lo_base + off, ll[j][0], ll[j][1], ll[j][2], ll[j][3]);
    }
  }
}

// ---- fast bodies for stages that lie completely inside the operand (no bounds tests).  The
// shared-memory offsets of a lane do not depend on the stage, so they are computed once per
// kernel (LanePlan) and a stage costs the loads, the split arithmetic and the stores.
struct LanePlan {
  uint32_t st_off;   // lane-constant part of the store offset inside a hi / lo tile
  uint32_t x[4];     // per-step term: swizzled chunk position (and row offset) of the step
  uint32_t g_row;    // first tile row this lane reads (row-contiguous) / its row (K-contiguous)
  uint32_t g_k;      // first k of the stage this lane reads
  bool active;       // this warp has a job for this operand
};

template <int ROWS> __device__ __forceinline__ LanePlan make_plan(int layout, int cw, int lane) {
  LanePlan pl;
  if (layout == kLayoutKContig) {
    const uint32_t q = lane & 15, half = lane >> 4;
    const uint32_t r0 = cw * (ROWS / CVT_PER_OPERAND); // multiple of 8
    const uint32_t u = (q >> 1) ^ half;
    pl.st_off = (r0 >> 3) * 1024u + half * 128u + (q & 1u) * 8u;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) pl.x[i] = (u ^ (2u * i)) << 4;
    pl.g_row = r0 + half;
    pl.g_k = 4 * q;
    pl.active = true;
  } else {
    const uint32_t h = lane & 1, cq = (lane >> 1) & 3, gq = lane >> 3;
    const uint32_t blk = cw >> 1, chi = cw & 1;
    const uint32_t chunk = 4 * chi + cq;
    pl.st_off = (blk * 4 + gq) * 1024u + 4u * h * 128u;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) pl.x[j] = j * 128u + (((chunk ^ (4u * h)) ^ j) << 4);
    pl.g_row = blk * 32 + gq * 8 + 4 * h;
    pl.g_k = 8 * chunk;
    pl.active = static_cast<uint32_t>(cw) < (ROWS / 32) * 2;
  }
  return pl;
}

// K-contiguous: p = the lane's address for step 0; consecutive steps are two rows apart.
template <int ROWS, bool SCALED>
__device__ __forceinline__ void fast_kcontig(const float *p, uint64_t two_rows, float scale,
                                             uint32_t hi_addr, uint32_t lo_delta,
                                             const LanePlan &pl, int diag = 0) {
  constexpr int STEPS = ROWS / (2 * CVT_PER_OPERAND);
  float4 x[STEPS];
  if (diag & 1) {
#pragma unroll
    for (int s = 0; s < STEPS; ++s) x[s] = make_float4(scale, 0.5f, 0.25f, 0.125f);
  } else {
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      x[s] = __ldg(reinterpret_cast<const float4 *>(p));
      p += two_rows;
    }
  }
  if (diag & 2) {
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < STEPS; ++s) acc += x[s].x + x[s].y + x[s].z + x[s].w;
    if (acc == 123.456f) st_shared_u32(hi_addr, __float_as_uint(acc));
    return;
  }
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const uint32_t c_s = static_cast<uint32_t>(s >> 2) * 1024u + static_cast<uint32_t>((2 * s) & 7) * 128u;
    float a = x[s].x, b = x[s].y, c = x[s].z, d = x[s].w;
    if (SCALED) {
      a *= scale;
      b *= scale;
      c *= scale;
      d *= scale;
    }
    uint32_t h0, l0, h1, l1;
    split2(a, b, h0, l0);
    split2(c, d, h1, l1);
    const uint32_t addr = hi_addr + pl.x[s & 3] + c_s;
    st_shared_v2(addr, h0, h1);
    st_shared_v2(addr + lo_delta, l0, l1);
  }
}

// Row-contiguous: p = the lane's address for the first k of its chunk; consecutive k values are
// one column (ld floats) apart.
template <bool SCALED>
__device__ __forceinline__ void fast_rcontig(const float *p, uint64_t ld, float scale,
                                             uint32_t hi_addr, uint32_t lo_delta,
                                             const LanePlan &pl) {
  float4 x[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    x[e] = __ldg(reinterpret_cast<const float4 *>(p));
    p += ld;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] = (j == 0 ? x[e].x : j == 1 ? x[e].y : j == 2 ? x[e].z : x[e].w);
      if (SCALED) v[e] *= scale;
    }
    uint32_t hh[4], ll[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) split2(v[2 * t], v[2 * t + 1], hh[t], ll[t]);
    const uint32_t addr = hi_addr + pl.x[j];
    st_shared_v4(addr, hh[0], hh[1], hh[2], hh[3]);
    st_shared_v4(addr + lo_delta, ll[0], ll[1], ll[2], ll[3]);
  }
}

// Complex A, op N: p = the lane's address for the first complex k of its chunk.
template <bool SCALED>
__device__ __forceinline__ void fast_cplx_a(const float *p, uint64_t ld, float scale,
                                            uint32_t hi_addr, uint32_t lo_delta,
                                            const LanePlan &pl, int diag = 0) {
  float4 x[4];
  if (diag & 1) {
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = make_float4(scale, 0.5f, 0.25f, 0.125f);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[e] = __ldg(reinterpret_cast<const float4 *>(p));
      p += ld;
    }
  }
  if (diag & 2) {
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc += x[e].x + x[e].y + x[e].z + x[e].w;
    if (acc == 123.456f) st_shared_u32(hi_addr, __float_as_uint(acc));
    return;
  }
  uint32_t hh[4][4], ll[4][4]; // [row j][k pair e]
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float re0 = x[e].x, im0 = x[e].y, re1 = x[e].z, im1 = x[e].w;
    if (SCALED) {
      re0 *= scale;
      im0 *= scale;
      re1 *= scale;
      im1 *= scale;
    }
    split2(re0, -im0, hh[0][e], ll[0][e]);
    split2(im0, re0, hh[1][e], ll[1][e]);
    split2(re1, -im1, hh[2][e], ll[2][e]);
    split2(im1, re1, hh[3][e], ll[3][e]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t addr = hi_addr + pl.x[j];
    st_shared_v4(addr, hh[j][0], hh[j][1], hh[j][2], hh[j][3]);
    st_shared_v4(addr + lo_delta, ll[j][0], ll[j][1], ll[j][2], ll[j][3]);
  }
}

template <int ROWS>
__device__ __forceinline__ void convert_operand(const FusedOperand &o, const float *src,
                                                uint32_t row0, uint32_t k0, uint32_t kmax,
                                                float scale, uint32_t hi_base, uint32_t lo_base,
                                                int cw, int lane, bool prefetch) {
  if (o.layout == kLayoutKContig)
    convert_kcontig<ROWS>(o, src, row0, k0, kmax, scale, hi_base, lo_base, cw, lane, prefetch);
  else if (o.layout == kLayoutRContig)
    convert_rcontig<ROWS>(o, src, row0, k0, kmax, scale, hi_base, lo_base, cw, lane, prefetch);
  else
    convert_cplx_a<ROWS>(o, src, row0, k0, kmax, scale, hi_base, lo_base, cw, lane, prefetch);
}

// Hints the operand tile (rows row0 .. row0 + rows_tile of the real operand, all of K) of one
// batch entry into L2, one prefetch per 128-byte line, lines dealt out over `nthreads` threads.
// Only addresses inside the operand are named.
__device__ __forceinline__ void prefetch_operand_tile(const FusedOperand &o, uint32_t batch,
                                                      uint32_t row0, uint32_t rows_tile,
                                                      uint32_t k, uint32_t t, uint32_t nthreads) {
  if (row0 >= o.rows) return;
  const uint32_t rows = (o.rows - row0 < rows_tile) ? o.rows - row0 : rows_tile;
  const float *base = o.src + static_cast<uint64_t>(batch) * o.stride;
  uint32_t nseg, seg_len; // segments of seg_len contiguous floats, o.ld floats apart
  if (o.layout == kLayoutKContig) {
    nseg = rows;
    seg_len = k;
    base += static_cast<uint64_t>(row0) * o.ld;
  } else {
    nseg = (o.layout == kLayoutRContig) ? k : (k >> 1);
    seg_len = rows;
    base += row0;
  }
  const uint32_t lps = (seg_len + 31u) >> 5; // 128-byte steps per segment
  const uint32_t total = nseg * lps;
  for (uint32_t i = t; i < total; i += nthreads) {
    const uint32_t seg = i / lps, j = i - seg * lps;
    ptx::prefetch_l2(base + static_cast<uint64_t>(seg) * o.ld + (j << 5));
  }
}

struct TileCoord {
  uint32_t batch;
  uint32_t m0, n0;
};

template <int BN>
__device__ __forceinline__ TileCoord tile_coord(uint32_t tile, const GemmKernelParams &p) {
  constexpr uint32_t GROUP_M = 8;
  const uint32_t tiles_per_batch = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.batch = tile / tiles_per_batch;
  const uint32_t t = tile - c.batch * tiles_per_batch;
  const uint32_t tiles_in_group = GROUP_M * p.tiles_n;
  const uint32_t group_id = t / tiles_in_group;
  const uint32_t first_m = group_id * GROUP_M;
  const uint32_t group_rows = min(p.tiles_m - first_m, GROUP_M);
  const uint32_t in_group = t - group_id * tiles_in_group;
  c.m0 = (first_m + in_group % group_rows) * BM;
  c.n0 = (in_group / group_rows) * BN;
  return c;
}

// Work item w of a launch: tile w with its whole K loop, or, with split-K, slice w % k_slices
// (stages [kb0, kb0 + kbn) of the K loop) of tile w / k_slices.
struct WorkItem {
  uint32_t tile, kb0, kbn, slice;
};
__device__ __forceinline__ WorkItem work_item(uint32_t w, const GemmKernelParams &p) {
  WorkItem x;
  if (p.k_slices <= 1) {
    x.tile = w;
    x.kb0 = 0;
    x.kbn = p.k_blocks;
    x.slice = 0;
  } else {
    x.tile = w / p.k_slices;
    x.slice = w - x.tile * p.k_slices;
    x.kb0 = x.slice * p.slice_blocks;
    x.kbn = min(p.slice_blocks, p.k_blocks - x.kb0);
  }
  return x;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1) tcec_gemm_fused_kernel(const FusedParams fp,
                                                                         const GemmKernelParams p) {
  using Cfg = FusedCfg<BN>;
  constexpr int K_STEPS = ROW_BYTES / 32;
  constexpr uint32_t IDESC = ptx::make_idesc(0, BM, BN);
  constexpr int CPT = BN / 2;
#ifdef CUMPSGEMM_FUSED_DIAG_BUILD
  const int kdiag = fp.diag;
#else
  constexpr int kdiag = 0;
#endif

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *d0_full = bars + 2 * STAGES;      // [2]
  uint64_t *d0_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t *tmem_base_ptr = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_ptr + 1);
  // tiles the issuing thread has started (read by the prefetching warps)
  volatile uint32_t *tiles_started = reinterpret_cast<volatile uint32_t *>(tmem_base_ptr + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t total_tiles = p.total_tiles;
  const uint32_t total_work = total_tiles * p.k_slices; // work items of the launch

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), NUM_CVT_WARPS);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&d0_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&d0_empty[b]), NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    *tiles_started = 0;
    ptx::mbar_init_fence();
  }
  if (warp == MMA_WARP) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_base_ptr), Cfg::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  const uint32_t k_blocks = p.k_blocks;

  const bool is_epilogue = warp >= FIRST_EPI_WARP && warp < FIRST_EPI_WARP + NUM_EPI_WARPS;
  if (warp >= MMA_WARP) {
    // ================================================================ MMA issuer
    ptx::setmaxnreg_dec<REGS_MMA>();
    if (warp == MMA_WARP && lane == 0) {
      bool ok = true;
      const uint32_t chunk = p.drain_chunk;
      const uint32_t first = p.first_chunk;
      // The issuing thread is one dependent instruction stream, and with 768 tensor-core
      // cycles per stage its own instruction count is on the critical path: stage index,
      // phase bits and chunk boundaries are kept as running counters (no division), and the
      // four operand descriptors of a stage are one base plus a per-stage constant.
      // chunk_idx counts drain chunks over the whole launch: chunk c accumulates in buffer
      // c & 1, so the epilogue warps drain one buffer while the tensor core fills the other.
      const uint64_t desc0 = ptx::make_kmajor_desc<ROW_BYTES>(ptx::smem_u32(smem));
      constexpr uint64_t kStageDesc = Cfg::STAGE_BYTES >> 4;
      constexpr uint64_t kALo = Cfg::A_TILE >> 4, kBHi = (2 * Cfg::A_TILE) >> 4;
      constexpr uint32_t IDESC2 = ptx::make_idesc(0, BM, 2 * BN);
      uint32_t s = 0, ph = 0, chunk_idx = 0;
      uint32_t started = 0;
      for (uint32_t w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        *tiles_started = ++started;
        const uint32_t k_blocks = work_item(w, p).kbn; // stages of this work item
        uint32_t chunk_end = 0; // first stage after the current chunk
        for (uint32_t kb = 0; kb < k_blocks; ++kb) {
          const bool first_in_chunk = (kb == chunk_end);
          if (first_in_chunk) {
            chunk_end = kb + (kb == 0 ? first : chunk);
            if (chunk_end > k_blocks) chunk_end = k_blocks;
          }
          const bool last_in_chunk = (kb + 1 == chunk_end);
          const uint32_t b0 = chunk_idx & 1u;
          const uint32_t acc_hh = tmem_base + b0 * (2 * BN); // [hi*hi | corrections]
          ok = ptx::mbar_wait_poll(ptx::smem_u32(&full_bar[s]), ph, abort_flag, p.status,
                                   ptx::kErrWaitFull);
          if (!ok) break;
          if (first_in_chunk) {
            // this buffer's previous content (two chunks ago) must have been drained
            ok = ptx::mbar_wait_poll(ptx::smem_u32(&d0_empty[b0]), ((chunk_idx >> 1) & 1u) ^ 1u,
                                     abort_flag, p.status, ptx::kErrWaitD0Empty);
            if (!ok) break;
          }
          ptx::tc_fence_after();
          const uint64_t a_hi = desc0 + s * kStageDesc;
          const uint64_t a_lo = a_hi + kALo, b_hi = a_hi + kBHi;
          // Issuing one tcgen05.mma costs the issuing thread about 120 cycles whatever its
          // size, which is more than a 128 x 128 x 16 product takes to execute.  The B_hi and
          // B_lo tiles of a stage are adjacent in shared memory, so A_hi x [B_hi; B_lo] is ONE
          // instruction of twice the width that yields hi*hi (columns 0..BN) and hi*lo
          // (columns BN..2BN); lo*hi is added onto the second half.  Eight instructions per
          // stage instead of twelve, and all three products of a chunk leave TMEM together.
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks) {
            ptx::mma_f16_ss(acc_hh, a_hi + 2 * ks, b_hi + 2 * ks, IDESC2,
                            (!first_in_chunk || ks > 0) ? 1u : 0u);
            ptx::mma_f16_ss(acc_hh + BN, a_lo + 2 * ks, b_hi + 2 * ks, IDESC, 1u);
          }
          if (last_in_chunk) ptx::tc_commit(ptx::smem_u32(&d0_full[b0]));
          ptx::tc_commit(ptx::smem_u32(&empty_bar[s]));
          if (last_in_chunk) ++chunk_idx;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    } else if (warp > MMA_WARP) {
      // The other three warps of the issuer's warpgroup pull the operand tiles of the CTA's
      // NEXT tile into L2 while the current one is computed, so that the converters' loads find
      // them there (a converter has one stage in flight and cannot look further ahead itself).
      // They follow the issuing thread's tile count; a hint engine only: if it falls behind or
      // gives up, nothing depends on it.
      const uint32_t t = threadIdx.x - (MMA_WARP + 1) * 32;
      constexpr uint32_t PF_THREADS = (NUM_THREADS / 32 - MMA_WARP - 1) * 32;
      uint32_t it = 0;
      // (not with split-K: a work item then reads one K slice of its tile only)
      for (uint32_t tile = blockIdx.x; tile < total_tiles && p.k_slices <= 1; tile += gridDim.x) {
        ++it;
        uint32_t polls = 0;
        while (*tiles_started < it && !*abort_flag && ++polls < (1u << 22)) __nanosleep(256);
        if (*tiles_started < it) break;
        const uint32_t next = tile + gridDim.x;
        if (next >= total_tiles) break;
        const TileCoord tn = tile_coord<BN>(next, p);
        prefetch_operand_tile(fp.a, tn.batch, tn.m0, BM, fp.k, t, PF_THREADS);
        prefetch_operand_tile(fp.b, tn.batch, tn.n0, BN, fp.k, t, PF_THREADS);
      }
    }
  } else if (!is_epilogue) {
    // ================================================================ converters
    ptx::setmaxnreg_dec<REGS_CVT>();
    const int ci = (warp < FIRST_EPI_WARP) ? warp : warp - NUM_EPI_WARPS; // 0..15
    const bool for_a = ci < CVT_PER_OPERAND;
    const int cw = ci & (CVT_PER_OPERAND - 1);
    const FusedOperand o = for_a ? fp.a : fp.b;
    float scale = 1.f;
    if (p.dyn != nullptr) scale = for_a ? p.dyn->scale_a : p.dyn->scale_b;
    const bool scaled = scale != 1.f;
    const uint32_t rows_tile = for_a ? BM : BN;
    const LanePlan pl = for_a ? make_plan<BM>(o.layout, cw, lane) : make_plan<BN>(o.layout, cw, lane);
    // offsets of this operand's hi tile inside a stage, and from hi to lo
    const uint32_t tile_off = for_a ? 0u : 2u * Cfg::A_TILE;
    const uint32_t lo_delta = for_a ? Cfg::A_TILE : Cfg::B_TILE;
    // floats from one stage to the next for this lane's loads
    const uint64_t stage_step = (o.layout == kLayoutKContig) ? KS
                                : (o.layout == kLayoutRContig) ? KS * o.ld
                                                               : (KS / 2) * o.ld;
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (uint32_t w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const WorkItem wi = work_item(w, p);
      const uint32_t k_blocks = wi.kbn;
      const TileCoord tc = tile_coord<BN>(wi.tile, p);
      const uint32_t row0 = for_a ? tc.m0 : tc.n0;
      const float *src = o.src + static_cast<uint64_t>(tc.batch) * o.stride;
      const bool rows_inside = row0 + rows_tile <= o.rows;
      // the lane's address in stage 0 (fast bodies)
      const float *lp;
      if (o.layout == kLayoutKContig)
        lp = src + (static_cast<uint64_t>(row0) + pl.g_row) * o.ld + pl.g_k;
      else if (o.layout == kLayoutRContig)
        lp = src + static_cast<uint64_t>(pl.g_k) * o.ld + row0 + pl.g_row;
      else
        lp = src + static_cast<uint64_t>(pl.g_k >> 1) * o.ld + row0 + pl.g_row;
      lp += static_cast<uint64_t>(wi.kb0) * stage_step;
      for (uint32_t kb = 0; kb < k_blocks; ++kb, lp += stage_step) {
        if (lane == 0)
          ok = ptx::mbar_wait_poll(ptx::smem_u32(&empty_bar[s]), ph ^ 1u, abort_flag, p.status,
                                   ptx::kErrWaitEmpty);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        const uint32_t hi_tile = ptx::smem_u32(smem + s * Cfg::STAGE_BYTES) + tile_off;
        const uint32_t k0 = (wi.kb0 + kb) * KS;
        if (rows_inside && k0 + KS <= fp.k) {
          const uint32_t hi_addr = hi_tile + pl.st_off;
          if (o.layout == kLayoutKContig) {
            if (for_a) {
              if (scaled) fast_kcontig<BM, true>(lp, 2 * o.ld, scale, hi_addr, lo_delta, pl, kdiag);
              else fast_kcontig<BM, false>(lp, 2 * o.ld, scale, hi_addr, lo_delta, pl, kdiag);
            } else {
              if (scaled) fast_kcontig<BN, true>(lp, 2 * o.ld, scale, hi_addr, lo_delta, pl, kdiag);
              else fast_kcontig<BN, false>(lp, 2 * o.ld, scale, hi_addr, lo_delta, pl, kdiag);
            }
          } else if (pl.active) {
            if (o.layout == kLayoutRContig) {
              if (scaled) fast_rcontig<true>(lp, o.ld, scale, hi_addr, lo_delta, pl);
              else fast_rcontig<false>(lp, o.ld, scale, hi_addr, lo_delta, pl);
            } else {
              if (scaled) fast_cplx_a<true>(lp, o.ld, scale, hi_addr, lo_delta, pl, kdiag);
              else fast_cplx_a<false>(lp, o.ld, scale, hi_addr, lo_delta, pl, kdiag);
            }
          }
        } else if (for_a) {
          convert_operand<BM>(o, src, row0, k0, fp.k, scale, hi_tile, hi_tile + lo_delta, cw, lane,
                              false);
        } else {
          convert_operand<BN>(o, src, row0, k0, fp.k, scale, hi_tile, hi_tile + lo_delta, cw, lane,
                              false);
        }
        fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&full_bar[s]));
        if (++s == STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else {
    // ================================================================ drain + epilogue
    ptx::setmaxnreg_inc<REGS_EPI>();
    const uint32_t quarter = static_cast<uint32_t>(warp & 3);
    const uint32_t half = static_cast<uint32_t>((warp - FIRST_EPI_WARP) >> 2);
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const uint32_t col_base = half * CPT;
    // with split-K the un-scaling belongs to the reduction kernel, like alpha and beta
    const float unscale = (p.dyn != nullptr && p.k_slices <= 1) ? p.dyn->unscale_c : 1.f;
    const float ar = p.alpha_r * unscale, ai = p.alpha_i * unscale;
    const float br = p.beta_r, bi = p.beta_i;
    const bool read_c = (br != 0.f) || (bi != 0.f);
    const float sgn = (lane & 1) ? 1.f : -1.f; // odd rows hold imaginary parts
    const float lsi = p.lo_scale_inv;

    uint32_t chunk_idx = 0;
    bool ok = true;
    for (uint32_t w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const WorkItem wi = work_item(w, p);
      const uint32_t n_chunks =
          1u + ((wi.kbn > p.first_chunk)
                    ? (wi.kbn - p.first_chunk + p.drain_chunk - 1) / p.drain_chunk
                    : 0u);
      const TileCoord tc = tile_coord<BN>(wi.tile, p);
      float acc[CPT];
#pragma unroll
      for (int i = 0; i < CPT; ++i) acc[i] = 0.f;
      const uint32_t row = tc.m0 + quarter * 32u + static_cast<uint32_t>(lane);
      const bool row_ok = row < p.m;
      // (split-K: p.c is the scratch for partial sums, one block of all tiles per slice)
      float *cbase = p.c + static_cast<uint64_t>(wi.slice) * p.slice_stride +
                     static_cast<uint64_t>(tc.batch) * p.stride_c + row;

      for (uint32_t c = 0; c < n_chunks; ++c, ++chunk_idx) {
        const uint32_t b0 = chunk_idx & 1u;
        ok = ptx::mbar_wait_backoff(ptx::smem_u32(&d0_full[b0]), (chunk_idx >> 1) & 1u, abort_flag,
                                    p.status, ptx::kErrWaitD0Full, 64);
        if (!ok) break;
        ptx::tc_fence_after();
        // running sum += hi*hi + (hi*lo + lo*hi) * 2^-11, both FP32 round-to-nearest adds
        // outside the tensor core
        const uint32_t t_hh = tmem_base + b0 * (2 * BN) + lane_addr + col_base;
#pragma unroll
        for (int pc = 0; pc < CPT / 16; ++pc) {
          uint32_t v[16], w[16];
          ptx::tmem_ld_32x32b_x16(t_hh + pc * 16, v);
          ptx::tmem_ld_32x32b_x16(t_hh + BN + pc * 16, w);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            acc[pc * 16 + i] =
                fmaf(__uint_as_float(w[i]), lsi, acc[pc * 16 + i] + __uint_as_float(v[i]));
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&d0_empty[b0]));
      }
      if (!ok) break;

      // C(row, col) = alpha * acc + beta * C(row, col)
      float *cp = cbase + static_cast<uint64_t>(tc.n0 + col_base) * p.ldc;
      const bool plain = (ai == 0.f) && !read_c; // real scalar, C not read
      if (plain && row_ok && tc.n0 + col_base + CPT <= p.n) {
        // the common case, kept as short as possible: the epilogue warps are the slowest
        // role of a short-K tile
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          __stcs(cp, ar * acc[i]);
          cp += p.ldc;
        }
        continue;
      }
      // general case; loads of a group of columns are all issued before its first store
      // (see tcec_gemm_pair.cu)
      constexpr int EPI_BATCH = 8;
#pragma unroll
      for (int i0 = 0; i0 < CPT; i0 += EPI_BATCH) {
        float old[EPI_BATCH];
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const uint32_t col = tc.n0 + col_base + static_cast<uint32_t>(i0 + j);
          old[j] = (read_c && row_ok && col < p.n)
                       ? __ldcs(cbase + static_cast<uint64_t>(col) * p.ldc)
                       : 0.f;
        }
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const int i = i0 + j;
          const uint32_t col = tc.n0 + col_base + static_cast<uint32_t>(i);
          if (col < p.n) { // uniform over the warp
            float out;
            if (p.is_complex) {
              const float acc_o = __shfl_xor_sync(0xffffffffu, acc[i], 1);
              const float old_o = __shfl_xor_sync(0xffffffffu, old[j], 1);
              out = ar * acc[i] + sgn * ai * acc_o;
              if (read_c) out += br * old[j] + sgn * bi * old_o;
            } else {
              out = ar * acc[i];
              if (read_c) out = fmaf(br, old[j], out);
            }
            if (row_ok) cbase[static_cast<uint64_t>(col) * p.ldc] = out;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let tensor-core work still in flight finish before shared memory and
    // TMEM are released
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN>
cudaError_t launch_fused_variant(const FusedGemmArgs &a, cudaStream_t stream) {
  using Cfg = FusedCfg<BN>;
  auto kernel = tcec_gemm_fused_kernel<BN>;
  static std::once_flag once[64];
  static cudaError_t setup_error[64];
  static int num_sms[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&]() {
    setup_error[dev] = cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_sms[dev] = sms > 0 ? sms : 1;
    // The register re-allocation inside the kernel assumes the CTA was launched with at least
    // 72 registers per thread; refuse to launch anything else (an inc that cannot be served
    // would wait for ever).
    cudaFuncAttributes attr;
    if (setup_error[dev] == cudaSuccess) {
      setup_error[dev] = cudaFuncGetAttributes(&attr, kernel);
      if (setup_error[dev] == cudaSuccess &&
          attr.numRegs * NUM_THREADS < 512 * REGS_CVT + 128 * REGS_MMA + 256 * REGS_EPI)
        setup_error[dev] = cudaErrorLaunchOutOfResources;
    }
  });
  if (setup_error[dev] != cudaSuccess) return setup_error[dev];

  FusedParams fp;
  fp.a.src = a.a;
  fp.a.ld = a.lda;
  fp.a.stride = a.stride_a;
  fp.a.rows = a.m;
  fp.a.layout = a.layout_a;
  fp.b.src = a.b;
  fp.b.ld = a.ldb;
  fp.b.stride = a.stride_b;
  fp.b.rows = a.n;
  fp.b.layout = a.layout_b;
  fp.k = a.k;
  fp.diag = 0;
#ifdef CUMPSGEMM_FUSED_DIAG_BUILD
  if (const char *e = std::getenv("CUMPSGEMM_FUSED_DIAG")) fp.diag = std::atoi(e);
#endif
  GemmKernelParams p;
  p.c = a.c;
  p.c_array = nullptr;
  p.ldc = a.ldc;
  p.stride_c = a.stride_c;
  p.m = a.m;
  p.n = a.n;
  p.k_blocks = (a.k + KS - 1) / KS;
  p.tiles_m = (a.m + BM - 1) / BM;
  p.tiles_n = (a.n + BN - 1) / BN;
  p.alpha_r = a.alpha_r;
  p.alpha_i = a.alpha_i;
  p.beta_r = a.beta_r;
  p.beta_i = a.beta_i;
  p.lo_scale_inv = 1.f / 2048.f;
  p.is_complex = a.is_complex ? 1 : 0;
  p.dyn = a.dyn;
  p.status = a.dev_status;
  p.debug = nullptr;
  p.wave_counter = nullptr;
  // drain every two stages (128 k values); the first chunk of a tile follows the accuracy rule
  // of the pair kernel (tcec_gemm_pair.cu): it may be longer while the epilogue warps still
  // store the previous tile
  p.drain_chunk = (a.tuning.drain_chunk >= 1) ? static_cast<uint32_t>(a.tuning.drain_chunk) : 2u;
  const uint32_t k_total = p.k_blocks * KS;
  const uint32_t first_k = (k_total >= 8192u) ? 512u : (k_total >= 2048u ? 256u : 128u);
  p.first_chunk = (a.tuning.first_chunk >= 1) ? static_cast<uint32_t>(a.tuning.first_chunk)
                                              : first_k / KS;
  if (p.first_chunk < p.drain_chunk) p.first_chunk = p.drain_chunk;
  const uint64_t total = static_cast<uint64_t>(p.tiles_m) * p.tiles_n * a.batch;
  if (total == 0 || total > 0x7fffffffull) return cudaErrorInvalidValue;
  p.total_tiles = static_cast<uint32_t>(total);
  p.k_slices = 1;
  p.slice_blocks = p.k_blocks;
  p.slice_stride = 0;
  if (a.k_slices > 1) {
    // plain partial sums into the caller's scratch, [slice][batch][column][row]; alpha, beta,
    // complex arithmetic and the un-scaling are the reduction kernel's
    if (a.partial == nullptr || a.k_slices > 0xffffu) return cudaErrorInvalidValue;
    p.slice_blocks = (p.k_blocks + a.k_slices - 1) / a.k_slices;
    const uint32_t slices = (p.k_blocks + p.slice_blocks - 1) / p.slice_blocks;
    if (slices != a.k_slices) return cudaErrorInvalidValue; // the caller sized the scratch
    p.k_slices = static_cast<uint16_t>(slices);
    p.c = a.partial;
    p.ldc = a.m;
    p.stride_c = static_cast<uint64_t>(a.m) * a.n;
    p.slice_stride = p.stride_c * a.batch;
    p.alpha_r = 1.f;
    p.alpha_i = 0.f;
    p.beta_r = 0.f;
    p.beta_i = 0.f;
    p.is_complex = 0;
  }
  const uint64_t work = total * p.k_slices;
  if (work > 0x7fffffffull) return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>(
      work < static_cast<uint64_t>(num_sms[dev]) ? work : num_sms[dev]);
  kernel<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(fp, p);
  return cudaGetLastError();
}

} // namespace

cudaError_t launch_tcec_gemm_fused(const FusedGemmArgs &a, cudaStream_t stream) {
  if (a.tile_n == 64) return launch_fused_variant<64>(a, stream);
  return launch_fused_variant<128>(a, stream);
}

} // namespace cumpsgemm_b200
