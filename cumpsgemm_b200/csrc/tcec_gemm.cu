// Error-corrected tensor-core GEMM for sm_100a.
//
// Replaces the reference's gemm_kernel / gemm_batchStrided_kernel /
// gemm_atomic_kernel (src/cumpsgemm_kernel.cuh:468-585) and the fragment
// arithmetic they call (src/device_tcec_wrapper.hpp:21-106).
//
// Inputs are the K-major hi/lo operand panels written by the split pass
// (split_kernels.cu).  One CTA owns a 128 x BN tile of C:
//   warp 0      : TMA producer (cp.async.bulk.tensor, no multicast)
//   warp 1      : TMEM allocation + single-thread tcgen05.mma issue
//   warps 4..11 : accumulator drain (tcgen05.ld), FP32 running sum in
//                 registers, alpha/beta epilogue with direct coalesced stores
// Per K stage (128 bytes of K per row = 64 FP16 or 32 TF32 values):
//   D0  = Ahi * Bhi            (overwritten every stage, drained every stage
//                               and added to the running sum with an FP32
//                               round-to-nearest add outside the tensor core)
//   D1 += Alo * Bhi + Ahi * Blo (stays in TMEM for the whole K loop)
// result = sum(D0 drains) + D1 * lo_scale_inv   (2^-11 for FP16, 1 for TF32).
// While the tensor core runs the two correction products of a stage the
// epilogue warps drain D0 of the same stage, so D0 needs no double buffering
// and the two accumulators fill the 512 TMEM columns at BN = 256.
#include "gemm_common.cuh"
#include "ptx.cuh"

#include <mutex>

namespace cumpsgemm_b200 {
namespace {

constexpr int BM = 128;
constexpr int ROW_BYTES = kGemmRowBytes;
constexpr int NUM_THREADS = 384;
constexpr int NUM_EPI_WARPS = 8;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t D1_COL = 256;
constexpr int SMEM_LIMIT = 227 * 1024;

template <int BN, bool EC> struct TileCfg {
  static constexpr int A_TILE = BM * ROW_BYTES;
  static constexpr int B_TILE = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = (A_TILE + B_TILE) * (EC ? 2 : 1);
  static constexpr int STAGES_RAW = (SMEM_LIMIT - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
  static_assert(STAGES >= 2, "need at least two stages");
};

using KernelParams = GemmKernelParams;

template <int KIND> __device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b,
                                                           uint32_t idesc, uint32_t acc) {
  if constexpr (KIND == 0) {
    ptx::mma_f16_ss(d, a, b, idesc, acc);
  } else {
    ptx::mma_tf32_ss(d, a, b, idesc, acc);
  }
}

template <int KIND, int BN, bool EC>
__device__ __forceinline__ void tcec_gemm_body(const CUtensorMap &map_a, const CUtensorMap &map_b,
                                               const KernelParams &p) {
  using Cfg = TileCfg<BN, EC>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int K_STEPS = ROW_BYTES / 32;    // tcgen05.mma consumes 32 bytes of K per instruction
  constexpr int MY_MODE = (KIND == 0) ? CUMPSGEMM_FP16TCEC : CUMPSGEMM_TF32TCEC;
  constexpr uint32_t IDESC = ptx::make_idesc(KIND == 0 ? 0 : 2, BM, BN);
  constexpr int CPT = BN / 2; // accumulator columns per epilogue thread

  // Gated launch: leave at once when the device-side decision picked the other kind.
  if (p.dyn != nullptr && p.dyn->gemm_mode != MY_MODE) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *d0_full = bars + 2 * STAGES;
  uint64_t *d0_empty = bars + 2 * STAGES + 1;
  uint64_t *d1_full = bars + 2 * STAGES + 2;
  uint32_t *tmem_base_ptr = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 3);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- tile coordinates: grouped raster so that concurrently resident CTAs
  //      share A and B panels in L2
  const uint32_t tiles_per_batch = p.tiles_m * p.tiles_n;
  const uint32_t slice = blockIdx.x % p.k_slices;
  const uint32_t tile_linear = blockIdx.x / p.k_slices;
  const uint32_t batch_id = tile_linear / tiles_per_batch;
  const uint32_t t = tile_linear - batch_id * tiles_per_batch;
  constexpr uint32_t GROUP_M = 16;
  const uint32_t tiles_in_group = GROUP_M * p.tiles_n;
  const uint32_t group_id = t / tiles_in_group;
  const uint32_t first_m = group_id * GROUP_M;
  const uint32_t group_rows = min(p.tiles_m - first_m, GROUP_M);
  const uint32_t in_group = t - group_id * tiles_in_group;
  const uint32_t tile_m = first_m + in_group % group_rows;
  const uint32_t tile_n = in_group / group_rows;
  const int m0 = static_cast<int>(tile_m * BM);
  const int n0 = static_cast<int>(tile_n * BN);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(d0_full), 1);
    ptx::mbar_init(ptx::smem_u32(d0_empty), NUM_EPI_WARPS);
    ptx::mbar_init(ptx::smem_u32(d1_full), 1);
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_base_ptr), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  // this CTA's part of the K loop: stages [kb0, kb0 + k_blocks) of the p.k_blocks in a panel
  const uint32_t kb0 = slice * p.slice_blocks;
  const uint32_t k_blocks = min(p.slice_blocks, p.k_blocks - kb0);
  const bool dbg = (p.debug != nullptr);
  unsigned long long dbg_wait = 0, dbg_wait2 = 0;

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0) {
      // launched with programmatic serialization behind the split pass: everything up to here
      // ran while that pass was still draining; the panels are complete after this
      ptx::griddep_wait();
      const int za = static_cast<int>(batch_id * (EC ? 2u : 1u));
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        const uint32_t s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1u;
        if (!ptx::mbar_wait_timed(ptx::smem_u32(&empty_bar[s]), ph ^ 1u, abort_flag, p.status,
                                  ptx::kErrWaitEmpty, dbg, &dbg_wait))
          break;
        const uint32_t fb = ptx::smem_u32(&full_bar[s]);
        ptx::mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
        uint8_t *st = smem + s * Cfg::STAGE_BYTES;
        // coordinates: (element in the K block, row, plane * k_blocks + K block)
        const int zh = static_cast<int>(static_cast<uint32_t>(za) * p.k_blocks + kb0 + kb);
        ptx::tma_load_3d(ptx::smem_u32(st), &map_a, fb, 0, m0, zh);
        if constexpr (EC) {
          const int zl = zh + static_cast<int>(p.k_blocks);
          ptx::tma_load_3d(ptx::smem_u32(st + Cfg::A_TILE), &map_a, fb, 0, m0, zl);
          ptx::tma_load_3d(ptx::smem_u32(st + 2 * Cfg::A_TILE), &map_b, fb, 0, n0, zh);
          ptx::tma_load_3d(ptx::smem_u32(st + 2 * Cfg::A_TILE + Cfg::B_TILE), &map_b, fb, 0, n0,
                           zl);
        } else {
          ptx::tma_load_3d(ptx::smem_u32(st + Cfg::A_TILE), &map_b, fb, 0, n0, zh);
        }
      }
      if (dbg) atomicAdd(p.debug + 2, dbg_wait);
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t d0 = tmem_base;
      const uint32_t d1 = tmem_base + D1_COL;
      bool ok = true;
      const long long dbg_t0 = clock64();
      for (uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
        const uint32_t s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1u;
        ok = ptx::mbar_wait_timed(ptx::smem_u32(&full_bar[s]), ph, abort_flag, p.status,
                                  ptx::kErrWaitFull, dbg, &dbg_wait);
        if (!ok) break;
        // D0 of the previous stage must have been drained before it is overwritten.
        ok = ptx::mbar_wait_timed(ptx::smem_u32(d0_empty), (kb & 1u) ^ 1u, abort_flag, p.status,
                                  ptx::kErrWaitD0Empty, dbg, &dbg_wait2);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t st = ptx::smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t a_hi = ptx::make_kmajor_desc<ROW_BYTES>(st);
        const uint64_t a_lo = ptx::make_kmajor_desc<ROW_BYTES>(st + Cfg::A_TILE);
        const uint64_t b_hi =
            ptx::make_kmajor_desc<ROW_BYTES>(st + (EC ? 2 : 1) * Cfg::A_TILE);
        const uint64_t b_lo =
            ptx::make_kmajor_desc<ROW_BYTES>(st + 2 * Cfg::A_TILE + Cfg::B_TILE);
#pragma unroll
        for (int ks = 0; ks < K_STEPS; ++ks) {
          // advancing K by 32 bytes inside the swizzle atom = +2 in the address field
          mma_ss<KIND>(d0, a_hi + 2 * ks, b_hi + 2 * ks, IDESC, ks > 0 ? 1u : 0u);
        }
        ptx::tc_commit(ptx::smem_u32(d0_full));
        if constexpr (EC) {
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks) {
            mma_ss<KIND>(d1, a_lo + 2 * ks, b_hi + 2 * ks, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks) {
            mma_ss<KIND>(d1, a_hi + 2 * ks, b_lo + 2 * ks, IDESC, 1u);
          }
        }
        ptx::tc_commit(ptx::smem_u32(&empty_bar[s]));
      }
      if (ok) ptx::tc_commit(ptx::smem_u32(d1_full));
      if (dbg) {
        atomicAdd(p.debug + 0, dbg_wait);
        atomicAdd(p.debug + 1, dbg_wait2);
        atomicAdd(p.debug + 4, static_cast<unsigned long long>(clock64() - dbg_t0));
        atomicAdd(p.debug + 5, 1ull);
      }
    }
  } else if (warp >= 4) {
    // ================================================================ drain + epilogue
    const uint32_t quarter = static_cast<uint32_t>(warp & 3);      // TMEM lanes [32q, 32q+32)
    const uint32_t half = static_cast<uint32_t>((warp - 4) >> 2);  // column half of the tile
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const uint32_t col_base = half * CPT;

    float acc[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) acc[i] = 0.f;

    bool ok = true;
    for (uint32_t kb = 0; kb < k_blocks; ++kb) {
      ok = ptx::mbar_wait_timed(ptx::smem_u32(d0_full), kb & 1u, abort_flag, p.status,
                                ptx::kErrWaitD0Full, dbg, &dbg_wait);
      if (!ok) break;
      ptx::tc_fence_after();
#pragma unroll
      for (int pc = 0; pc < CPT / 32; ++pc) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + lane_addr + col_base + pc * 32, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[pc * 32 + i] += __uint_as_float(v[i]);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(d0_empty));
    }

    if (dbg && warp == 4 && lane == 0) atomicAdd(p.debug + 3, dbg_wait);
    if (ok && EC) {
      ok = ptx::mbar_wait(ptx::smem_u32(d1_full), 0u, abort_flag, p.status, ptx::kErrWaitD1Full);
      if (ok) {
        ptx::tc_fence_after();
        const float lsi = p.lo_scale_inv;
#pragma unroll
        for (int pc = 0; pc < CPT / 32; ++pc) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(tmem_base + D1_COL + lane_addr + col_base + pc * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            acc[pc * 32 + i] = fmaf(__uint_as_float(v[i]), lsi, acc[pc * 32 + i]);
        }
      }
    }

    if (ok) {
      // C(row, col) = alpha * acc + beta * C(row, col); lanes hold consecutive rows of a
      // column-major C, so each warp store covers 128 contiguous bytes.
      // (split-K partial sums are stored plain; scaling and alpha / beta belong to the reduction)
      const float unscale = (p.dyn != nullptr && p.k_slices == 1) ? p.dyn->unscale_c : 1.f;
      const float ar = p.alpha_r * unscale, ai = p.alpha_i * unscale;
      const float br = p.beta_r, bi = p.beta_i;
      const bool read_c = (br != 0.f) || (bi != 0.f);
      const uint32_t row = static_cast<uint32_t>(m0) + quarter * 32u + static_cast<uint32_t>(lane);
      const bool row_ok = row < p.m;
      float *cbase = ((p.c_array != nullptr) ? p.c_array[batch_id]
                                              : p.c + static_cast<uint64_t>(batch_id) * p.stride_c +
                                                    static_cast<uint64_t>(slice) * p.slice_stride) +
                     row;
      const float sgn = (lane & 1) ? 1.f : -1.f; // odd rows hold imaginary parts
      // Columns go in groups: all loads of a group are issued before its first store (the
      // compiler must assume a store may alias the next load, which would put one memory
      // latency per column on the tile's critical path when beta != 0).
      constexpr int EPI_BATCH = (CPT >= 8) ? 8 : CPT;
#pragma unroll
      for (int i0 = 0; i0 < CPT; i0 += EPI_BATCH) {
        float old[EPI_BATCH];
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const uint32_t col = static_cast<uint32_t>(n0) + col_base + static_cast<uint32_t>(i0 + j);
          old[j] = (read_c && row_ok && col < p.n)
                       ? __ldcs(cbase + static_cast<uint64_t>(col) * p.ldc)
                       : 0.f;
        }
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const int i = i0 + j;
          const uint32_t col = static_cast<uint32_t>(n0) + col_base + static_cast<uint32_t>(i);
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
    // A wait gave up.  Give copies that may still be in flight time to land in
    // this CTA's shared memory before it is released.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int KIND, int BN, bool EC>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    tcec_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, const KernelParams p) {
  tcec_gemm_body<KIND, BN, EC>(map_a, map_b, p);
}

// AUTO: the kind is decided on the device; both kinds' tensor maps and parameters travel with
// the launch (see tcec_gemm_pair.cu).  Shared memory is sized for the TF32 kind's stages,
// which are the same bytes as the FP16 kind's.
template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    tcec_gemm_auto_kernel(const __grid_constant__ CUtensorMap map_a16,
                          const __grid_constant__ CUtensorMap map_b16, const KernelParams p16,
                          const __grid_constant__ CUtensorMap map_a32,
                          const __grid_constant__ CUtensorMap map_b32, const KernelParams p32) {
  if (p16.dyn->gemm_mode == CUMPSGEMM_TF32TCEC)
    tcec_gemm_body<1, BN, true>(map_a32, map_b32, p32);
  else
    tcec_gemm_body<0, BN, true>(map_a16, map_b16, p16);
}

} // namespace

// ---------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// Tensor map over a K-blocked panel (layout: split_kernels.cu); see gemm_common.cuh.
bool make_panel_map(CUtensorMap *map, SplitKind kind, const void *panel, uint32_t k_pad,
                    uint32_t rows_pad, uint32_t planes, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  const uint32_t es = (kind == SplitKind::fp16) ? 2u : 4u;
  // K-blocked panel: 128-byte K slices of all rows of one K block are contiguous.
  const uint32_t kbe = ROW_BYTES / es;
  const uint32_t k_blocks = k_pad / kbe;
  const cuuint64_t dims[3] = {kbe, rows_pad, static_cast<cuuint64_t>(planes) * k_blocks};
  const cuuint64_t strides[2] = {ROW_BYTES, static_cast<cuuint64_t>(ROW_BYTES) * rows_pad};
  const cuuint32_t box[3] = {kbe, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      (kind == SplitKind::fp16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r =
      fn(map, dt, 3, const_cast<void *>(panel), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

namespace {

// Tensor maps, kernel parameters and grid size of one kind.
template <int BN, bool EC>
bool prepare_variant(const TcecGemmArgs &a, SplitKind kind, CUtensorMap *map_a, CUtensorMap *map_b,
                     KernelParams *pp, unsigned *grid_out) {
  const uint32_t planes = a.batch * (EC ? 2u : 1u);
  if (!make_panel_map(map_a, kind, a.panel_a, a.k_pad, a.rows_pad_a, planes, BM) ||
      !make_panel_map(map_b, kind, a.panel_b, a.k_pad, a.rows_pad_b, planes, BN)) {
    return false;
  }
  KernelParams &p = *pp;
  p.c = a.c;
  p.c_array = a.c_array;
  p.ldc = a.ldc;
  p.stride_c = a.stride_c;
  p.m = a.m;
  p.n = a.n;
  const uint32_t es = (kind == SplitKind::fp16) ? 2u : 4u;
  p.k_blocks = a.k_pad / (ROW_BYTES / es);
  p.tiles_m = (a.m + BM - 1) / BM;
  p.tiles_n = (a.n + BN - 1) / BN;
  p.alpha_r = a.alpha_r;
  p.alpha_i = a.alpha_i;
  p.beta_r = a.beta_r;
  p.beta_i = a.beta_i;
  p.lo_scale_inv = (kind == SplitKind::fp16) ? (1.f / 2048.f) : 1.f;
  p.is_complex = a.is_complex ? 1 : 0;
  p.dyn = a.dyn;
  p.status = a.dev_status;
  p.debug = a.debug;
  p.wave_counter = nullptr;
  p.drain_chunk = 1;
  p.first_chunk = 1;
  p.total_tiles = 0;
  p.k_slices = 1;
  p.slice_blocks = p.k_blocks;
  p.slice_stride = 0;
  if (a.k_slices > 1) {
    // partial sums: plain floats into the caller's scratch, one m x n block per slice and batch
    // entry; the slice length is the same number of 64-k-value units for both kinds
    const uint32_t units = a.k_pad / 64;
    const uint32_t per_slice_units = (units + a.k_slices - 1) / a.k_slices;
    p.slice_blocks = per_slice_units * (64 / (ROW_BYTES / es));
    const uint32_t slices = (p.k_blocks + p.slice_blocks - 1) / p.slice_blocks;
    p.k_slices = static_cast<uint16_t>(slices);
    if (slices != a.k_slices || slices > 0xffffu || a.partial == nullptr || a.c_array != nullptr)
      return false;
    p.c = a.partial;
    p.c_array = nullptr;
    p.ldc = a.m;
    p.stride_c = static_cast<uint64_t>(a.m) * a.n;
    p.slice_stride = p.stride_c * a.batch;
    p.alpha_r = 1.f;
    p.alpha_i = 0.f;
    p.beta_r = 0.f;
    p.beta_i = 0.f;
    p.is_complex = 0;
  }
  const uint64_t grid = static_cast<uint64_t>(p.tiles_m) * p.tiles_n * a.batch * p.k_slices;
  if (grid == 0 || grid > 0x7fffffffull) return false;
  *grid_out = static_cast<unsigned>(grid);
  return true;
}

// Shared-memory attribute of a kernel, once per device.  TAG tells kernels of equal function
// type apart.
template <int TAG, class Kernel> cudaError_t smem_setup(Kernel kernel, int smem_bytes) {
  static std::once_flag once[64];
  static cudaError_t setup_error[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&]() {
    setup_error[dev] =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  });
  return setup_error[dev];
}

// Launch with programmatic stream serialization: the kernel may be scheduled while the
// kernel before it in the stream (the split pass) is still draining; the producer's
// griddep_wait() orders the first panel load behind that kernel's completion.
template <class Kernel, class... Args>
cudaError_t launch_after_split(Kernel kernel, unsigned grid, int smem_bytes, cudaStream_t stream,
                               Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int KIND, int BN, bool EC>
cudaError_t launch_variant(const TcecGemmArgs &a, cudaStream_t stream) {
  using Cfg = TileCfg<BN, EC>;
  auto kernel = tcec_gemm_kernel<KIND, BN, EC>;
  const cudaError_t se = smem_setup<KIND * 8 + (BN / 64) * 2 + (EC ? 1 : 0)>(kernel, Cfg::SMEM_BYTES);
  if (se != cudaSuccess) return se;
  CUtensorMap map_a, map_b;
  KernelParams p;
  unsigned grid = 0;
  if (!prepare_variant<BN, EC>(a, KIND == 0 ? SplitKind::fp16 : SplitKind::tf32, &map_a, &map_b, &p,
                               &grid))
    return cudaErrorInvalidValue;
  return launch_after_split(kernel, grid, Cfg::SMEM_BYTES, stream, map_a, map_b, p);
}

template <int BN> cudaError_t launch_auto_variant(const TcecGemmArgs &a, cudaStream_t stream) {
  using Cfg = TileCfg<BN, true>;
  auto kernel = tcec_gemm_auto_kernel<BN>;
  const cudaError_t se = smem_setup<100 + BN / 64>(kernel, Cfg::SMEM_BYTES);
  if (se != cudaSuccess) return se;
  CUtensorMap a16, b16, a32, b32;
  KernelParams p16, p32;
  unsigned grid = 0;
  if (!prepare_variant<BN, true>(a, SplitKind::fp16, &a16, &b16, &p16, &grid) ||
      !prepare_variant<BN, true>(a, SplitKind::tf32, &a32, &b32, &p32, &grid))
    return cudaErrorInvalidValue;
  return launch_after_split(kernel, grid, Cfg::SMEM_BYTES, stream, a16, b16, p16, a32, b32, p32);
}

template <int KIND, bool EC> cudaError_t launch_by_tile(const TcecGemmArgs &a, cudaStream_t s) {
  switch (a.tile_n) {
  case 256:
    return launch_variant<KIND, 256, EC>(a, s);
  case 128:
    return launch_variant<KIND, 128, EC>(a, s);
  case 64:
    return launch_variant<KIND, 64, EC>(a, s);
  default:
    return cudaErrorInvalidValue;
  }
}

// One CTA waits, with the library's bounded wait, on an mbarrier that nothing ever signals.
// The wait must give up after limit_ns, record kErrWaitFull in *status and let the kernel
// return normally: this is the path every GEMM wait takes if a copy or an MMA never completes.
__global__ void bounded_wait_selftest_kernel(int *status, unsigned long long limit_ns,
                                             unsigned long long *waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    abort_flag = 0;
    ptx::mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = ptx::globaltimer_ns();
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0u, &abort_flag, status,
                                   ptx::kErrWaitFull, limit_ns);
    *waited_ns = ptx::globaltimer_ns() - t0;
    if (ok) atomicCAS(status, 0, -1); // a wait on an idle barrier must not succeed
  }
  __syncthreads();
}

} // namespace

cudaError_t launch_bounded_wait_selftest(int *dev_status, unsigned long long limit_ns,
                                         unsigned long long *dev_waited_ns, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(dev_status, limit_ns, dev_waited_ns);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- split-K reduction
namespace {
__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(const float *partial, uint32_t slices, uint64_t slice_stride,
                         uint64_t total, uint32_t m, uint32_t n, float *c, uint64_t ldc,
                         uint64_t stride_c, float alpha_r, float alpha_i, float beta_r,
                         float beta_i, int is_complex, const DynParams *dyn) {
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint64_t per_batch = static_cast<uint64_t>(m) * n;
  const uint64_t b = idx / per_batch;
  const uint64_t r = idx - b * per_batch;
  const uint32_t col = static_cast<uint32_t>(r / m);
  const uint32_t row = static_cast<uint32_t>(r - static_cast<uint64_t>(col) * m);
  // slices in ascending order: the sum does not depend on which CTA finished first
  float sum = 0.f, sum_o = 0.f;
  const float *pp = partial + idx;
  for (uint32_t s = 0; s < slices; ++s) sum += pp[s * slice_stride];
  const float unscale = (dyn != nullptr) ? dyn->unscale_c : 1.f;
  const float ar = alpha_r * unscale, ai = alpha_i * unscale;
  float *cp = c + b * stride_c + static_cast<uint64_t>(col) * ldc + row;
  const bool read_c = (beta_r != 0.f) || (beta_i != 0.f);
  float out;
  if (is_complex) {
    // rows 2i / 2i+1 hold the real / imaginary part of complex row i
    const float *po = partial + (idx ^ 1ull);
    for (uint32_t s = 0; s < slices; ++s) sum_o += po[s * slice_stride];
    const float sgn = (row & 1u) ? 1.f : -1.f;
    out = ar * sum + sgn * ai * sum_o;
    if (read_c) {
      float *co = (row & 1u) ? cp - 1 : cp + 1;
      out += beta_r * (*cp) + sgn * beta_i * (*co);
    }
  } else {
    out = ar * sum;
    if (read_c) out = fmaf(beta_r, *cp, out);
  }
  // complex: the partner thread reads this element of C as well; all reads happen before the
  // writes of the pair because both threads are in the same warp (m is even, idx ^ 1 adjacent)
  __syncwarp();
  *cp = out;
}
} // namespace

std::uint32_t split_k_slices(std::uint32_t k_pad, std::uint32_t wanted) {
  const std::uint32_t units = k_pad / 64;
  if (wanted <= 1 || units <= 1) return 1;
  if (wanted > units) wanted = units;
  const std::uint32_t per = (units + wanted - 1) / wanted;
  return (units + per - 1) / per;
}

cudaError_t launch_splitk_reduce(const TcecGemmArgs &a, cudaStream_t stream) {
  if (a.k_slices <= 1 || a.partial == nullptr || a.c == nullptr) return cudaErrorInvalidValue;
  const uint64_t total = static_cast<uint64_t>(a.m) * a.n * a.batch;
  const uint64_t blocks = (total + 255) / 256;
  if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
  splitk_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      a.partial, a.k_slices, total, total, a.m, a.n, a.c, a.ldc, a.stride_c, a.alpha_r, a.alpha_i,
      a.beta_r, a.beta_i, a.is_complex ? 1 : 0, a.dyn);
  return cudaGetLastError();
}

cudaError_t launch_tcec_gemm_auto(const TcecGemmArgs &a, cudaStream_t stream) {
  if (!a.error_correction || a.dyn == nullptr) return cudaErrorInvalidValue;
  switch (a.tile_n) {
  case 256:
    return launch_auto_variant<256>(a, stream);
  case 128:
    return launch_auto_variant<128>(a, stream);
  case 64:
    return launch_auto_variant<64>(a, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

cudaError_t launch_tcec_gemm(const TcecGemmArgs &a, cudaStream_t stream) {
  if (a.kind == SplitKind::fp16) {
    return a.error_correction ? launch_by_tile<0, true>(a, stream)
                              : launch_by_tile<0, false>(a, stream);
  }
  return a.error_correction ? launch_by_tile<1, true>(a, stream)
                            : launch_by_tile<1, false>(a, stream);
}

int tcec_gemm_stages(int tile_n, bool ec) {
  switch (tile_n) {
  case 256:
    return ec ? TileCfg<256, true>::STAGES : TileCfg<256, false>::STAGES;
  case 128:
    return ec ? TileCfg<128, true>::STAGES : TileCfg<128, false>::STAGES;
  case 64:
    return ec ? TileCfg<64, true>::STAGES : TileCfg<64, false>::STAGES;
  default:
    return 0;
  }
}

} // namespace cumpsgemm_b200
