// Error-corrected tensor-core GEMM, persistent CTA-pair variant (tcgen05 cta_group::2).
//
// Same arithmetic, panels and barrier protocol as tcec_gemm.cu (which replaces the
// reference's src/cumpsgemm_kernel.cuh:468-585); what changes is the tile and the schedule.
// A cluster of two CTAs owns 256 x 256 tiles of C: each CTA loads its own 128 rows of A
// (hi, lo) and its own 128-row half of the B tile (hi, lo), the even CTA issues every
// tcgen05.mma for the pair, and each CTA's TMEM receives its own 128 x 256 part of the
// accumulators, which its own epilogue warps drain.  Per SM and k-stage this moves 64 KiB from
// L2 instead of 96 KiB and leaves room for three stages instead of two.
//
// The kernel is persistent: the grid holds at most one cluster per SM pair and every cluster
// walks the tiles  t = cluster, cluster + #clusters, ...  The producer and the MMA issuer run
// ahead into the next tile while the epilogue warps still write the previous one: the next
// tile's operands are loaded and its hi*hi products start as soon as the last drain of D0 is
// done; its correction products wait only until the epilogue has copied D1 into registers.
// Three schedule details came out of measurements and are explained where they are coded:
// clusters announce every tile start on a device counter and wait for their wave (keeps
// clusters that share panel rows at the same k, so the rows are fetched from DRAM once per
// wave); the first drain chunk of a tile is longer than the others (the epilogue warps are
// still storing the previous tile then); with beta != 0 the C tile is prefetched into L2 and
// read in groups of columns.
//
// Barriers (one set per CTA at identical shared-memory offsets; "leader" = cluster rank 0):
//   full[s]   leader's only: 1 arrival (leader's producer, expect_tx of both CTAs' bytes);
//             both CTAs' TMA loads complete on it (cta_group::2 loads, no multicast)
//   empty[s]  in both CTAs: 1 arrival, tcgen05.commit multicast from the leader
//   d0_full   in both CTAs: commit multicast after the hi*hi products of a chunk of stages
//   d0_empty  leader's only: 16 arrivals = 8 drain warps of each CTA (remote mbarrier arrive)
//   d1_full   in both CTAs: commit multicast after the last stage of a tile
//   d1_empty  leader's only: 16 arrivals, after the epilogue warps have read D1
// Every wait is bounded; no TMA multicast is used.
#include "gemm_common.cuh"
#include "ptx.cuh"

#include <mutex>

namespace cumpsgemm_b200 {
namespace {

constexpr int BM_CTA = 128;  // rows of C per CTA
constexpr int BN_PAIR = 256; // columns of C per pair (each CTA stores 128 rows of B)
constexpr int ROW_BYTES = kGemmRowBytes;
constexpr int NUM_THREADS = 384;
constexpr int NUM_EPI_WARPS = 8;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t D1_COL = 256;
constexpr int TILE_BYTES = 128 * ROW_BYTES; // every sub-tile is 128 rows
constexpr int STAGE_BYTES = 4 * TILE_BYTES; // A_hi, A_lo, B_hi, B_lo
constexpr int STAGES = 3;
constexpr uint32_t kPaceMinStages = 32; // shortest K loop (in stages) that is paced
constexpr uint32_t C_PREFETCH_LEAD = 8; // drain chunks between the L2 prefetch of C and its use
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

template <int KIND>
__device__ __forceinline__ void mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                         uint32_t acc) {
  if constexpr (KIND == 0) {
    ptx::mma_f16_ss_pair(d, a, b, idesc, acc);
  } else {
    ptx::mma_tf32_ss_pair(d, a, b, idesc, acc);
  }
}

struct TileCoord {
  uint32_t batch;
  int m0; // first row of this CTA's 128 rows
  int n0; // first column of the pair's 256 columns
};

// Grouped raster over pair tiles: tiles that run at the same time share A and B panels in L2.
__device__ __forceinline__ TileCoord tile_coord(uint32_t tile, const GemmKernelParams &p,
                                                uint32_t rank) {
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
  const uint32_t tile_m = first_m + in_group % group_rows;
  const uint32_t tile_n = in_group / group_rows;
  c.m0 = static_cast<int>(tile_m * 2 * BM_CTA + rank * BM_CTA);
  c.n0 = static_cast<int>(tile_n * BN_PAIR);
  return c;
}

// K-split of the last, partly filled wave.  With T tiles on C clusters the last wave has
// T mod C tiles; when that is at most half of C, each of those tiles is cut into `slices` K
// ranges that run on different clusters at the same time, so the wave takes 1/slices of a
// tile's time instead of a whole one (m=n=k=4096: 256 tiles on 74 clusters = 3.46 waves, the
// last 34 tiles are cut in two and the launch takes 3.5 tile times instead of 4).  Every slice
// writes its plain FP32 partial sums to scratch memory and takes a ticket from the tile's
// counter; the CTA that draws the last ticket adds the slices in ascending order (so the
// result does not depend on which one that is) and runs the alpha / beta epilogue.  Nobody
// waits for anybody, hence no assumption about which clusters are resident together.
// Work item w of a launch: w < split_begin is tile w with its whole K loop; beyond that,
// item split_begin + u is slice u % slices of tile split_begin + u / slices.
struct PairTail {
  float *partial;          // [tail tile][slice][CTA rank][256 columns][128 rows]
  unsigned int *counters;  // [tail tile][CTA rank], zero at launch
  uint32_t split_begin;    // first tile that is split (= total tiles when nothing is split)
  uint32_t slices;         // K slices per split tile (1: nothing is split)
  uint32_t slice_blocks;   // stages per slice (the last one may be shorter)
  uint32_t work_items;     // split_begin + (total tiles - split_begin) * slices
};

struct WorkItem {
  uint32_t tile, kb0, kbn, slice;
};

__device__ __forceinline__ WorkItem work_item(uint32_t w, const PairTail &t, uint32_t k_blocks) {
  WorkItem x;
  if (w < t.split_begin) {
    x.tile = w;
    x.kb0 = 0;
    x.kbn = k_blocks;
    x.slice = 0;
  } else {
    const uint32_t u = w - t.split_begin;
    const uint32_t ti = u / t.slices;
    x.tile = t.split_begin + ti;
    x.slice = u - ti * t.slices;
    x.kb0 = x.slice * t.slice_blocks;
    x.kbn = min(t.slice_blocks, k_blocks - x.kb0);
  }
  return x;
}

template <int KIND>
__device__ __forceinline__ void pair_body(const CUtensorMap &map_a, const CUtensorMap &map_b,
                                          const GemmKernelParams &p, const PairTail &tail) {
  constexpr int K_STEPS = ROW_BYTES / 32;
  constexpr int MY_MODE = (KIND == 0) ? CUMPSGEMM_FP16TCEC : CUMPSGEMM_TF32TCEC;
  constexpr uint32_t IDESC = ptx::make_idesc(KIND == 0 ? 0 : 2, 2 * BM_CTA, BN_PAIR);
  constexpr int CPT = BN_PAIR / 2;

  if (p.dyn != nullptr && p.dyn->gemm_mode != MY_MODE) return; // uniform over the cluster

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *d0_full = bars + 2 * STAGES;
  uint64_t *d0_empty = bars + 2 * STAGES + 1;
  uint64_t *d1_full = bars + 2 * STAGES + 2;
  uint64_t *d1_empty = bars + 2 * STAGES + 3;
  uint64_t *tail_bar = bars + 2 * STAGES + 4; // the eight epilogue warps of this CTA (tail split)
  uint32_t *tmem_base_ptr = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_base_ptr + 1);
  volatile uint32_t *ticket_smem = reinterpret_cast<volatile uint32_t *>(tmem_base_ptr + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = (rank == 0);
  const uint32_t cluster_id = blockIdx.x >> 1;
  const uint32_t num_clusters = gridDim.x >> 1;
  const uint32_t work_items = tail.work_items;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(d0_full), 1);
    ptx::mbar_init(ptx::smem_u32(d0_empty), 2 * NUM_EPI_WARPS);
    ptx::mbar_init(ptx::smem_u32(d1_full), 1);
    ptx::mbar_init(ptx::smem_u32(d1_empty), 2 * NUM_EPI_WARPS);
    ptx::mbar_init(ptx::smem_u32(tail_bar), NUM_EPI_WARPS);
    *abort_flag = 0;
    ptx::mbar_init_fence();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_base_ptr), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before any remote arrive / remote TMA completion
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  const uint32_t k_blocks = p.k_blocks;
  const bool dbg = (p.debug != nullptr);
  unsigned long long dbg_wait = 0, dbg_wait2 = 0;

  if (warp == 0) {
    // ================================================================ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0; // stage uses since kernel start, across tiles
      bool ok = true;
      bool pace = leader && p.wave_counter != nullptr && work_items > num_clusters;
      uint32_t wave = 0;
      for (uint32_t w = cluster_id; w < work_items && ok; w += num_clusters, ++wave) {
        const WorkItem wi = work_item(w, tail, k_blocks);
        const TileCoord tc = tile_coord(wi.tile, p, rank);
        const int za = static_cast<int>(tc.batch * 2u);
        const int nb0 = tc.n0 + static_cast<int>(rank) * 128; // this CTA's rows of the B tile
        if (pace) {
          // Keep the clusters in step.  Clusters that run at the same time share panel rows
          // through L2 only while they are at about the same k; left alone they drift apart
          // by about 2 % per tile and, once the drift exceeds what L2 retains, most loads go
          // to DRAM (measured at m=n=k=16384: 88 GB read per launch against 4 GB of panels
          // and C).  So every cluster announces each tile start and waits until all clusters
          // of the wave have.  The wait is only a pacing aid: it gives up after 100 us, and
          // then this cluster stops pacing for the rest of the launch, so clusters that are
          // not resident at the same time cost one time-out and never a wrong result.
          atomicAdd(p.wave_counter, 1u);
          const uint32_t target = min(work_items, (wave + 1) * num_clusters);
          const uint64_t t0 = ptx::globaltimer_ns();
          while (*reinterpret_cast<volatile unsigned int *>(p.wave_counter) < target) {
            if (ptx::globaltimer_ns() - t0 > 100000ull) {
              pace = false;
              break;
            }
            __nanosleep(64);
          }
        }
        for (uint32_t kb = 0; kb < wi.kbn; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait_timed(ptx::smem_u32(&empty_bar[s]), ph ^ 1u, abort_flag, p.status,
                                    ptx::kErrWaitEmpty, dbg, &dbg_wait);
          if (!ok) break;
          const uint32_t fb_local = ptx::smem_u32(&full_bar[s]);
          if (leader) ptx::mbar_arrive_expect_tx(fb_local, 2 * STAGE_BYTES);
          const uint32_t fb = ptx::map_to_cta(fb_local, 0); // the leader's barrier
          const uint32_t st = ptx::smem_u32(smem + s * STAGE_BYTES);
          // coordinates: (element in the K block, row, plane * k_blocks + K block); each box
          // is one contiguous 16 KiB run of the K-blocked panel
          const int zh = static_cast<int>(static_cast<uint32_t>(za) * k_blocks + wi.kb0 + kb);
          const int zl = zh + static_cast<int>(k_blocks);
          ptx::tma_load_3d_pair(st, &map_a, fb, 0, tc.m0, zh);
          ptx::tma_load_3d_pair(st + TILE_BYTES, &map_a, fb, 0, tc.m0, zl);
          ptx::tma_load_3d_pair(st + 2 * TILE_BYTES, &map_b, fb, 0, nb0, zh);
          ptx::tma_load_3d_pair(st + 3 * TILE_BYTES, &map_b, fb, 0, nb0, zl);
        }
      }
      if (dbg) atomicAdd(p.debug + 2, dbg_wait);
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (leader only)
    if (leader && lane == 0) {
      const uint32_t d0 = tmem_base;
      const uint32_t d1 = tmem_base + D1_COL;
      constexpr uint16_t BOTH = 0x3;
      bool ok = true;
      const long long dbg_t0 = clock64();
      const uint32_t chunk = p.drain_chunk;
      const uint32_t first = p.first_chunk; // stages in the first chunk of every tile
      // Chunks of a tile: [0, first), then pieces of `chunk` stages.
      auto chunk_start = [&](uint32_t kb) {
        return kb == 0 || (kb >= first && (kb - first) % chunk == 0);
      };
      uint32_t it = 0, chunk_idx = 0, tile_iter = 0;
      for (uint32_t w = cluster_id; w < work_items && ok; w += num_clusters, ++tile_iter) {
        const uint32_t kbn = work_item(w, tail, k_blocks).kbn;
        for (uint32_t kb = 0; kb < kbn && ok; ++kb, ++it) {
          const bool first_in_chunk = chunk_start(kb);
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          ok = ptx::mbar_wait_timed(ptx::smem_u32(&full_bar[s]), ph, abort_flag, p.status,
                                    ptx::kErrWaitFull, dbg, &dbg_wait);
          if (!ok) break;
          if (first_in_chunk) {
            // D0 of the previous chunk must have been drained before it is overwritten.
            ok = ptx::mbar_wait_timed(ptx::smem_u32(d0_empty), (chunk_idx & 1u) ^ 1u, abort_flag,
                                      p.status, ptx::kErrWaitD0Empty, dbg, &dbg_wait2);
            if (!ok) break;
          }
          ptx::tc_fence_after();
          const uint32_t st = ptx::smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_hi = ptx::make_kmajor_desc<ROW_BYTES>(st);
          const uint64_t a_lo = ptx::make_kmajor_desc<ROW_BYTES>(st + TILE_BYTES);
          const uint64_t b_hi = ptx::make_kmajor_desc<ROW_BYTES>(st + 2 * TILE_BYTES);
          const uint64_t b_lo = ptx::make_kmajor_desc<ROW_BYTES>(st + 3 * TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks)
            mma_pair<KIND>(d0, a_hi + 2 * ks, b_hi + 2 * ks, IDESC,
                           (!first_in_chunk || ks > 0) ? 1u : 0u);
          const bool last_in_chunk = (kb + 1 == kbn) || chunk_start(kb + 1);
          if (last_in_chunk) ptx::tc_commit_pair(ptx::smem_u32(d0_full), BOTH);
          if (kb == 0) {
            // D1 still holds the previous tile's corrections until its epilogue has read them.
            ok = ptx::mbar_wait_timed(ptx::smem_u32(d1_empty), (tile_iter & 1u) ^ 1u, abort_flag,
                                      p.status, ptx::kErrWaitD1Empty, dbg, &dbg_wait2);
            if (!ok) break;
            ptx::tc_fence_after();
          }
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks)
            mma_pair<KIND>(d1, a_lo + 2 * ks, b_hi + 2 * ks, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < K_STEPS; ++ks)
            mma_pair<KIND>(d1, a_hi + 2 * ks, b_lo + 2 * ks, IDESC, 1u);
          ptx::tc_commit_pair(ptx::smem_u32(&empty_bar[s]), BOTH);
          if (last_in_chunk) ++chunk_idx;
        }
        if (ok) ptx::tc_commit_pair(ptx::smem_u32(d1_full), BOTH);
      }
      if (dbg) {
        atomicAdd(p.debug + 0, dbg_wait);
        atomicAdd(p.debug + 1, dbg_wait2);
        atomicAdd(p.debug + 4, static_cast<unsigned long long>(clock64() - dbg_t0));
        atomicAdd(p.debug + 5, 1ull);
      }
    }
  } else if (warp >= 4) {
    // ================================================================ drain + epilogue (both CTAs)
    const uint32_t quarter = static_cast<uint32_t>(warp & 3);
    const uint32_t half = static_cast<uint32_t>((warp - 4) >> 2);
    const uint32_t lane_addr = (quarter * 32u) << 16;
    const uint32_t col_base = half * CPT;
    const uint32_t d0_empty_leader = ptx::map_to_cta(ptx::smem_u32(d0_empty), 0);
    const uint32_t d1_empty_leader = ptx::map_to_cta(ptx::smem_u32(d1_empty), 0);
    const float unscale = (p.dyn != nullptr) ? p.dyn->unscale_c : 1.f;
    const float ar = p.alpha_r * unscale, ai = p.alpha_i * unscale;
    const float br = p.beta_r, bi = p.beta_i;
    const bool read_c = (br != 0.f) || (bi != 0.f);
    const float sgn = (lane & 1) ? 1.f : -1.f; // odd rows hold imaginary parts
    const float lsi = p.lo_scale_inv;

    uint32_t chunk_idx = 0, tile_iter = 0, tail_phase = 0;
    bool ok = true;
    for (uint32_t w = cluster_id; w < work_items && ok; w += num_clusters, ++tile_iter) {
      const WorkItem wi = work_item(w, tail, k_blocks);
      const bool split = w >= tail.split_begin; // this item is one K slice of a tile
      const uint32_t n_chunks =
          1u + ((wi.kbn > p.first_chunk)
                    ? (wi.kbn - p.first_chunk + p.drain_chunk - 1) / p.drain_chunk
                    : 0u);
      const TileCoord tc = tile_coord(wi.tile, p, rank);
      float acc[CPT];
#pragma unroll
      for (int i = 0; i < CPT; ++i) acc[i] = 0.f;

      // C(row, col): lanes hold consecutive rows of the column-major C, so each warp access
      // covers 128 contiguous bytes of one column.
      const uint32_t row =
          static_cast<uint32_t>(tc.m0) + quarter * 32u + static_cast<uint32_t>(lane);
      const bool row_ok = row < p.m;
      float *cbase = ((p.c_array != nullptr) ? p.c_array[tc.batch]
                                              : p.c + static_cast<uint64_t>(tc.batch) * p.stride_c) +
                     row;
      const uint32_t prefetch_at = (n_chunks > C_PREFETCH_LEAD) ? n_chunks - C_PREFETCH_LEAD : 0u;

      for (uint32_t c = 0; c < n_chunks; ++c, ++chunk_idx) {
        if (read_c && !split && c == prefetch_at) {
          // beta != 0: pull this warp's part of the C tile into L2 a few chunks before the
          // epilogue reads it (lane l fetches the line of columns l, l+32, ...)
#pragma unroll
          for (int q = 0; q < CPT / 32; ++q) {
            const uint32_t col = static_cast<uint32_t>(tc.n0) + col_base +
                                 static_cast<uint32_t>(q * 32 + lane);
            if (col < p.n && row - lane < p.m)
              ptx::prefetch_l2(cbase - lane + static_cast<uint64_t>(col) * p.ldc);
          }
        }
        ok = ptx::mbar_wait_timed(ptx::smem_u32(d0_full), chunk_idx & 1u, abort_flag, p.status,
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
        if (lane == 0) ptx::mbar_arrive_cluster(d0_empty_leader);
      }
      if (!ok) break;

      ok = ptx::mbar_wait(ptx::smem_u32(d1_full), tile_iter & 1u, abort_flag, p.status,
                          ptx::kErrWaitD1Full);
      if (!ok) break;
      ptx::tc_fence_after();
#pragma unroll
      for (int pc = 0; pc < CPT / 32; ++pc) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + D1_COL + lane_addr + col_base + pc * 32, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          acc[pc * 32 + i] = fmaf(__uint_as_float(v[i]), lsi, acc[pc * 32 + i]);
      }
      // D1 is in registers: the issuer may start the next tile's correction products
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(d1_empty_leader);

      if (split) {
        // one K slice of a tile: park the partial sums, take a ticket, and go on to the
        // epilogue only with the last ticket of this CTA's half of the tile
        const uint32_t ti = wi.tile - tail.split_begin;
        constexpr uint32_t HALF = BN_PAIR * BM_CTA; // floats of one CTA's 128 x 256 half
        float *tbase = tail.partial + (static_cast<uint64_t>(ti) * tail.slices * 2u + rank) * HALF +
                       quarter * 32u + static_cast<uint32_t>(lane);
        float *mine = tbase + static_cast<uint64_t>(wi.slice) * 2u * HALF;
#pragma unroll
        for (int i = 0; i < CPT; ++i) __stcg(mine + (col_base + i) * BM_CTA, acc[i]);
        __threadfence();
        // the eight epilogue warps meet twice (all partial sums stored; ticket published) on
        // an mbarrier of their own, with the bounded wait every other wait here uses
        auto meet = [&]() -> bool {
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(tail_bar));
          const bool met = ptx::mbar_wait(ptx::smem_u32(tail_bar), tail_phase, abort_flag,
                                          p.status, ptx::kErrWaitTail);
          tail_phase ^= 1u;
          return met;
        };
        ok = meet();
        if (!ok) break;
        if (warp == 4 && lane == 0) *ticket_smem = atomicAdd(tail.counters + ti * 2u + rank, 1u);
        ok = meet();
        if (!ok) break;
        if (*ticket_smem != tail.slices - 1u) continue;
        __threadfence();
#pragma unroll
        for (int i = 0; i < CPT; ++i) acc[i] = __ldcg(tbase + (col_base + i) * BM_CTA);
        for (uint32_t sl = 1; sl < tail.slices; ++sl) {
          const float *other = tbase + static_cast<uint64_t>(sl) * 2u * HALF;
#pragma unroll
          for (int i = 0; i < CPT; ++i) acc[i] += __ldcg(other + (col_base + i) * BM_CTA);
        }
      }

      // C(row, col) = alpha * acc + beta * C(row, col)
      // Columns go in groups of EPI_BATCH: all loads of a group are issued before its first
      // store, otherwise every load would wait for the store before it (the compiler must
      // assume they alias) and a tile would spend 128 memory latencies here.
      constexpr int EPI_BATCH = 8;
#pragma unroll
      for (int i0 = 0; i0 < CPT; i0 += EPI_BATCH) {
        float old[EPI_BATCH];
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const uint32_t col =
              static_cast<uint32_t>(tc.n0) + col_base + static_cast<uint32_t>(i0 + j);
          old[j] = (read_c && row_ok && col < p.n)
                       ? __ldcs(cbase + static_cast<uint64_t>(col) * p.ldc)
                       : 0.f;
        }
#pragma unroll
        for (int j = 0; j < EPI_BATCH; ++j) {
          const int i = i0 + j;
          const uint32_t col = static_cast<uint32_t>(tc.n0) + col_base + static_cast<uint32_t>(i);
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
    if (dbg && warp == 4 && lane == 0) atomicAdd(p.debug + 3, dbg_wait);
  }

  // ---------------------------------------------------------------- teardown
  // The peer's shared memory and TMEM are in use by the leader's MMAs until the last d1_full
  // has fired in both CTAs; the cluster barrier below keeps either CTA from leaving before
  // the other has finished its last epilogue.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (*abort_flag) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    tcec_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_b, const GemmKernelParams p,
                          const PairTail tail) {
  pair_body<KIND>(map_a, map_b, p, tail);
}

// AUTO: both kinds' tensor maps and parameters travel with the launch; the device-side
// decision picks the pipeline (uniform over the grid).  The reference launches the kernels of
// both kinds and lets the deselected one exit at once (src/cumpsgemm_kernel.cuh:478-489).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    tcec_gemm_pair_auto_kernel(const __grid_constant__ CUtensorMap map_a16,
                               const __grid_constant__ CUtensorMap map_b16,
                               const GemmKernelParams p16,
                               const __grid_constant__ CUtensorMap map_a32,
                               const __grid_constant__ CUtensorMap map_b32,
                               const GemmKernelParams p32, const PairTail tail16,
                               const PairTail tail32) {
  if (p16.dyn->gemm_mode == CUMPSGEMM_TF32TCEC) {
    pair_body<1>(map_a32, map_b32, p32, tail32);
  } else {
    pair_body<0>(map_a16, map_b16, p16, tail16);
  }
}

// Per device and kernel, once (any thread): shared-memory attribute and the number of
// clusters the device can keep resident.  TAG tells the kernels apart (two of them have the
// same function type, which alone would make them share the statics below).
template <int TAG, class Kernel> cudaError_t pair_setup(Kernel kernel, int *clusters_out) {
  static std::once_flag once[64];
  static cudaError_t setup_error[64];
  static int max_clusters[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&]() {
    setup_error[dev] =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // one cluster per SM pair; if the device can co-schedule fewer, use what it reports
    int clusters = sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    int active = 0;
    if (setup_error[dev] == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&active, kernel, &cfg) == cudaSuccess) {
      if (active > 0 && active < clusters) clusters = active;
    } else {
      cudaGetLastError();
    }
    max_clusters[dev] = clusters > 0 ? clusters : 1;
  });
  *clusters_out = max_clusters[dev];
  return setup_error[dev];
}

// Tensor maps and kernel parameters of one kind.  Returns false on invalid sizes.
bool pair_prepare(const TcecGemmArgs &a, SplitKind kind, CUtensorMap *map_a, CUtensorMap *map_b,
                  GemmKernelParams *pp) {
  const uint32_t planes = a.batch * 2u;
  if (!make_panel_map(map_a, kind, a.panel_a, a.k_pad, a.rows_pad_a, planes, 128) ||
      !make_panel_map(map_b, kind, a.panel_b, a.k_pad, a.rows_pad_b, planes, 128)) {
    return false;
  }
  GemmKernelParams &p = *pp;
  p.c = a.c;
  p.c_array = a.c_array;
  p.ldc = a.ldc;
  p.stride_c = a.stride_c;
  p.m = a.m;
  p.n = a.n;
  const uint32_t es = (kind == SplitKind::fp16) ? 2u : 4u;
  p.k_blocks = a.k_pad / (ROW_BYTES / es);
  p.tiles_m = (a.m + 2 * BM_CTA - 1) / (2 * BM_CTA);
  p.tiles_n = (a.n + BN_PAIR - 1) / BN_PAIR;
  p.alpha_r = a.alpha_r;
  p.alpha_i = a.alpha_i;
  p.beta_r = a.beta_r;
  p.beta_i = a.beta_i;
  p.lo_scale_inv = (kind == SplitKind::fp16) ? (1.f / 2048.f) : 1.f;
  p.is_complex = a.is_complex ? 1 : 0;
  p.dyn = a.dyn;
  p.status = a.dev_status;
  p.debug = a.debug;
  {
    const int v = a.tuning.drain_chunk;
    // Default: two stages (128 FP16 / 64 TF32 k values) per drain.  Measured at m=n=k=16384,
    // uniform(-1,1): residual 3.1e-7 / 2.8e-7 / 3.7e-7 / 6.5e-7 / 2.5e-6 / 1.9e-5 for 1 / 2 / 4 /
    // 8 / 32 / 256 stages per drain (FP32 cuBLAS SGEMM on the same inputs: 2.3e-6).
    p.drain_chunk = static_cast<uint16_t>((v >= 1) ? (v > 0xffff ? 0xffff : v) : 2);
    // The first chunk of every tile is longer: while it accumulates, the epilogue warps are
    // still storing the previous tile, and the issuer would otherwise wait about 17,000 cycles
    // per tile for them to drain a short first chunk (measured: 5 % of a tile at k=16384, 18 %
    // at k=4096).  Its length is bounded by accuracy: the tensor core's own accumulation loses
    // about 1.2e-9 relative accuracy per accumulated k value, and the first chunk's share of
    // the result is sqrt(first / k), so the result stays as close to the FP64 product as with
    // short chunks only if first^1.5 <= ~80 sqrt(k).  Measured residuals (FP16TCEC, m=n=4096,
    // FP32 cuBLAS in brackets): k=512 with 128 / 256 / 512 values in the first chunk 2.0e-7 /
    // 2.8e-7 / 6.5e-7 (4.1e-7); k=4096 with 256 / 512: 2.3e-7 / 3.1e-7 (1.2e-6); k=16384 with
    // 128 / 512 / 1024: 2.8e-7 / 3.0e-7 / 4.2e-7 (2.3e-6).  TF32 products carry more bits into
    // the accumulator and lose twice as much, so that kind gets half the length.
    const uint32_t k_per_stage = ROW_BYTES / es;
    const uint32_t k_total = p.k_blocks * k_per_stage;
    uint32_t first_k = (k_total >= 8192u) ? 512u : (k_total >= 2048u ? 256u : 128u);
    if (kind != SplitKind::fp16) first_k /= 2u;
    const int fv = a.tuning.first_chunk;
    const uint32_t first = (fv >= 1) ? static_cast<uint32_t>(fv) : first_k / k_per_stage;
    p.first_chunk = static_cast<uint16_t>(first > 0xffffu ? 0xffffu : first);
    if (p.first_chunk < p.drain_chunk) p.first_chunk = p.drain_chunk;
  }
  const uint64_t total = static_cast<uint64_t>(p.tiles_m) * p.tiles_n * a.batch;
  if (total == 0 || total > 0x7fffffffull) return false;
  if (a.rows_pad_a < p.tiles_m * 2 * BM_CTA || a.rows_pad_b < p.tiles_n * BN_PAIR) return false;
  p.total_tiles = static_cast<uint32_t>(total);
  p.wave_counter = nullptr;
  return true;
}

// Plan of the tail split (see PairTail) for a launch on at most `max_clusters` clusters.  A
// slice keeps at least 1024 k values, so that a slice's prologue and drain stay amortised.
PairTail plan_tail(const TcecGemmArgs &a, SplitKind kind, const GemmKernelParams &p,
                   uint32_t max_clusters) {
  PairTail t;
  t.partial = nullptr;
  t.counters = nullptr;
  t.split_begin = p.total_tiles;
  t.slices = 1;
  t.slice_blocks = p.k_blocks;
  t.work_items = p.total_tiles;
  if (a.tail_partial == nullptr || a.wave_counter == nullptr || a.tuning.tail_split == 0) return t;
  const uint32_t rem = p.total_tiles % max_clusters;
  if (rem == 0 || 2 * rem > max_clusters || 2 * rem > static_cast<uint32_t>(kPairTailCounters))
    return t;
  const uint32_t k_per_stage = ROW_BYTES / ((kind == SplitKind::fp16) ? 2u : 4u);
  const uint32_t min_stages = 1024u / k_per_stage;
  uint32_t slices = max_clusters / rem;
  if (slices > p.k_blocks / min_stages) slices = p.k_blocks / min_stages;
  if (slices > 8u) slices = 8u;
  if (a.tuning.tail_split > 1 && slices > static_cast<uint32_t>(a.tuning.tail_split))
    slices = static_cast<uint32_t>(a.tuning.tail_split);
  if (slices < 2u) return t;
  const uint32_t per = (p.k_blocks + slices - 1) / slices;
  slices = (p.k_blocks + per - 1) / per; // no empty slice
  if (slices < 2u) return t;
  t.partial = a.tail_partial;
  t.counters = a.wave_counter + 1;
  t.split_begin = p.total_tiles - rem;
  t.slices = slices;
  t.slice_blocks = per;
  t.work_items = t.split_begin + rem * slices;
  return t;
}

// Pacing pays when tiles are long (the drift it removes is 2 % of a tile) and clusters share
// panel rows; for short tiles a barrier per tile costs more than it saves.
bool wants_pacing(const TcecGemmArgs &a, uint32_t clusters, const GemmKernelParams &p,
                  const PairTail &t) {
  return a.wave_counter != nullptr && t.work_items > clusters && p.k_blocks >= kPaceMinStages &&
         a.tuning.pace != 0;
}

// The wave counter and the tail-split counters behind it start every launch at zero.
cudaError_t reset_counters(const TcecGemmArgs &a, bool tail, cudaStream_t stream) {
  return cudaMemsetAsync(a.wave_counter, 0,
                         sizeof(unsigned int) * (tail ? 1 + kPairTailCounters : 1), stream);
}

template <int KIND> cudaError_t launch_pair(const TcecGemmArgs &a, cudaStream_t stream) {
  auto kernel = tcec_gemm_pair_kernel<KIND>;
  int max_clusters = 1;
  const cudaError_t se = pair_setup<KIND>(kernel, &max_clusters);
  if (se != cudaSuccess) return se;
  constexpr SplitKind kind = KIND == 0 ? SplitKind::fp16 : SplitKind::tf32;
  CUtensorMap map_a, map_b;
  GemmKernelParams p;
  if (!pair_prepare(a, kind, &map_a, &map_b, &p)) return cudaErrorInvalidValue;
  const PairTail tail = plan_tail(a, kind, p, static_cast<uint32_t>(max_clusters));
  const uint32_t clusters =
      tail.work_items < static_cast<uint32_t>(max_clusters) ? tail.work_items : max_clusters;
  const bool pace = wants_pacing(a, clusters, p, tail);
  if (pace) p.wave_counter = a.wave_counter;
  if (pace || tail.slices > 1) {
    const cudaError_t me = reset_counters(a, tail.slices > 1, stream);
    if (me != cudaSuccess) return me;
  }
  kernel<<<2 * clusters, NUM_THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p, tail);
  return cudaGetLastError();
}

} // namespace

cudaError_t launch_tcec_gemm_pair(const TcecGemmArgs &a, cudaStream_t stream) {
  if (!a.error_correction) return cudaErrorInvalidValue;
  return (a.kind == SplitKind::fp16) ? launch_pair<0>(a, stream) : launch_pair<1>(a, stream);
}

cudaError_t launch_tcec_gemm_pair_auto(const TcecGemmArgs &a, cudaStream_t stream) {
  if (!a.error_correction || a.dyn == nullptr) return cudaErrorInvalidValue;
  auto kernel = tcec_gemm_pair_auto_kernel;
  int max_clusters = 1;
  const cudaError_t se = pair_setup<2>(kernel, &max_clusters);
  if (se != cudaSuccess) return se;
  CUtensorMap a16, b16, a32, b32;
  GemmKernelParams p16, p32;
  if (!pair_prepare(a, SplitKind::fp16, &a16, &b16, &p16) ||
      !pair_prepare(a, SplitKind::tf32, &a32, &b32, &p32))
    return cudaErrorInvalidValue;
  const PairTail t16 = plan_tail(a, SplitKind::fp16, p16, static_cast<uint32_t>(max_clusters));
  const PairTail t32 = plan_tail(a, SplitKind::tf32, p32, static_cast<uint32_t>(max_clusters));
  // one grid for whichever kind runs: the larger of the two work lists, capped at what fits
  uint32_t clusters = t16.work_items > t32.work_items ? t16.work_items : t32.work_items;
  if (clusters > static_cast<uint32_t>(max_clusters)) clusters = max_clusters;
  // pacing depends on the K loop length, which differs by kind: one counter serves whichever runs
  const bool pace16 = wants_pacing(a, clusters, p16, t16), pace32 = wants_pacing(a, clusters, p32, t32);
  if (pace16) p16.wave_counter = a.wave_counter;
  if (pace32) p32.wave_counter = a.wave_counter;
  const bool tail = t16.slices > 1 || t32.slices > 1;
  if (pace16 || pace32 || tail) {
    const cudaError_t me = reset_counters(a, tail, stream);
    if (me != cudaSuccess) return me;
  }
  kernel<<<2 * clusters, NUM_THREADS, SMEM_BYTES, stream>>>(a16, b16, p16, a32, b32, p32, t16, t32);
  return cudaGetLastError();
}

} // namespace cumpsgemm_b200

extern "C" int cuMpSGEMM_plan_pair_tail(unsigned total_tiles, unsigned clusters, unsigned k_pad,
                                        int tf32, unsigned *split_begin, unsigned *slices,
                                        unsigned *slice_k, unsigned *work_items) {
  using namespace cumpsgemm_b200;
  if (total_tiles == 0 || clusters == 0 || k_pad == 0 || k_pad % 64 != 0 ||
      split_begin == nullptr || slices == nullptr || slice_k == nullptr || work_items == nullptr)
    return 1;
  const SplitKind kind = tf32 ? SplitKind::tf32 : SplitKind::fp16;
  const unsigned k_per_stage = ROW_BYTES / (tf32 ? 4u : 2u);
  // the plan only looks at whether scratch and counters exist, never at their contents
  static float scratch_marker;
  static unsigned int counter_marker[2];
  TcecGemmArgs a = {};
  a.tail_partial = &scratch_marker;
  a.wave_counter = counter_marker;
  a.tuning = Tuning{};
  GemmKernelParams p = {};
  p.total_tiles = total_tiles;
  p.k_blocks = k_pad / k_per_stage;
  const PairTail t = plan_tail(a, kind, p, clusters);
  *split_begin = t.split_begin;
  *slices = t.slices;
  *slice_k = t.slice_blocks * k_per_stage;
  *work_items = t.work_items;
  return 0;
}
