// Pieces shared by the single-CTA and the CTA-pair TCEC GEMM kernels.
#pragma once
#include "internal.hpp"

#include <cuda.h>

namespace cumpsgemm_b200 {

constexpr int kGemmRowBytes = 128; // K extent of one stage in bytes = one 128-byte swizzle atom

// Kernel arguments besides the two tensor maps.
struct GemmKernelParams {
  // The struct is kept at 128 bytes (checked below): past that size the compiler stops reading
  // the fields straight from the constant bank and goes through a pointer to the parameter
  // instead, reloading them after every store and asm statement (measured: the pair kernel 4 %
  // slower at 4096^3, 20 % slower on short-K batches).  Hence the 16-bit fields at the end.
  float *c;
  float *const *c_array; // pointer-array batches: C of batch b starts at c_array[b] (or null)
  uint64_t ldc;
  uint64_t stride_c;
  const DynParams *dyn;
  int *status;
  // Optional stall breakdown (8 x u64, nullable): cycles the MMA issuer waited for operands [0]
  // and for the accumulator drain [1], the producer for a free stage [2], drain warp 4 for
  // a finished chunk [3]; MMA loop cycles [4]; contributing CTAs [5].
  unsigned long long *debug;
  // Pair kernel, nullable: arrivals of clusters at tile starts (see the kernel's producer).
  unsigned int *wave_counter;
  // Split-K (single-CTA kernel): the K loop of a tile is cut into k_slices pieces of
  // slice_blocks stages, one CTA each (blockIdx.x = tile * k_slices + slice).  With more than
  // one slice a CTA writes its plain partial sum (alpha = 1, beta = 0, no complex arithmetic)
  // to c + slice * slice_stride floats, and a second kernel adds the slices in a fixed order.
  uint64_t slice_stride;
  uint32_t m, n;
  uint32_t k_blocks;
  uint32_t tiles_m, tiles_n;
  float alpha_r, alpha_i, beta_r, beta_i;
  float lo_scale_inv;
  // Pair tiles in the whole launch (tiles_m * tiles_n * batch); the persistent pair kernel
  // walks them with a stride of the number of clusters in the grid.
  uint32_t total_tiles;
  uint32_t slice_blocks;
  uint16_t k_slices;
  // Stages whose hi*hi products accumulate in TMEM before one drain (pair kernel; 1 or 2).
  uint16_t drain_chunk;
  // Stages in the first chunk of every tile (pair kernel; >= drain_chunk).
  uint16_t first_chunk;
  uint16_t is_complex;
};
static_assert(sizeof(GemmKernelParams) <= 128, "see the comment at the top of the struct");

// Tensor map over a K-blocked panel: dims {elements per 128 bytes, rows_pad, planes * k_blocks},
// box {128 bytes of K, box_rows, 1}, 128-byte swizzle; a load's coordinates are
// (0, first row, plane * k_blocks + K block).  Returns false if the driver entry point is unavailable or rejects it.
bool make_panel_map(CUtensorMap *map, SplitKind kind, const void *panel, uint32_t k_pad,
                    uint32_t rows_pad, uint32_t planes, uint32_t box_rows);

// CTA-pair kernel (tcec_gemm_pair.cu): 256 x 256 tile per cluster of two CTAs.
cudaError_t launch_tcec_gemm_pair(const TcecGemmArgs &a, cudaStream_t stream);
cudaError_t launch_tcec_gemm_pair_auto(const TcecGemmArgs &a, cudaStream_t stream);

} // namespace cumpsgemm_b200
