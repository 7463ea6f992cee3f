// What the two MXFP8 GEMM kernels (single CTAs: gemm_mxfp8.cu, CTA pairs: gemm_mxfp8_2sm.cu) share.
#pragma once
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace wk {

struct TileCoord {
  int m_blk, n_blk;
};
// Tiles in groups of `group_m` rows of tiles, M fastest inside a group: the CTAs that run at the same time share
// their operand rows in L2.
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int group_m) {
  const int per_group = group_m * num_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gsz = min(group_m, num_m - first_m);
  const int local = tile - g * per_group;
  TileCoord c;
  c.m_blk = first_m + local % gsz;
  c.n_blk = local / gsz;
  return c;
}

struct GemmParams {
  void* out;
  const uint8_t* sfa;   // swizzled atoms [M/128][K/128][512]
  const uint8_t* sfb;   // swizzled atoms [N/128][K/128][512]
  Epilogue epi;         // scales, accumulate, activation, MXFP8 copy
  int M, N, K;
  int group_m;
  int* status;
};

// the CTA-pair kernel; a and b as the caller passed them, p filled in; `after_retile`: a kernel that re-tiles scales
// was just enqueued, and this launch may start under its tail
int launch_gemm_mxfp8_2sm(const void* a, const void* b, const GemmParams& p, cudaStream_t stream, bool after_retile);

}  // namespace wk
