// MXFP8 block-scaled GEMM on CTA pairs (tcgen05 cta_group::2); the product and the epilogue of gemm_mxfp8.cu.
//
// Two CTAs of a cluster share one 256 x 256 output tile.  Per stage of 128 K elements each CTA loads its own 128 rows
// of A and its own 128 of the tile's 256 rows of B (32 KiB instead of the 48 of the single-CTA kernel), its own
// scale-factor atom of A and BOTH atoms of B: an SM's tensor core scales all 256 columns of its accumulator rows, and
// it reads the scale factors from its own tensor memory.  The even CTA copies the atoms into both tensor memories
// (tcgen05.cp.cta_group::2 reads each CTA's shared memory at the same offset) and issues four
// tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale (M256 N256 K32) per stage.
//
// The scale atoms are fetched as TMA tiles (one 512-byte line each), not as plain bulk copies: only the TMA form
// can count its bytes on the other CTA's barrier.  The "full" barrier of a stage lives in the even CTA and takes one
// arrival, from the even CTA's producer, which announces the bytes of both CTAs (pair.cuh says why).
//
// Tensor memory as in the single-CTA kernel: two 256-column accumulators that share 64 columns, the epilogue drains
// the shared columns of a tile first; four scale-factor slots of 12 columns from column 448 on, used in turn.
//
// Measured on B200: within 3 % of the single-CTA kernel either way (2.2-2.4 PFLOP/s at 8192 x 14336 x 4096 and
// 8192^3, 8 % behind at 4096^3), so wk_gemm_mxfp8 runs it only on request (cta_pair = 1).  What keeps it from the
// gain the 16-bit pair kernel shows: the three tcgen05.cp per stage occupy the tensor pipe (without them: +12 %),
// and the hand-over of the shared accumulator columns crosses the pair once per tile.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_mxfp8.h"
#include "host_common.h"
#include "pair.cuh"

namespace wk {
namespace {

constexpr int Q_BM = 256;  // output rows per CTA pair
constexpr int Q_BN = 256;
constexpr int Q_BK = 128;  // bytes == e4m3 elements
constexpr int Q_STAGES = 6;
constexpr int Q_SF_SLOTS = 4;  // scale-factor slots in tensor memory, used in turn
constexpr int Q_A_BYTES = 128 * Q_BK;  // this CTA's 128 rows of A
constexpr int Q_B_BYTES = 128 * Q_BK;  // this CTA's 128 of the tile's 256 rows of B
constexpr int Q_AB_BYTES = Q_A_BYTES + Q_B_BYTES;
constexpr int Q_SF_ATOM = 512;
constexpr int Q_SF_BYTES = 3 * Q_SF_ATOM;  // A: this CTA's rows; B: all 256 columns
constexpr int Q_STAGE_TX = Q_AB_BYTES + Q_SF_BYTES;
constexpr int Q_SMEM_BYTES = Q_STAGES * (Q_AB_BYTES + Q_SF_BYTES) + 1024 + 256;
constexpr int Q_THREADS = 192;
constexpr int Q_TMEM_COLS = 512;
constexpr int Q_ACC_STRIDE = 192;   // accumulator slot a lives in columns [192 a, 192 a + 256)
constexpr int Q_SF_COL = 448;       // scale-factor columns start here
constexpr int Q_SF_SLOT_COLS = 12;  // 4 (A: 128 rows) + 8 (B: 256 columns)
static_assert(Q_SF_COL + Q_SF_SLOTS * Q_SF_SLOT_COLS <= Q_TMEM_COLS, "scale-factor slots must fit");

__device__ __forceinline__ void mma_mxf8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], "
      "[%5], p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// 32 rows x 16 bytes of shared memory to four 32-lane groups of tensor memory, in both CTAs of the pair
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Q_THREADS, 1)
gemm_mxfp8_2sm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                      const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sf_base = smem_base + Q_STAGES * Q_AB_BYTES;  // the operand stages stay 1024-byte aligned
  const uint32_t bar_base = sf_base + Q_STAGES * Q_SF_BYTES;
  // barriers: full[STAGES] (used in the even CTA), empty[STAGES], tmem_full[2], then in the even CTA tmem_empty[2]
  // and "shared columns drained", then the TMEM base slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Q_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * Q_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * Q_STAGES + 2 + a); };
  const uint32_t ovl_bar = bar_base + 8u * (2 * Q_STAGES + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * Q_STAGES + 5);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs
  const int pair = blockIdx.x / 2;
  const int num_pairs = gridDim.x / 2;
  const int num_m = (p.M + Q_BM - 1) / Q_BM;  // M and N are multiples of 128: the last tile may be half outside,
  const int num_n = (p.N + Q_BN - 1) / Q_BN;  // where the loads read zeros and the epilogue stores nothing
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K / Q_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the even CTA's producer, which announces the bytes of both CTAs
      mbar_init(empty_bar(s), 1);  // the pair's commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // four epilogue warps in each CTA
    }
    mbar_init(ovl_bar, 8);
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_sfa);
    prefetch_tmap(&tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Q_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the other CTA's barriers are initialised before anybody signals them
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      pdl_wait();  // the launch may overlap the end of the kernel that re-tiles the scales: load nothing before it is done
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m);
        const int a_rows = tc.m_blk * 2 + rank;  // in units of 128 rows
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * Q_AB_BYTES;
          const uint32_t ssf = sf_base + stage * Q_SF_BYTES;
          const uint32_t full0 = mapa(full_bar(stage), 0);
          // the other CTA's bytes may land before this announcement: the count just goes negative meanwhile
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * Q_STAGE_TX);
          tma_load_2d_pair(sa, &tmap_a, full0, kb * Q_BK, a_rows * 128);
          tma_load_2d_pair(sa + Q_A_BYTES, &tmap_b, full0, kb * Q_BK, tc.n_blk * Q_BN + 128 * rank);
          // a block of 128 rows that lies outside the matrix reads as zeros, like the operand rows themselves
          tma_load_3d_pair(ssf, &tmap_sfa, full0, 0, kb, a_rows);
          tma_load_3d_pair(ssf + Q_SF_ATOM, &tmap_sfb, full0, 0, kb, tc.n_blk * 2);
          tma_load_3d_pair(ssf + 2 * Q_SF_ATOM, &tmap_sfb, full0, 0, kb, tc.n_blk * 2 + 1);
          if (++stage == Q_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // descriptors of stage 0 (the same offsets hold in the other CTA); a later stage only moves the
      // 16-byte-granular start address field
      const uint64_t a_desc0 = smem_desc_sw128(smem_base, 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_base + Q_A_BYTES, 16, 1024);
      const uint64_t sf_desc0 = smem_desc_plain(sf_base, 16, 128);
      // The scale factors of a stage are copied to tensor memory one stage ahead of the MMAs that read them: a
      // tcgen05.cp issued right in front of its MMAs holds them up (12 % of the kernel's time, measured), one
      // issued a stage earlier runs beside the MMAs of the stage before.
      int stage = 0, cp_stage = 0, slot = 0, cp_slot = 0;
      uint32_t phase = 0, cp_phase = 0;
      bool ok = true;
      const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
      const long total_kb = static_cast<long>(my_tiles) * num_kb;
      auto copy_scales = [&]() {  // waits for the next stage's bytes and sends its scale factors on their way
        if (!mbar_wait(full_bar(cp_stage), cp_phase, p.status, WK_ERR_TIMEOUT_LOAD)) return false;
        tc_fence_after();
        const uint64_t sf_desc = sf_desc0 + static_cast<uint64_t>(cp_stage) * (Q_SF_BYTES / 16);
        // the slot was last read by the MMAs four stages back; tcgen05 operations of one thread run in issue order
        const uint32_t sf_tmem = tmem_base + Q_SF_COL + cp_slot * Q_SF_SLOT_COLS;
        cp_slot = (cp_slot + 1) & (Q_SF_SLOTS - 1);
        tmem_cp_32x128b_warpx4_pair(sf_tmem + 0, sf_desc);
        tmem_cp_32x128b_warpx4_pair(sf_tmem + 4, sf_desc + Q_SF_ATOM / 16);
        tmem_cp_32x128b_warpx4_pair(sf_tmem + 8, sf_desc + 2 * Q_SF_ATOM / 16);
        if (++cp_stage == Q_STAGES) {
          cp_stage = 0;
          cp_phase ^= 1;
        }
        return true;
      };
      long it = 0;
      if (total_kb > 0) ok = copy_scales();
      for (int local = 0; ok && local < my_tiles; ++local) {
        const int acc = local & 1;
        // this slot was drained two tiles ago, and the previous tile has given up the columns it shares
        if (!mbar_wait_cluster(tempty_bar(acc), ((local >> 1) & 1) ^ 1, p.status, WK_ERR_TIMEOUT_TMEM)) break;
        if (local > 0 && !mbar_wait_cluster(ovl_bar, (local - 1) & 1, p.status, WK_ERR_TIMEOUT_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Q_ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          if (it + 1 < total_kb && !copy_scales()) {
            ok = false;
            break;
          }
          const uint64_t ab_step = static_cast<uint64_t>(stage) * (Q_AB_BYTES / 16);
          const uint32_t sf_tmem = tmem_base + Q_SF_COL + slot * Q_SF_SLOT_COLS;
          slot = (slot + 1) & (Q_SF_SLOTS - 1);
#pragma unroll
          for (int k = 0; k < Q_BK / 32; ++k) {
            mma_mxf8_ss_pair(d_tmem, a_desc0 + ab_step + 2 * k, b_desc0 + ab_step + 2 * k,
                             make_idesc_mx(Q_BM, Q_BN, k, k), sf_tmem, sf_tmem + 4, (kb | k) != 0);
          }
          // the stage is free in both CTAs once these MMAs have read it: one commit per CTA
          tc_commit_pair(mapa(empty_bar(stage), 0));
          tc_commit_pair(mapa(empty_bar(stage), 1));
          if (++stage == Q_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          tc_commit_pair(mapa(tfull_bar(acc), 0));
          tc_commit_pair(mapa(tfull_bar(acc), 1));
        }
      }
      (void)phase;
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are visible to this warp
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m);
      const int acc = local & 1;
      if (!mbar_wait_warp(tfull_bar(acc), (local >> 1) & 1, p.status, WK_ERR_TIMEOUT_MMA)) break;
      tc_fence_after();
      // column chunks in the order they are drained: the 64 columns shared with the other slot first
      const int first_chunk = acc == 0 ? 6 : 0;
      const int row = tc.m_blk * Q_BM + 128 * rank + quad * 32 + lane;
      const bool row_ok = row < p.M;  // the same for the whole CTA
      const float row_scale = row_ok ? epilogue_row_scale(p.epi, row) : 0.f;
#pragma unroll 1
      for (int ci = 0; ci < Q_BN / 32; ++ci) {
        const int c = (ci + first_chunk) & 7;
        const int col = tc.n_blk * Q_BN + c * 32;
        const bool store = row_ok && col < p.N;
        uint32_t v[32];
        if (store) {
          tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * Q_ACC_STRIDE + c * 32, v);
          tc_wait_ld();
        }
        if (ci == 1) {
          // both shared chunks are in registers (or not wanted): the next tile's main loop may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa(ovl_bar, 0));
        }
        if (store) epilogue_chunk(p.epi, v, row_scale, row, col, p.N, p.out);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // nobody leaves while the other CTA may still signal this one's barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Q_TMEM_COLS);
  }
}

}  // namespace

// Launches the CTA-pair kernel.  The caller has checked the arguments (M and N multiples of 128, K of 128) and
// re-tiled the scale factors into p.sfa / p.sfb.
int launch_gemm_mxfp8_2sm(const void* a, const void* b, const GemmParams& p, cudaStream_t stream, bool after_retile) {
  CUtensorMap ta, tb, tsa, tsb;
  const uint32_t box[2] = {Q_BK, 128};
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(p.K)};
    if (int r = encode_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return r;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(p.K)};
    if (int r = encode_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return r;
  }
  // the re-tiled scale factors as [rows / 128][K / 128] lines of 512 bytes (128 32-bit words)
  const uint64_t num_kb = static_cast<uint64_t>(p.K / Q_BK);
  const uint32_t sf_box[3] = {Q_SF_ATOM / 4, 1, 1};
  const uint64_t sf_strides[2] = {Q_SF_ATOM, Q_SF_ATOM * num_kb};
  {
    const uint64_t dims[3] = {Q_SF_ATOM / 4, num_kb, static_cast<uint64_t>(p.M / 128)};
    if (int r = encode_tmap(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.sfa, dims, sf_strides, sf_box,
                            CU_TENSOR_MAP_SWIZZLE_NONE))
      return r;
  }
  {
    const uint64_t dims[3] = {Q_SF_ATOM / 4, num_kb, static_cast<uint64_t>(p.N / 128)};
    if (int r = encode_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.sfb, dims, sf_strides, sf_box,
                            CU_TENSOR_MAP_SWIZZLE_NONE))
      return r;
  }
  if (allow_smem(reinterpret_cast<const void*>(gemm_mxfp8_2sm_kernel), Q_SMEM_BYTES)) return WK_E_CUDA;
  const int sms = sm_count();
  if (sms < 2) return WK_E_CUDA;
  const int num_tiles = ((p.M + Q_BM - 1) / Q_BM) * ((p.N + Q_BN - 1) / Q_BN);
  const int max_pairs = sms / 2;
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(Q_THREADS);
  cfg.dynamicSmemBytes = Q_SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = after_retile ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_mxfp8_2sm_kernel, ta, tb, tsa, tsb, p) == cudaSuccess ? 0 : WK_E_CUDA;
}

}  // namespace wk
