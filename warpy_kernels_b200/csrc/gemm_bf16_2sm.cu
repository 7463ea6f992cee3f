// BF16 / FP16 GEMM on CTA pairs (tcgen05 cta_group::2): out[M,N] = a[M,K] . b[N,K]^T.
//
// Two CTAs of a cluster (two neighbouring SMs) share one 256 x 256 output tile.  Each CTA loads its own 128 rows
// of A and its own 128 of the tile's 256 rows of B (32 KiB per stage instead of 48), the even CTA issues one
// tcgen05.mma.cta_group::2 (M256 N256 K16) per K step for both, and each CTA's tensor memory holds the
// accumulator rows of its own half of M.  Against the single-CTA kernel (gemm_bf16.cu) a pair reads a third less
// shared memory per flop and a quarter less from L2 / DRAM.  Measured at 8192^3: 1.50-1.54 PFLOP/s against 1.40 of
// the single-CTA kernel, bit-identical results.
// The "full" barrier of a stage lives in the even CTA and takes ONE arrival: the even CTA's producer announces the
// bytes of both CTAs, and the odd CTA's loads just complete against it (its bytes may land first; the count goes
// negative meanwhile).  An announcement sent from the odd CTA instead (a remote mbarrier.arrive.expect_tx) held
// its producer for about a thousand cycles per stage and capped the kernel at 0.76-1.2 PFLOP/s.
//   warp 0      TMA producer in both CTAs; its loads signal the even CTA's "full" barrier
//   warp 1      both: tensor-memory allocation for the pair; even CTA only: MMA issue; its commits release the
//               stage in both CTAs and announce the finished accumulator to both
//   warps 2-5   epilogue in both CTAs (the fused epilogue of gemm_epilogue.cuh), then they hand the accumulator
//               back to the even CTA
// Every wait is bounded (common.cuh); the two cluster-wide barriers at start and end are plain hardware barriers
// that both CTAs always reach.
//
// Reached through wk_gemm_16bit (cta_pair = 1, or 0 when the pairs fill the GPU better); operands row-major or
// transposed, M and N multiples of 128 and K of 64 as there.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "host_common.h"
#include "pair.cuh"

namespace wk {
namespace {

constexpr int P_BM = 256;  // output rows per CTA pair
constexpr int P_BN = 256;
constexpr int P_BK = 64;  // one 128-byte swizzle span per row
constexpr int P_STAGES = 7;
constexpr int P_CHUNK_BYTES = 128 * 64 * 2;    // 128 rows x 64 K elements (one swizzle span)
constexpr int P_CHUNKS = P_BK / 64;            // swizzle spans per row of a stage
constexpr int P_T_CHUNK_BYTES = 64 * P_BK * 2; // 64 K lines x 64 rows of a transposed operand
constexpr int P_A_BYTES = P_CHUNKS * P_CHUNK_BYTES;   // this CTA's 128 rows of A
constexpr int P_B_BYTES = P_CHUNKS * P_CHUNK_BYTES;   // this CTA's 128 of the tile's 256 rows of B
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int P_THREADS = 192;
constexpr int P_TMEM_COLS = 512;

struct PairTile {
  int m_blk, n_blk;
};
__device__ __forceinline__ PairTile pair_tile(int tile, int num_m, int num_n, int group_m) {
  const int per_group = group_m * num_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gsz = min(group_m, num_m - first_m);
  const int local = tile - g * per_group;
  PairTile c;
  c.m_blk = first_m + local % gsz;
  c.n_blk = local / gsz;
  return c;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     void* __restrict__ out, int M, int N, int K, int group_m, int in_f16, int a_trans, int b_trans,
                     const __grid_constant__ Epilogue epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + P_STAGES * P_STAGE_BYTES;
  // barriers: full[STAGES] (used in the even CTA), empty[STAGES], tmem_full[2], tmem_empty[2] (used in the even
  // CTA), then the TMEM base slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (P_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * P_STAGES + 4);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs
  const int pair = blockIdx.x / 2;
  const int num_pairs = gridDim.x / 2;
  const int num_m = (M + P_BM - 1) / P_BM;  // M and N are multiples of 128: the last tile may be half outside,
  const int num_n = (N + P_BN - 1) / P_BN;  // where the loads read zeros and the epilogue stores nothing
  const int num_tiles = num_m * num_n;
  const int num_kb = K / P_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the even CTA's producer, which announces the bytes of both CTAs
      mbar_init(empty_bar(s), 1);  // the pair's commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // four epilogue warps in each CTA
    }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, P_TMEM_COLS);
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
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        const PairTile tc = pair_tile(tile, num_m, num_n, group_m);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, status, WK_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }

          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          const uint32_t full0 = mapa(full_bar(stage), 0);
          // the other CTA's bytes may land before this announcement: the count just goes negative meanwhile
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);
          // An operand stored [rows, K] arrives as one box of 128 rows x 64 K elements (K-major tile).  A transposed
          // operand, stored [K, rows], arrives as two boxes of 64 K lines x 64 rows (128 bytes of rows per K line),
          // 8 KiB apart: an MN-major tile.
          const int a_row = tc.m_blk * P_BM + 128 * rank, b_row = tc.n_blk * P_BN + 128 * rank;
          if (a_trans) {
            tma_load_2d_pair(sa, &tmap_a, full0, a_row, kb * P_BK);
            tma_load_2d_pair(sa + P_T_CHUNK_BYTES, &tmap_a, full0, a_row + 64, kb * P_BK);
          } else {
            tma_load_2d_pair(sa, &tmap_a, full0, kb * P_BK, a_row);
          }
          if (b_trans) {
            tma_load_2d_pair(sa + P_A_BYTES, &tmap_b, full0, b_row, kb * P_BK);
            tma_load_2d_pair(sa + P_A_BYTES + P_T_CHUNK_BYTES, &tmap_b, full0, b_row + 64, kb * P_BK);
          } else {
            tma_load_2d_pair(sa + P_A_BYTES, &tmap_b, full0, kb * P_BK, b_row);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t fmt = in_f16 ? 0 : 1;
      const uint32_t idesc = make_idesc(fmt, fmt, a_trans ? 1 : 0, b_trans ? 1 : 0, P_BM, P_BN);
      // descriptors of stage 0 (the same offsets hold in the other CTA); a later stage only moves the
      // 16-byte-granular start address field
      // K-major tile: 16 elements of K = 32 bytes inside the 128-byte swizzle span.  MN-major tile: the leading
      // byte offset is the distance between the two 64-row chunks, 16 K lines = 2048 bytes.
      const uint64_t a_desc0 = smem_desc_sw128(smem_base, a_trans ? P_T_CHUNK_BYTES : 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_base + P_A_BYTES, b_trans ? P_T_CHUNK_BYTES : 16, 1024);
      const uint64_t a_kstep = a_trans ? 2048 / 16 : 32 / 16;
      const uint64_t b_kstep = b_trans ? 2048 / 16 : 32 / 16;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait_cluster(tempty_bar(acc), acc_phase ^ 1, status, WK_ERR_TIMEOUT_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t step = static_cast<uint64_t>(stage) * (P_STAGE_BYTES / 16);
#pragma unroll
          for (int k = 0; k < P_BK / 16; ++k) {
            mma_f16_ss_pair(d_tmem, a_desc0 + step + k * a_kstep, b_desc0 + step + k * b_kstep, idesc, (kb | k) != 0);
          }
          // the stage is free in both CTAs once these MMAs have read it: one commit per CTA
          tc_commit_pair(mapa(empty_bar(stage), 0));
          tc_commit_pair(mapa(empty_bar(stage), 1));
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          tc_commit_pair(mapa(tfull_bar(acc), 0));
          tc_commit_pair(mapa(tfull_bar(acc), 1));
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are visible to this warp
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const PairTile tc = pair_tile(tile, num_m, num_n, group_m);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, status, WK_ERR_TIMEOUT_MMA)) break;
      tc_fence_after();
      const int row = tc.m_blk * P_BM + 128 * rank + quad * 32 + lane;
      const bool row_ok = row < M;  // the same for the whole CTA
      const float row_scale = row_ok ? epilogue_row_scale(epi, row) : 0.f;
#pragma unroll 1
      for (int c = 0; c < P_BN / 32; ++c) {
        const int col = tc.n_blk * P_BN + c * 32;
        if (!row_ok || col >= N) break;
        uint32_t v[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * P_BN + c * 32, v);
        tc_wait_ld();
        epilogue_chunk(epi, v, row_scale, row, col, N, out);
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
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

}  // namespace

// Launches the CTA-pair kernel.  The caller has checked the arguments; M and N are multiples of 128, K of 64.
int launch_gemm_16bit_2sm(const void* a, const void* b, void* out, int m, int n, int k, int group_m, int f16, int a_trans,
                          int b_trans, const Epilogue& e, int* status, cudaStream_t stream) {
  const CUtensorMapDataType dt = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap ta, tb;
  // [rows, K] operand: boxes of 128 rows x 64 K; transposed ([K, rows]): boxes of 64 K lines x 64 rows
  auto encode_operand = [&](CUtensorMap* t, const void* ptr, int rows, int trans) {
    if (trans) {
      const uint64_t dims[2] = {static_cast<uint64_t>(rows), static_cast<uint64_t>(k)};
      const uint64_t strides[1] = {static_cast<uint64_t>(rows) * 2};
      const uint32_t box[2] = {64, P_BK};
      return encode_tmap(t, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
    const uint32_t box[2] = {P_BK, 128};
    return encode_tmap(t, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (int r = encode_operand(&ta, a, m, a_trans)) return r;
  if (int r = encode_operand(&tb, b, n, b_trans)) return r;
  if (allow_smem(reinterpret_cast<const void*>(gemm_bf16_2sm_kernel), P_SMEM_BYTES)) return WK_E_CUDA;
  const int sms = sm_count();
  if (sms <= 0) return WK_E_CUDA;
  const int num_tiles = ((m + P_BM - 1) / P_BM) * ((n + P_BN - 1) / P_BN);
  const int max_pairs = sms / 2;
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  gemm_bf16_2sm_kernel<<<2 * pairs, P_THREADS, P_SMEM_BYTES, stream>>>(ta, tb, out, m, n, k, group_m, f16, a_trans, b_trans, e,
                                                                        status);
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}

}  // namespace wk
