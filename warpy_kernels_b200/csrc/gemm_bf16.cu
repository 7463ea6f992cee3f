// BF16 GEMM for sm_100a: out[M,N] = a[M,K] . b[N,K]^T, fp32 accumulation in tensor
// memory, bf16 output.
//
// Persistent, warp-specialised CTA (one per SM), 128 x 256 output tile:
//   warp 0      TMA producer: A (128 x 64) and B (256 x 64) bf16 tiles, 128-byte
//               swizzle, into a 4-stage shared-memory ring (48 KiB per stage)
//   warp 1      allocates 512 TMEM columns and issues tcgen05.mma kind::f16
//               (M128 N256 K16, four per stage); two 256-column accumulators so the
//               epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-5   epilogue: tcgen05.ld (32 lanes x 32 columns), fp32 -> bf16, 64-byte
//               row segments straight to global memory
// Tiles are visited in groups of `group_m` row blocks that sweep all column blocks
// (the reference's L2-friendly order, warpy_kernels/utils/sched.py:8-16).
//
// Tensor-core bound: 2*M*N*K flops per launch.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "host_common.h"

namespace wk {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // 64 rows x 64 K elements of a transposed operand
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;

struct TileCoord {
  int m_blk, n_blk;
};
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

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 void* __restrict__ out, int M, int N, int K, int group_m, int in_f16, int a_trans, int b_trans,
                 const __grid_constant__ Epilogue epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then the TMEM base slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int num_m = M / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, status, WK_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          // An operand stored [rows, K] arrives as one box of `rows` x 64 K elements (K-major tile).  A transposed
          // operand, stored [K, rows], arrives as boxes of 64 K x 64 rows (128 bytes of rows per K line), one per
          // 64 rows, 8 KiB apart: an MN-major tile.
          if (a_trans) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * CHUNK_BYTES, &tmap_a, full_bar(stage), tc.m_blk * BM + 64 * c, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, full_bar(stage), kb * BK, tc.m_blk * BM);
          }
          if (b_trans) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sa + A_BYTES + c * CHUNK_BYTES, &tmap_b, full_bar(stage), tc.n_blk * BN + 64 * c, kb * BK);
          } else {
            tma_load_2d(sa + A_BYTES, &tmap_b, full_bar(stage), kb * BK, tc.n_blk * BN);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t fmt = in_f16 ? 0 : 1;
      const uint32_t idesc = make_idesc(fmt, fmt, a_trans ? 1 : 0, b_trans ? 1 : 0, BM, BN);
      // descriptors of stage 0; a later stage only moves the 16-byte-granular start address field.
      // K-major tile: 8-row groups 1024 bytes apart, 16 K elements = 32 bytes further along a row.
      // MN-major tile: 64-row chunks 8 KiB apart (leading offset), groups of 8 K lines 1024 bytes apart,
      // 16 K elements = 16 lines = 2048 bytes further on.
      const uint64_t a_desc0 = smem_desc_sw128(smem_base, a_trans ? CHUNK_BYTES : 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_base + A_BYTES, b_trans ? CHUNK_BYTES : 16, 1024);
      const uint64_t a_kstep = a_trans ? 2048 / 16 : 32 / 16;
      const uint64_t b_kstep = b_trans ? 2048 / 16 : 32 / 16;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, status, WK_ERR_TIMEOUT_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t step = static_cast<uint64_t>(stage) * (STAGE_BYTES / 16);
          const uint64_t a_desc = a_desc0 + step;
          const uint64_t b_desc = b_desc0 + step;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            mma_f16_ss(d_tmem, a_desc + a_kstep * k, b_desc + b_kstep * k, idesc, (kb | k) != 0);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(tfull_bar(acc));
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are visible to this warp
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const TileCoord tc = tile_coord(tile, num_m, num_n, group_m);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, status, WK_ERR_TIMEOUT_MMA)) break;
      tc_fence_after();
      const int row = tc.m_blk * BM + quad * 32 + lane;
      const float row_scale = epilogue_row_scale(epi, row);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + c * 32, v);
        tc_wait_ld();
        const int col = tc.n_blk * BN + c * 32;
        if (col < N) epilogue_chunk(epi, v, row_scale, row, col, N, out);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// the CTA-pair kernel (gemm_bf16_2sm.cu)
int launch_gemm_16bit_2sm(const void* a, const void* b, void* out, int m, int n, int k, int group_m, int f16, int a_trans,
                          int b_trans, const Epilogue& e, int* status, cudaStream_t stream);
}  // namespace wk

extern "C" int wk_gemm_16bit(const wk_gemm16_args* g, void* stream) {
  using namespace wk;
  if (!g) return WK_E_ARG;
  const int m = g->m, n = g->n, k = g->k;
  if (m < 0 || n < 0 || k < 0 || m % BM || n % 128 || k % BK) return WK_E_ARG;
  if (m == 0 || n == 0) return 0;
  if (k == 0) return WK_E_ARG;
  if (!g->a || !g->b || !g->out || !aligned16(g->a) || !aligned16(g->b) || !aligned16(g->out)) return WK_E_ARG;
  if (g->act < 0 || g->act > 2 || (g->act == ACT_DGELU && !g->pre_in)) return WK_E_ARG;
  if ((g->pre_out && !aligned16(g->pre_out)) || (g->pre_in && !aligned16(g->pre_in))) return WK_E_ARG;
  if (g->scale_b && g->scale_b_cols && !aligned16(g->scale_b)) return WK_E_ARG;
  if ((g->q_mx != nullptr) != (g->s_mx != nullptr) || (g->q_mx && !aligned16(g->q_mx))) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;

  const CUtensorMapDataType dt = g->f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap ta, tb;
  // [rows, K] operand: boxes of `tile_rows` x 64 K; transposed ([K, rows]): boxes of 64 K lines x 64 rows
  auto encode_operand = [&](CUtensorMap* t, const void* ptr, int rows, int tile_rows, int trans) {
    if (trans) {
      const uint64_t dims[2] = {static_cast<uint64_t>(rows), static_cast<uint64_t>(k)};
      const uint64_t strides[1] = {static_cast<uint64_t>(rows) * 2};
      const uint32_t box[2] = {64, BK};
      return encode_tmap(t, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(tile_rows)};
    return encode_tmap(t, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (int r = encode_operand(&ta, g->a, m, BM, g->a_trans)) return r;
  if (int r = encode_operand(&tb, g->b, n, BN, g->b_trans)) return r;
  Epilogue e;
  e.scale_a = g->scale_a;
  e.scale_b = g->scale_b;
  e.scale_a_rows = g->scale_a_rows;
  e.scale_b_cols = g->scale_b_cols;
  e.accum = g->accum;
  e.act = g->act;
  e.out_f16 = g->f16;
  e.pre_out = g->pre_out;
  e.pre_in = g->pre_in;
  e.q_mx = static_cast<uint8_t*>(g->q_mx);
  e.s_mx = static_cast<uint8_t*>(g->s_mx);
  // cta_pair: 1 the CTA-pair kernel, 2 this file's kernel, 0 whichever should finish
  // first: a pair works through a 256 x 256 tile about 10 % faster than two SMs through two 128 x 256 tiles
  // (1.53 against 1.40 PFLOP/s at 8192^3), but a small problem fills 148 SMs better with the smaller tiles
  if (g->cta_pair < 0 || g->cta_pair > 2 || g->group_m < 0) return WK_E_ARG;
  const int group_m = g->group_m ? g->group_m : 8;
  const int sms = sm_count();
  if (sms <= 0) return WK_E_CUDA;
  const int num_tiles = (m / BM) * ((n + BN - 1) / BN);
  bool pair = g->cta_pair == 1;
  if (g->cta_pair == 0 && sms >= 2) {
    const long pair_tiles = static_cast<long>((m + 255) / 256) * ((n + 255) / 256);
    const long pair_waves = (pair_tiles + sms / 2 - 1) / (sms / 2);
    const long single_waves = (num_tiles + sms - 1) / sms;
    // a pair finishes its tile in the time of a single-CTA tile less 10 %; below two waves of pairs the shorter
    // start-up of the single-CTA kernel wins (measured: 2048^3 0.63 against 0.69 PFLOP/s, 3072^3 equal)
    pair = pair_tiles > sms && pair_waves * 10 < single_waves * 11;
  }
  if (pair) {
    return launch_gemm_16bit_2sm(g->a, g->b, g->out, m, n, k, group_m, g->f16, g->a_trans, g->b_trans, e, status,
                                 static_cast<cudaStream_t>(stream));
  }
  if (allow_smem(reinterpret_cast<const void*>(gemm_bf16_kernel), SMEM_BYTES)) return WK_E_CUDA;
  const int grid = num_tiles < sms ? num_tiles : sms;
  gemm_bf16_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(ta, tb, g->out, m, n, k, group_m,
                                                                                     g->f16, g->a_trans, g->b_trans, e, status);
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}

extern "C" int wk_gemm_bf16(const void* a, const void* b, void* out, int m, int n, int k, void* stream) {
  wk_gemm16_args g = {};
  g.a = a;
  g.b = b;
  g.out = out;
  g.m = m;
  g.n = n;
  g.k = k;
  return wk_gemm_16bit(&g, stream);
}
