// BF16 flash-attention backward for sm_100a, head dimension 128.
//
//   S = alpha . q k^T,  P = softmax(S) = 2^(S . log2e - L)   (L: the forward's base-2 lse)
//   dV = P^T dO,  dP = dO v^T,  D = rowsum(dO * O),  dS = P * (dP - D),
//   dQ = alpha . dS k,  dK = alpha . dS^T q
// as in the reference's bf16 backward (warpy_kernels/attn/bwd_common.py:88-304, bwd_sm120.py:436-464).  Same three
// kernels and the same pipeline as the FP8 backward (attn_bwd_fp8.cu), with tcgen05.mma kind::f16 and P^T, dS^T
// rounded to bf16 instead of MXFP8:
//
//  1. attn_bwd_prep_kernel: per query row D = sum(dO . O) and the row record (-L, -D).
//  2. attn_bwd_dkdv_kernel: CTA = 128 keys of one (batch, kv head), K and V resident in shared memory, loop over
//     the group's query heads and query tiles; S^T = K Q^T and dP^T = V dO^T into TMEM, threads turn them into
//     bf16 P^T and dS^T back in TMEM, dV += P^T dO and dK += dS^T Q (A from TMEM, B = the same Q / dO tiles read
//     MN-major).  dV and dK stay in TMEM for the whole CTA.
//  3. attn_bwd_dq_kernel: CTA = 128 queries, loop over key tiles, recomputes S and dP, dQ += dS K in TMEM: no
//     atomics, deterministic.
// A row of a tile is 256 bytes, two 128-byte swizzle spans: every tile is two boxes of 64 head-dim elements,
// 16 KiB apart in shared memory.
//
// Tensor-core bound: 10 . B . Hq . Nq . Nk . d flops of algorithmic work (half when causal).
#include <math.h>

#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

constexpr int BM = 128;  // queries per tile
constexpr int BN = 128;  // keys per tile
constexpr int D = 128;  // largest head dimension; with 64 (the main kernels are instantiated per head dimension) a row is one swizzle span instead of
                        // two: the second box of every tile is not loaded and the products take half the K steps
constexpr int CHUNK = 64;                        // head-dim elements per 128-byte swizzle span
constexpr int CHUNK_BYTES = 128 * CHUNK * 2;     // 16 KiB: 128 rows x 128 bytes
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;      // 32 KiB: 128 rows x 256 bytes
constexpr int SF_BYTES = 512;
constexpr int THREADS = 576;          // TMA warp, MMA warp, 16 element-wise warps (four threads per row)
constexpr int HALF_THREADS = 256;     // the element-wise threads of one 64-column half of a tile: two per row
constexpr int HALF_COLS = 64;
constexpr int TMEM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;

// ---------------------------------------------------------------------------
// 1. prep
// ---------------------------------------------------------------------------
struct PrepParams {
  const __nv_bfloat16* dout;  // [B,Hq,Nq,D] with element strides
  const __nv_bfloat16* out;
  const float* lse;           // [B,Hq,*] base 2
  float* qstat;               // [B,Hq,Nq_pad/128][2][128]: per 128 rows the arrays -L and -D
  int64_t do_sb, do_sh, do_sn;
  int64_t o_sb, o_sh, o_sn;
  int64_t lse_sb, lse_sh;
  int B, Hq, Nq, nq_pad, d;
};

// one warp per query row, 4 consecutive elements per lane
__global__ void __launch_bounds__(256) attn_bwd_bf16_prep_kernel(const PrepParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  const int64_t rows = static_cast<int64_t>(p.B) * p.Hq * p.nq_pad;
  if (warp >= rows) return;
  const int i = warp % p.nq_pad;
  const int h = (warp / p.nq_pad) % p.Hq;
  const int b = warp / (p.nq_pad * p.Hq);
  // the two values of row i sit 128 floats apart inside the row's tile of 128
  float* stat = p.qstat + ((static_cast<int64_t>(b) * p.Hq + h) * p.nq_pad + (i & ~127)) * 2 + (i & 127);
  if (i >= p.Nq) {
    // padding rows: lse = +inf makes every probability zero
    if (lane < 2) stat[lane * 128] = lane == 0 ? -INFINITY : 0.f;
    return;
  }
  const __nv_bfloat16* dsrc = p.dout + b * p.do_sb + h * p.do_sh + static_cast<int64_t>(i) * p.do_sn + lane * 4;
  const __nv_bfloat16* osrc = p.out + b * p.o_sb + h * p.o_sh + static_cast<int64_t>(i) * p.o_sn + lane * 4;
  const bool mine = lane * 4 < p.d;  // head dimension 64: half the lanes only join the reduction
  const uint2 draw = mine ? *reinterpret_cast<const uint2*>(dsrc) : make_uint2(0, 0);
  const uint2 oraw = mine ? *reinterpret_cast<const uint2*>(osrc) : make_uint2(0, 0);
  float dsum = __uint_as_float(draw.x << 16) * __uint_as_float(oraw.x << 16) +
               __uint_as_float(draw.x & 0xffff0000u) * __uint_as_float(oraw.x & 0xffff0000u) +
               __uint_as_float(draw.y << 16) * __uint_as_float(oraw.y << 16) +
               __uint_as_float(draw.y & 0xffff0000u) * __uint_as_float(oraw.y & 0xffff0000u);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
  if (lane == 0) {
    stat[0] = -p.lse[b * p.lse_sb + h * p.lse_sh + i];
    stat[128] = -dsum;
  }
}

// The same for tensors whose strides are multiples of 8 elements: four query rows per warp, 8 lanes per row and 16
// consecutive elements per lane, read with 16-byte loads (the kernel is HBM-bound; one row per warp keeps too few
// bytes in flight).
__global__ void __launch_bounds__(256) attn_bwd_bf16_prep4_kernel(const PrepParams p) {
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  const int sub = lane & 7;
  const int64_t rows = static_cast<int64_t>(p.B) * p.Hq * p.nq_pad;  // a multiple of 128
  if (warp * 4 >= rows) return;
  const int64_t row_id = warp * 4 + (lane >> 3);
  const int i = static_cast<int>(row_id % p.nq_pad);
  const int h = static_cast<int>((row_id / p.nq_pad) % p.Hq);
  const int b = static_cast<int>(row_id / (static_cast<int64_t>(p.nq_pad) * p.Hq));
  const bool live = i < p.Nq;  // padding rows take part in the shuffles with zeros
  uint4 draw[2] = {}, oraw[2] = {};
  if (live && sub * 16 < p.d) {  // head dimension 64: half the lanes only join the reduction
    const uint4* dsrc = reinterpret_cast<const uint4*>(p.dout + b * p.do_sb + h * p.do_sh +
                                                       static_cast<int64_t>(i) * p.do_sn + sub * 16);
    const uint4* osrc =
        reinterpret_cast<const uint4*>(p.out + b * p.o_sb + h * p.o_sh + static_cast<int64_t>(i) * p.o_sn + sub * 16);
    draw[0] = dsrc[0];
    draw[1] = dsrc[1];
    oraw[0] = osrc[0];
    oraw[1] = osrc[1];
  }
  const uint32_t dw[8] = {draw[0].x, draw[0].y, draw[0].z, draw[0].w, draw[1].x, draw[1].y, draw[1].z, draw[1].w};
  const uint32_t ow[8] = {oraw[0].x, oraw[0].y, oraw[0].z, oraw[0].w, oraw[1].x, oraw[1].y, oraw[1].z, oraw[1].w};
  float dsum = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    dsum += __uint_as_float(dw[c] << 16) * __uint_as_float(ow[c] << 16) +
            __uint_as_float(dw[c] & 0xffff0000u) * __uint_as_float(ow[c] & 0xffff0000u);
  }
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
  // the two values of row i sit 128 floats apart inside the row's tile of 128
  float* stat = p.qstat + ((static_cast<int64_t>(b) * p.Hq + h) * p.nq_pad + (i & ~127)) * 2 + (i & 127);
  if (!live) {
    // padding rows: lse = +inf makes every probability zero
    if (sub < 2) stat[sub * 128] = sub == 0 ? -INFINITY : 0.f;
  } else if (sub == 0) {
    stat[0] = -p.lse[b * p.lse_sb + h * p.lse_sh + i];
    stat[128] = -dsum;
  }
}

// ---------------------------------------------------------------------------
// helpers shared by the two main kernels
// ---------------------------------------------------------------------------
// Four consecutive floats from shared memory (the row records: every thread reads the same address, a broadcast).
__device__ __forceinline__ float4 lds_f4(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}

// The element-wise code keeps a block of 32 values as 16 packed fp32 pairs; they go to TMEM as 16 bf16 pairs.
__device__ __forceinline__ void store_block_bf16(const uint64_t (&x)[16], uint32_t taddr) {
  uint32_t lo[8], hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float a, b, c, d;
    unpack_f32x2(x[i], a, b);
    unpack_f32x2(x[8 + i], c, d);
    lo[i] = pack_bf16x2(a, b);
    hi[i] = pack_bf16x2(c, d);
  }
  tmem_st8(taddr, lo);
  tmem_st8(taddr + 8, hi);
}

struct BwdParams {
  const float* qstat;    // [B,Hq,nq_pad/128][2][128]: -L and -D of 128 rows
  __nv_bfloat16* dq;     // [B,Hq,Nq,D] contiguous
  __nv_bfloat16* dk;     // [B,Hkv,Nk,D] contiguous
  __nv_bfloat16* dv;
  int B, Hq, Hkv, Nq, Nk, nq_pad;
  int d;  // head dimension, 128 or 64
  int causal;
  float softmax_scale;
  int* status;
};

// ---------------------------------------------------------------------------
// 2. dK / dV
// ---------------------------------------------------------------------------
constexpr int A_STAGES = 2;
constexpr int A_STAT_BYTES = BM * 8;
constexpr int A_STAGE_BYTES = 2 * TILE_BYTES + A_STAT_BYTES;
// Requested size is padded past half an SM's shared memory: each CTA allocates all 512 TMEM columns, so a second
// resident CTA could only spin in tcgen05.alloc.
constexpr int A_SMEM_BYTES = 2 * TILE_BYTES + A_STAGES * A_STAGE_BYTES + 1024 + 256;  // 197 KiB: one CTA per SM
constexpr int A_ST_COL = 0, A_DPT_COL = 128, A_DV_COL = 256, A_DK_COL = 384;
template <int DH>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_bf16_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t k_smem = smem_base;
  const uint32_t v_smem = k_smem + TILE_BYTES;
  const uint32_t stage_smem = v_smem + TILE_BYTES;  // per stage: Q tile, dO tile, row records
  const uint32_t bar_base = stage_smem + A_STAGES * A_STAGE_BYTES;
  const uint32_t kv_full = bar_base;
  auto q_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bar_base + 8u * (1 + A_STAGES + s); };
  // the two 64-query halves of a tile are handed back and forth separately (h = 0, 1)
  auto s_full = [&](int h) { return bar_base + 8u * (1 + 2 * A_STAGES + h); };
  auto p_full = [&](int h) { return bar_base + 8u * (3 + 2 * A_STAGES + h); };
  const uint32_t acc_full = bar_base + 8u * (5 + 2 * A_STAGES);
  const uint32_t tmem_slot = acc_full + 8;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int n_blk = blockIdx.x;
  const int hkv = blockIdx.y;
  const int b = blockIdx.z;
  const int n0 = n_blk * BN;
  const int group = p.Hq / p.Hkv;
  const int shift = p.Nk - p.Nq;
  const int num_m = (p.Nq + BM - 1) / BM;
  // first query tile that sees a key of this block (bottom-right aligned causal mask)
  const int m_first = p.causal ? min(num_m, max(0, n0 - shift) / BM) : 0;
  const int tiles_per_head = num_m - m_first;
  const int n_iter = group * tiles_per_head;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full(h), 1);
      mbar_init(p_full(h), HALF_THREADS);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
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
    if (lane == 0 && n_iter > 0) {
      const int chunks = DH / CHUNK;
      mbar_expect_tx(kv_full, 2 * chunks * CHUNK_BYTES);
      for (int c = 0; c < chunks; ++c) {
        tma_load_4d(k_smem + c * CHUNK_BYTES, &tmap_k, kv_full, c * CHUNK, n0, hkv, b);
        tma_load_4d(v_smem + c * CHUNK_BYTES, &tmap_v, kv_full, c * CHUNK, n0, hkv, b);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % A_STAGES;
        const uint32_t ph = (it / A_STAGES) & 1;
        const int hq = hkv * group + it / tiles_per_head;
        const int m0 = (m_first + it % tiles_per_head) * BM;
        if (!mbar_wait(q_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        const uint32_t base = stage_smem + s * A_STAGE_BYTES;
        mbar_expect_tx(q_full(s), 2 * chunks * CHUNK_BYTES + A_STAT_BYTES);
        for (int c = 0; c < chunks; ++c) {
          tma_load_4d(base + c * CHUNK_BYTES, &tmap_q, q_full(s), c * CHUNK, m0, hq, b);
          tma_load_4d(base + TILE_BYTES + c * CHUNK_BYTES, &tmap_do, q_full(s), c * CHUNK, m0, hq, b);
        }
        bulk_load(base + 2 * TILE_BYTES, p.qstat + ((static_cast<int64_t>(b) * p.Hq + hq) * p.nq_pad + m0) * 2,
                  A_STAT_BYTES, q_full(s));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      // A tile is processed as two halves of 64 queries, each with its own pair of barriers, so that the tensor
      // pipe works on one half while the element-wise warps of the other half are busy:
      //   S^T, dP^T (h) -> element-wise (h) -> dV, dK += (h) -> S^T, dP^T of the next tile (h) -> ...
      // All MMAs come from this one thread, so the products of the next tile overwrite a half's columns only
      // after the products that read its codes (the tensor pipe runs in issue order).
      constexpr uint32_t idesc_ss = make_idesc(1, 1, 0, 0, BN, BM / 2);
      const uint32_t idesc_ts = make_idesc(1, 1, 0, 1, BN, DH);  // B read MN-major, N = head dimension
      const uint32_t st_tmem = tmem_base + A_ST_COL;
      const uint32_t dpt_tmem = tmem_base + A_DPT_COL;
      bool ok = mbar_wait(kv_full, 0, p.status, WK_ERR_TIMEOUT_LOAD);
      const uint64_t k_desc = smem_desc_sw128(k_smem, 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(v_smem, 16, 1024);
      auto stage_base = [&](int it) { return stage_smem + (it % A_STAGES) * A_STAGE_BYTES; };
      // S^T = K Q^T and dP^T = V dO^T for queries [64 h, 64 h + 64) of tile `it`: rows 64 h.. of the Q and dO
      // tiles are 64 x 128 bytes further on (+512 in descriptor units); 16 head-dim elements per MMA = 32 bytes
      // inside a span, the second span one chunk (16 KiB) further on
      auto ss_half = [&](int it, int h) {
        const uint64_t q_desc = smem_desc_sw128(stage_base(it), 16, 1024) + 512 * h;
        const uint64_t do_desc = q_desc + (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = (k >> 2) * (CHUNK_BYTES >> 4) + 2 * (k & 3);
          if (16 * k < DH) mma_f16_ss(st_tmem + HALF_COLS * h, k_desc + off, q_desc + off, idesc_ss, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = (k >> 2) * (CHUNK_BYTES >> 4) + 2 * (k & 3);
          if (16 * k < DH) mma_f16_ss(dpt_tmem + HALF_COLS * h, v_desc + off, do_desc + off, idesc_ss, k != 0);
        }
        tc_commit(s_full(h));
      };
      // dV += P^T dO and dK += dS^T Q over the same 64 queries.  B operands: the dO / Q tiles again, now read
      // MN-major (K = queries, 16 per step = 2048 bytes; N = head dim, its two spans 16 KiB apart)
      auto ts_half = [&](int it, int h) {
        const uint64_t q_desc = smem_desc_sw128(stage_base(it), CHUNK_BYTES, 1024);
        const uint64_t do_desc = q_desc + (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 16 queries = 8 columns; a block of 32 queries keeps its pairs at the start of its own 32 columns
          mma_f16_ts(tmem_base + A_DV_COL, st_tmem + HALF_COLS * h + 32 * (k >> 1) + 8 * (k & 1),
                     do_desc + 128 * (4 * h + k), idesc_ts, (it | h | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          mma_f16_ts(tmem_base + A_DK_COL, dpt_tmem + HALF_COLS * h + 32 * (k >> 1) + 8 * (k & 1),
                     q_desc + 128 * (4 * h + k), idesc_ts, (it | h | k) != 0);
        }
      };
      ok = ok && mbar_wait(q_full(0), 0, p.status, WK_ERR_TIMEOUT_LOAD);
      if (ok) {
        tc_fence_after();
        ss_half(0, 0);
        ss_half(0, 1);
      }
      for (int it = 0; ok && it < n_iter; ++it) {
        const int s = it % A_STAGES;
        const bool more = it + 1 < n_iter;
        if (!mbar_wait(p_full(0), it & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        tc_fence_after();
        ts_half(it, 0);
        if (more) {
          if (!mbar_wait(q_full((it + 1) % A_STAGES), ((it + 1) / A_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
          tc_fence_after();
          ss_half(it + 1, 0);
        }
        if (!mbar_wait(p_full(1), it & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        tc_fence_after();
        ts_half(it, 1);
        tc_commit(q_empty(s));
        if (more) ss_half(it + 1, 1);
        if (!more) tc_commit(acc_full);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int c = (warp - 2) >> 2;   // which block of 32 of the tile's 128 columns this thread handles
    const int half = c >> 1;         // the half the block is handed over with
    const int r = quad * 32 + lane;  // key row of the tile == TMEM lane
    const int key = n0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    // this thread's block: scores in columns [32 c, 32 c + 32) of both buffers
    const uint32_t st_tmem = tmem_base + lane_addr + A_ST_COL + 32 * c;
    const uint32_t dpt_tmem = tmem_base + lane_addr + A_DPT_COL + 32 * c;
    const float beta = p.softmax_scale * LOG2E;
    bool ok = true;

    for (int it = 0; it < n_iter; ++it) {
      const int s = it % A_STAGES;
      const int m0 = (m_first + it % tiles_per_head) * BM;
      if (!mbar_wait_warp(s_full(half), it & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // the tile's row records: arrays -L and -D of 128 queries each, read four queries at a time
      const uint32_t stat = stage_smem + s * A_STAGE_BYTES + 2 * TILE_BYTES;
      // query column c is visible to this key iff key < Nk and (not causal or key <= m0 + c + shift)
      const int first_col = key >= p.Nk ? BM : (p.causal ? max(0, key - shift - m0) : 0);
      // uniform over the CTA: does this (key block, query tile) pair contain any masked score?
      const bool tile_masked = (n0 + BN > p.Nk) || (p.causal && n0 + BN - 1 > m0 + shift);
      {
        uint32_t sraw[32], draw[32];
        tmem_ld32(st_tmem, sraw);
        tmem_ld32(dpt_tmem, draw);
        tc_wait_ld();
        const uint64_t beta2 = pack_f32x2(beta, beta);
        // 16 queries at a time: their bf16 pairs go to the first columns of the block, which its scores have left
#pragma unroll
        for (int hq16 = 0; hq16 < 2; ++hq16) {
          uint32_t pw[8], dw[8];
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const int i = 4 * hq16 + ii;
            // the same addresses for every thread: shared-memory broadcasts
            const float4 nl = lds_f4(stat + 16 * (c * 8 + i)), nd = lds_f4(stat + 16 * (32 + c * 8 + i));
            float x0, x1, x2, x3;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i]), __uint_as_float(sraw[4 * i + 1])), beta2,
                                   pack_f32x2(nl.x, nl.y)), x0, x1);
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i + 2]), __uint_as_float(sraw[4 * i + 3])), beta2,
                                   pack_f32x2(nl.z, nl.w)), x2, x3);
            float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
            if (tile_masked) {
              if (c * 32 + 4 * i + 0 < first_col) p0 = 0.f;
              if (c * 32 + 4 * i + 1 < first_col) p1 = 0.f;
              if (c * 32 + 4 * i + 2 < first_col) p2 = 0.f;
              if (c * 32 + 4 * i + 3 < first_col) p3 = 0.f;
            }
            // dS = P (dP - D)
            float d0, d1, d2, d3;
            unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1),
                                   add_f32x2(pack_f32x2(__uint_as_float(draw[4 * i]), __uint_as_float(draw[4 * i + 1])),
                                             pack_f32x2(nd.x, nd.y))), d0, d1);
            unpack_f32x2(mul_f32x2(pack_f32x2(p2, p3),
                                   add_f32x2(pack_f32x2(__uint_as_float(draw[4 * i + 2]), __uint_as_float(draw[4 * i + 3])),
                                             pack_f32x2(nd.z, nd.w))), d2, d3);
            pw[2 * ii] = pack_bf16x2(p0, p1);
            pw[2 * ii + 1] = pack_bf16x2(p2, p3);
            dw[2 * ii] = pack_bf16x2(d0, d1);
            dw[2 * ii + 1] = pack_bf16x2(d2, d3);
          }
          tmem_st8(st_tmem + 8 * hq16, pw);
          tmem_st8(dpt_tmem + 8 * hq16, dw);
        }
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(half));
    }

    if (n_iter > 0 && ok) ok = mbar_wait_warp(acc_full, 0, p.status, WK_ERR_TIMEOUT_MMA);
    if (ok) {
      tc_fence_after();
      const float dk_scale = p.softmax_scale;
      const int64_t row_off = ((static_cast<int64_t>(b) * p.Hkv + hkv) * p.Nk + key) * DH;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = tmem_base + lane_addr + (which == 0 ? A_DV_COL : A_DK_COL);
        __nv_bfloat16* dst_row = (which == 0 ? p.dv : p.dk) + row_off;
        const float scale = which == 0 ? 1.f : dk_scale;
#pragma unroll 1
        {
          uint32_t v[32];
          if (n_iter > 0) {  // uniform: TMEM loads are warp-wide
            tmem_ld32(src + c * 32, v);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0;
          }
          if (key < p.Nk && c * 32 < DH) {
            uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * scale, __uint_as_float(v[8 * i + 1]) * scale);
              w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * scale, __uint_as_float(v[8 * i + 3]) * scale);
              w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * scale, __uint_as_float(v[8 * i + 5]) * scale);
              w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * scale, __uint_as_float(v[8 * i + 7]) * scale);
              dst[i] = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// 3. dQ
// ---------------------------------------------------------------------------
constexpr int B_STAGES = 2;
constexpr int B_STAGE_BYTES = 2 * TILE_BYTES;  // K tile, V tile
constexpr int B_SMEM_BYTES = 2 * TILE_BYTES + B_STAGES * B_STAGE_BYTES + 1024 + 256;  // 193 KiB: one CTA per SM
constexpr int B_S_COL = 0, B_DP_COL = 128, B_DQ_COL = 256;

template <int DH>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_bf16_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t do_smem = q_smem + TILE_BYTES;
  const uint32_t stage_smem = do_smem + TILE_BYTES;
  const uint32_t bar_base = stage_smem + B_STAGES * B_STAGE_BYTES;
  const uint32_t q_full = bar_base;
  auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + B_STAGES + s); };
  // the two 64-key halves of a tile are handed back and forth separately (h = 0, 1)
  auto s_full = [&](int h) { return bar_base + 8u * (1 + 2 * B_STAGES + h); };
  auto p_full = [&](int h) { return bar_base + 8u * (3 + 2 * B_STAGES + h); };
  const uint32_t acc_full = bar_base + 8u * (5 + 2 * B_STAGES);
  const uint32_t tmem_slot = acc_full + 8;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int m_blk = gridDim.x - 1 - blockIdx.x;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int m0 = m_blk * BM;
  const int shift = p.Nk - p.Nq;
  int n_tiles = (p.Nk + BN - 1) / BN;
  if (p.causal) {
    const int last_key = min(m0 + BM, p.Nq) - 1 + shift;
    n_tiles = last_key < 0 ? 0 : min(n_tiles, last_key / BN + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < B_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full(h), 1);
      mbar_init(p_full(h), HALF_THREADS);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
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
    if (lane == 0 && n_tiles > 0) {
      const int chunks = DH / CHUNK;
      mbar_expect_tx(q_full, 2 * chunks * CHUNK_BYTES);
      for (int c = 0; c < chunks; ++c) {
        tma_load_4d(q_smem + c * CHUNK_BYTES, &tmap_q, q_full, c * CHUNK, m0, hq, b);
        tma_load_4d(do_smem + c * CHUNK_BYTES, &tmap_do, q_full, c * CHUNK, m0, hq, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % B_STAGES;
        const uint32_t ph = (j / B_STAGES) & 1;
        if (!mbar_wait(kv_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        const uint32_t base = stage_smem + s * B_STAGE_BYTES;
        mbar_expect_tx(kv_full(s), 2 * chunks * CHUNK_BYTES);
        for (int c = 0; c < chunks; ++c) {
          tma_load_4d(base + c * CHUNK_BYTES, &tmap_k, kv_full(s), c * CHUNK, j * BN, hkv, b);
          tma_load_4d(base + TILE_BYTES + c * CHUNK_BYTES, &tmap_v, kv_full(s), c * CHUNK, j * BN, hkv, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      // Key tiles are processed as two halves of 64 keys, as in the dK/dV kernel: the tensor pipe works on one
      // half while the element-wise warps of the other are busy.
      constexpr uint32_t idesc_ss = make_idesc(1, 1, 0, 0, BM, BN / 2);
      const uint32_t idesc_ts = make_idesc(1, 1, 0, 1, BM, DH);  // B read MN-major, N = head dimension
      const uint32_t s_tmem = tmem_base + B_S_COL;
      const uint32_t dp_tmem = tmem_base + B_DP_COL;
      bool ok = mbar_wait(q_full, 0, p.status, WK_ERR_TIMEOUT_LOAD);
      const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
      const uint64_t do_desc = smem_desc_sw128(do_smem, 16, 1024);
      auto stage_base = [&](int j) { return stage_smem + (j % B_STAGES) * B_STAGE_BYTES; };
      // S = Q K^T and dP = dO V^T for keys [64 h, 64 h + 64) of tile j (rows 64 h.. of the K and V tiles: +512 in
      // descriptor units)
      auto ss_half = [&](int j, int h) {
        const uint64_t k_desc = smem_desc_sw128(stage_base(j), 16, 1024) + 512 * h;
        const uint64_t v_desc = k_desc + (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = (k >> 2) * (CHUNK_BYTES >> 4) + 2 * (k & 3);
          if (16 * k < DH) mma_f16_ss(s_tmem + HALF_COLS * h, q_desc + off, k_desc + off, idesc_ss, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = (k >> 2) * (CHUNK_BYTES >> 4) + 2 * (k & 3);
          if (16 * k < DH) mma_f16_ss(dp_tmem + HALF_COLS * h, do_desc + off, v_desc + off, idesc_ss, k != 0);
        }
        tc_commit(s_full(h));
      };
      // dQ += dS K over the same 64 keys: A = dS as bf16 in the dP columns, B = the K tile read MN-major
      auto ts_half = [&](int j, int h) {
        const uint64_t k_desc = smem_desc_sw128(stage_base(j), CHUNK_BYTES, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 16 keys = 8 columns; a block of 32 keys keeps its pairs at the start of its own 32 columns
          mma_f16_ts(tmem_base + B_DQ_COL, dp_tmem + HALF_COLS * h + 32 * (k >> 1) + 8 * (k & 1),
                     k_desc + 128 * (4 * h + k), idesc_ts, (j | h | k) != 0);
        }
      };
      ok = ok && mbar_wait(kv_full(0), 0, p.status, WK_ERR_TIMEOUT_LOAD);
      if (ok) {
        tc_fence_after();
        ss_half(0, 0);
        ss_half(0, 1);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % B_STAGES;
        const bool more = j + 1 < n_tiles;
        if (!mbar_wait(p_full(0), j & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        tc_fence_after();
        ts_half(j, 0);
        if (more) {
          if (!mbar_wait(kv_full((j + 1) % B_STAGES), ((j + 1) / B_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
          tc_fence_after();
          ss_half(j + 1, 0);
        }
        if (!mbar_wait(p_full(1), j & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        tc_fence_after();
        ts_half(j, 1);
        tc_commit(kv_empty(s));
        if (more) ss_half(j + 1, 1);
        if (!more) tc_commit(acc_full);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int c = (warp - 2) >> 2;  // which block of 32 of the tile's 128 columns this thread handles
    const int half = c >> 1;        // the half the block is handed over with
    const int r = quad * 32 + lane;
    const int row = m0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    // this thread's block: scores in columns [32 c, 32 c + 32) of both buffers
    const uint32_t s_tmem = tmem_base + lane_addr + B_S_COL + 32 * c;
    const uint32_t dp_tmem = tmem_base + lane_addr + B_DP_COL + 32 * c;
    const float beta = p.softmax_scale * LOG2E;
    const float* rec = p.qstat + ((static_cast<int64_t>(b) * p.Hq + hq) * p.nq_pad + m0) * 2 + r;
    const float neg_l = rec[0], neg_d = rec[128];  // -L and -D of this query
    const int row_limit = min(p.causal ? row + shift : p.Nk - 1, p.Nk - 1);
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait_warp(s_full(half), j & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int limit = row_limit - j * BN;  // columns > limit are masked
      // uniform over the CTA: does this tile contain any masked score?
      const bool tile_masked = (j * BN + BN > p.Nk) || (p.causal && j * BN + BN - 1 > m0 + shift);
      {
        uint32_t sraw[32], draw[32];
        tmem_ld32(s_tmem, sraw);
        tmem_ld32(dp_tmem, draw);
        tc_wait_ld();
        uint64_t ds[16];  // dS of this query for 32 keys, as packed pairs
        const uint64_t beta2 = pack_f32x2(beta, beta), nl2 = pack_f32x2(neg_l, neg_l), nd2 = pack_f32x2(neg_d, neg_d);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[2 * i]), __uint_as_float(sraw[2 * i + 1])), beta2, nl2),
                       x0, x1);
          float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          if (tile_masked) {
            if (c * 32 + 2 * i > limit) p0 = 0.f;
            if (c * 32 + 2 * i + 1 > limit) p1 = 0.f;
          }
          ds[i] = mul_f32x2(pack_f32x2(p0, p1),
                            add_f32x2(pack_f32x2(__uint_as_float(draw[2 * i]), __uint_as_float(draw[2 * i + 1])), nd2));
        }
        store_block_bf16(ds, dp_tmem);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(half));
    }

    if (n_tiles > 0 && ok) ok = mbar_wait_warp(acc_full, 0, p.status, WK_ERR_TIMEOUT_MMA);
    if (ok) {
      tc_fence_after();
      const float scale = p.softmax_scale;
      __nv_bfloat16* dst_row = p.dq + ((static_cast<int64_t>(b) * p.Hq + hq) * p.Nq + row) * DH;
#pragma unroll 1
      {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem_base + lane_addr + B_DQ_COL + c * 32, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row < p.Nq && c * 32 < DH) {
          uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * scale, __uint_as_float(v[8 * i + 1]) * scale);
            w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * scale, __uint_as_float(v[8 * i + 3]) * scale);
            w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * scale, __uint_as_float(v[8 * i + 5]) * scale);
            w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * scale, __uint_as_float(v[8 * i + 7]) * scale);
            dst[i] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int make_map4(CUtensorMap* m, const void* base, int d, int n, int h, int b, const int64_t* strides) {
  const uint64_t dims[4] = {static_cast<uint64_t>(d), static_cast<uint64_t>(n), static_cast<uint64_t>(h), static_cast<uint64_t>(b)};
  const uint64_t str[3] = {static_cast<uint64_t>(strides[2]) * 2, static_cast<uint64_t>(strides[1]) * 2,
                           static_cast<uint64_t>(strides[0]) * 2};
  const uint32_t box[4] = {CHUNK, 128, 1, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace
}  // namespace wk

extern "C" int64_t wk_attn_bwd_bf16_workspace_bytes(int B, int Hq, int Nq) {
  if (B < 0 || Hq < 0 || Nq < 0) return WK_E_ARG;
  const int64_t nq_pad = (static_cast<int64_t>(Nq) + 127) / 128 * 128;
  return static_cast<int64_t>(B) * Hq * nq_pad * 16 + 256;
}

extern "C" int wk_attn_bwd_bf16(const wk_attn_bwd_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nk <= 0 || (a->d != 128 && a->d != 64)) return WK_E_ARG;
  if (a->Hq % a->Hkv || a->B > 65535 || a->Hq > 65535) return WK_E_ARG;
  if (!a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv) return WK_E_ARG;
  if (a->q_descale || a->k_descale || a->v_descale || !a->workspace) return WK_E_ARG;
  if (!(a->softmax_scale > 0.f)) return WK_E_ARG;
  const void* ptrs[] = {a->q, a->k, a->v, a->dout, a->dq, a->dk, a->dv, a->workspace};
  for (const void* ptr : ptrs)
    if (!aligned16(ptr)) return WK_E_ARG;
  if (reinterpret_cast<uintptr_t>(a->out) & 7) return WK_E_ARG;
  for (int i = 0; i < 3; ++i) {
    if (a->q_strides[i] % 8 || a->k_strides[i] % 8 || a->v_strides[i] % 8 || a->dout_strides[i] % 8) return WK_E_ARG;
    if (a->q_strides[i] <= 0 || a->k_strides[i] <= 0 || a->v_strides[i] <= 0 || a->dout_strides[i] <= 0)
      return WK_E_ARG;
    if (a->out_strides[i] % 4 || a->out_strides[i] <= 0) return WK_E_ARG;
  }
  if (a->workspace_bytes < wk_attn_bwd_bf16_workspace_bytes(a->B, a->Hq, a->Nq)) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int nq_pad = (a->Nq + 127) / 128 * 128;
  float* qstat = static_cast<float*>(a->workspace);

  PrepParams pp;
  pp.dout = static_cast<const __nv_bfloat16*>(a->dout);
  pp.out = static_cast<const __nv_bfloat16*>(a->out);
  pp.lse = a->lse;
  pp.qstat = qstat;
  pp.do_sb = a->dout_strides[0];
  pp.do_sh = a->dout_strides[1];
  pp.do_sn = a->dout_strides[2];
  pp.o_sb = a->out_strides[0];
  pp.o_sh = a->out_strides[1];
  pp.o_sn = a->out_strides[2];
  pp.lse_sb = a->lse_strides[0];
  pp.lse_sh = a->lse_strides[1];
  pp.B = a->B;
  pp.Hq = a->Hq;
  pp.Nq = a->Nq;
  pp.nq_pad = nq_pad;
  pp.d = a->d;
  {
    const int64_t rows = static_cast<int64_t>(a->B) * a->Hq * nq_pad;
    bool wide_loads = aligned16(a->out) && aligned16(a->dout);  // 16-byte loads: rows on 16-byte boundaries
    for (int i = 0; i < 3; ++i) wide_loads = wide_loads && a->out_strides[i] % 8 == 0 && a->dout_strides[i] % 8 == 0;
    if (wide_loads) {
      attn_bwd_bf16_prep4_kernel<<<static_cast<unsigned>((rows + 31) / 32), 256, 0, st>>>(pp);
    } else {
      const int64_t blocks = (rows + 7) / 8;
      attn_bwd_bf16_prep_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(pp);
    }
    if (cudaGetLastError() != cudaSuccess) return WK_E_CUDA;
  }

  CUtensorMap tq, tk, tv, tdo;
  int r = make_map4(&tq, a->q, a->d, a->Nq, a->Hq, a->B, a->q_strides);
  if (r) return r;
  r = make_map4(&tk, a->k, a->d, a->Nk, a->Hkv, a->B, a->k_strides);
  if (r) return r;
  r = make_map4(&tv, a->v, a->d, a->Nk, a->Hkv, a->B, a->v_strides);
  if (r) return r;
  r = make_map4(&tdo, a->dout, a->d, a->Nq, a->Hq, a->B, a->dout_strides);
  if (r) return r;

  BwdParams p;
  p.qstat = qstat;
  p.dq = static_cast<__nv_bfloat16*>(a->dq);
  p.dk = static_cast<__nv_bfloat16*>(a->dk);
  p.dv = static_cast<__nv_bfloat16*>(a->dv);
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Nq = a->Nq;
  p.Nk = a->Nk;
  p.nq_pad = nq_pad;
  p.d = a->d;
  p.causal = a->causal;
  p.softmax_scale = a->softmax_scale;
  p.status = status;

  if (allow_smem((a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_bf16_dkdv_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_bf16_dkdv_kernel<128>)), A_SMEM_BYTES)) return WK_E_CUDA;
  if (allow_smem((a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_bf16_dq_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_bf16_dq_kernel<128>)), B_SMEM_BYTES)) return WK_E_CUDA;
  {
    dim3 grid((a->Nk + BN - 1) / BN, a->Hkv, a->B);
    void* args[] = {&tq, &tk, &tv, &tdo, &p};
    const void* kernel = a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_bf16_dkdv_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_bf16_dkdv_kernel<128>);
    if (cudaLaunchKernel(kernel, grid, dim3(THREADS), args, A_SMEM_BYTES, st) != cudaSuccess) return WK_E_CUDA;
  }
  {
    dim3 grid((a->Nq + BM - 1) / BM, a->Hq, a->B);
    void* args[] = {&tq, &tk, &tv, &tdo, &p};
    const void* kernel = a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_bf16_dq_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_bf16_dq_kernel<128>);
    if (cudaLaunchKernel(kernel, grid, dim3(THREADS), args, B_SMEM_BYTES, st) != cudaSuccess) return WK_E_CUDA;
  }
  return 0;
}
