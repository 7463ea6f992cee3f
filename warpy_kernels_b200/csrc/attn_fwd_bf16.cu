// BF16 flash-attention forward for sm_100a, head dimension 128.
//
// Same structure as the FP8 forward (attn_fwd_fp8.cu): one CTA = 128 queries of one (batch, query head), two
// CTAs per SM, key tiles of 64, 320 threads:
//   warp 0      TMA producer: Q tile once, then K and V tiles into two-stage rings.  A row is 256 bytes, two
//               128-byte swizzle spans, so every tile is loaded as two boxes of 64 head-dim elements
//   warp 1      allocates 256 TMEM columns (two S buffers of 64 columns, O: 128..255) and issues tcgen05.mma
//               kind::f16:  S = Q.K^T (both operands K-major from shared memory) two tiles ahead,
//               O += P.V (P read from TMEM, V MN-major from shared memory) as soon as a tile's P is there
//   warps 2-9   softmax in two groups of four warps that take the key tiles in turn; inside a group one thread
//               per query row: read S from TMEM, write P as bf16 back over the S columns, row sums; finally
//               O / l -> bf16, lse (base 2) and pmax
//
// Numerics follow the reference's bf16 forward (warpy_kernels/attn/fwd_base.py:297-360, 374-416, 939-988):
// logits in base 2 with beta = softmax_scale . log2(e), bottom-right aligned causal mask, P rounded to bf16,
// lse = m_ref + log2(l), pmax = 2^(m_true - lse), empty rows give out = 0, lse = +inf, pmax = 0.  Where the
// reference moves its reference exponent with the running maximum and rescales O, this kernel fixes m_ref per
// row at the maximum of the first tile and never rescales: bf16 has the exponent range of fp32, so
// P = 2^(s.beta - m_ref) keeps its eight significant bits whether it lies above or below 1.  Scores that outgrow
// m_ref by more than 2^100 make the kernel flag the query block in the call's workspace, and attn_fwd_redo.cu
// computes it again with the exact row maximum (without a workspace: WK_ERR_RANGE in the status word).
//
// Tensor-core bound: 4 . B . Hq . Nq . Nk . d flops (half of that when causal).
#include <math.h>

#include "attn_fwd_redo.h"
#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

constexpr int BM = 128;       // queries per CTA
constexpr int BN = 64;        // keys per tile
constexpr int D = 128;        // largest head dimension; the kernel is instantiated for DH = 128 and 64 (one 128-byte
                              // span per row instead of two: the second box of every tile is simply not loaded)
constexpr int CHUNK = 64;     // head-dim elements per 128-byte swizzle span
constexpr int KV_STAGES = 2;
constexpr int Q_CHUNK_BYTES = BM * CHUNK * 2;   // 16 KiB: 128 rows x 128 bytes
constexpr int KV_CHUNK_BYTES = BN * CHUNK * 2;  // 8 KiB
constexpr int Q_BYTES = 2 * Q_CHUNK_BYTES;      // 32 KiB
constexpr int KV_BYTES = 2 * KV_CHUNK_BYTES;    // 16 KiB
constexpr int THREADS = 320;
constexpr int GROUP_THREADS = 128;  // one softmax group
constexpr int TMEM_COLS = 256;
constexpr int S_COLS = 64;    // one S buffer; buffer b starts at column 64 b
constexpr int O_COL = 128;
constexpr float MAX_BLOCK_EXP = 100.f;  // how far (log2) a block may rise above the row reference
// After the softmax the first 32 columns of an S buffer hold P: block k of 32 keys keeps its bf16 pairs in
// columns [16 k, 16 k + 16).
constexpr int XCH_BYTES = 7 * BM * 4;  // row reference plus (l, lq, m_true) of each group
constexpr int SMEM_BYTES = Q_BYTES + 2 * KV_STAGES * KV_BYTES + XCH_BYTES + 1024 + 256;

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  float* pmax;
  int64_t out_stride_b, out_stride_h, out_stride_n;  // elements
  int64_t lse_stride_b, lse_stride_h;                // elements
  int B, Hq, Hkv, Nq, Nk;
  int causal;
  int write_lse;
  int lse_natural;
  const int* seqused_k;  // [B] or null
  float softmax_scale;
  int m_first;  // first query block of this launch (the grid covers gridDim.x blocks from here)
  int* status;
  int* redo;    // one flag per query block, or null: blocks whose scores outgrow the row reference are recomputed
};

// One block of 32 keys of one row: P as 16 bf16 pairs and the sum of the unrounded values.
__device__ __forceinline__ void softmax_block(const uint32_t (&sraw)[32], float beta, float bias, uint32_t (&w)[16],
                                              float& sum_exact) {
  const uint64_t beta2 = pack_f32x2(beta, beta), bias2 = pack_f32x2(bias, bias);
  uint64_t acc01 = 0, acc23 = 0;  // packed fp32 partial sums
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float p0, p1, p2, p3;
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i + 0]), __uint_as_float(sraw[4 * i + 1])), beta2, bias2),
                 p0, p1);
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i + 2]), __uint_as_float(sraw[4 * i + 3])), beta2, bias2),
                 p2, p3);
    p0 = ex2_approx(p0);
    p1 = ex2_approx(p1);
    p2 = ex2_approx(p2);
    p3 = ex2_approx(p3);
    acc01 = add_f32x2(acc01, pack_f32x2(p0, p1));
    acc23 = add_f32x2(acc23, pack_f32x2(p2, p3));
    w[2 * i] = pack_bf16x2(p0, p1);
    w[2 * i + 1] = pack_bf16x2(p2, p3);
  }
  {
    float a0, a1, a2, a3;
    unpack_f32x2(acc01, a0, a1);
    unpack_f32x2(acc23, a2, a3);
    sum_exact = (a0 + a1) + (a2 + a3);
  }
}

__device__ __forceinline__ float block_max(const uint32_t (&s)[32]) {
  float a0 = fmaxf(__uint_as_float(s[0]), __uint_as_float(s[1]));
  float a1 = fmaxf(__uint_as_float(s[2]), __uint_as_float(s[3]));
  float a2 = fmaxf(__uint_as_float(s[4]), __uint_as_float(s[5]));
  float a3 = fmaxf(__uint_as_float(s[6]), __uint_as_float(s[7]));
#pragma unroll
  for (int i = 8; i < 32; i += 8) {
    a0 = max3(a0, __uint_as_float(s[i + 0]), __uint_as_float(s[i + 1]));
    a1 = max3(a1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
    a2 = max3(a2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
    a3 = max3(a3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
  }
  return fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
}

template <int DH>
__global__ void __launch_bounds__(THREADS, 2)
attn_fwd_bf16_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + Q_BYTES;
  const uint32_t v_smem = k_smem + KV_STAGES * KV_BYTES;
  const uint32_t xch_smem = v_smem + KV_STAGES * KV_BYTES;  // exchange between the two softmax groups
  const uint32_t bar_base = xch_smem + XCH_BYTES;
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (1 + KV_STAGES + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (1 + 2 * KV_STAGES + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (1 + 3 * KV_STAGES + s); };
  const uint32_t misc_bar = bar_base + 8u * (1 + 4 * KV_STAGES);
  auto s_full = [&](int b) { return misc_bar + 8u * b; };
  auto p_full = [&](int b) { return misc_bar + 8u * (2 + b); };
  const uint32_t o_full = misc_bar + 8u * 4;
  const uint32_t tmem_slot = misc_bar + 8u * 5;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int m_blk = p.m_first + gridDim.x - 1 - blockIdx.x;  // longest (latest) causal blocks first
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int m0 = m_blk * BM;
  // keys this batch item attends to; the causal diagonal is aligned to that length
  const int nk = p.seqused_k ? max(0, min(p.Nk, p.seqused_k[b])) : p.Nk;
  const int shift = nk - p.Nq;  // key j is visible to query i iff j <= i + shift (causal)

  // number of key tiles this query block touches
  int n_tiles = (nk + BN - 1) / BN;
  if (p.causal) {
    const int last_row = min(m0 + BM, p.Nq) - 1;
    const int last_key = last_row + shift;  // may be negative
    n_tiles = last_key < 0 ? 0 : min(n_tiles, last_key / BN + 1);
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), GROUP_THREADS);
    }
    mbar_init(o_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
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
      mbar_expect_tx(q_full, (DH / CHUNK) * Q_CHUNK_BYTES);
      tma_load_4d(q_smem, &tmap_q, q_full, 0, m0, hq, b);
      if (DH > CHUNK) tma_load_4d(q_smem + Q_CHUNK_BYTES, &tmap_q, q_full, CHUNK, m0, hq, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(k_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(k_full(s), (DH / CHUNK) * KV_CHUNK_BYTES);
        tma_load_4d(k_smem + s * KV_BYTES, &tmap_k, k_full(s), 0, j * BN, hkv, b);
        if (DH > CHUNK) tma_load_4d(k_smem + s * KV_BYTES + KV_CHUNK_BYTES, &tmap_k, k_full(s), CHUNK, j * BN, hkv, b);
        if (!mbar_wait(v_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(v_full(s), (DH / CHUNK) * KV_CHUNK_BYTES);
        tma_load_4d(v_smem + s * KV_BYTES, &tmap_v, v_full(s), 0, j * BN, hkv, b);
        if (DH > CHUNK) tma_load_4d(v_smem + s * KV_BYTES + KV_CHUNK_BYTES, &tmap_v, v_full(s), CHUNK, j * BN, hkv, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(1, 1, 0, 0, BM, BN);
      constexpr uint32_t idesc_pv = make_idesc(1, 1, 0, 1, BM, DH);  // B = V read MN-major
      const uint32_t o_tmem = tmem_base + O_COL;
      const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
      bool ok = mbar_wait(q_full, 0, p.status, WK_ERR_TIMEOUT_LOAD);
      // S(j) = Q.K(j)^T into buffer j & 1.  The tensor pipe runs in issue order, so this also waits for the
      // P.V product that last read that buffer.
      auto issue_qk = [&](int j) -> bool {
        const int s = j % KV_STAGES;
        if (!mbar_wait(k_full(s), (j / KV_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) return false;
        tc_fence_after();
        const uint64_t k_desc = smem_desc_sw128(k_smem + s * KV_BYTES, 16, 1024);
        const uint32_t s_tmem = tmem_base + (j & 1) * S_COLS;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          // 16 bf16 = 32 bytes along the head dimension inside a 128-byte swizzle span; the second span of
          // a tile starts one chunk further on
          mma_f16_ss(s_tmem, q_desc + (k >> 2) * (Q_CHUNK_BYTES >> 4) + 2 * (k & 3),
                     k_desc + (k >> 2) * (KV_CHUNK_BYTES >> 4) + 2 * (k & 3), idesc_qk, k != 0);
        }
        tc_commit(k_empty(s));
        tc_commit(s_full(j & 1));
        return true;
      };
      ok = ok && issue_qk(0);
      if (ok && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const int sb = j & 1;
        const uint32_t s_tmem = tmem_base + sb * S_COLS;
        if (!mbar_wait(p_full(sb), (j >> 1) & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        if (!mbar_wait(v_full(s), (j / KV_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        tc_fence_after();
        // V tile: 64 keys (the MMA's K) x 128 head-dim elements (the MMA's N): MN-major, two 128-byte spans
        // 8 KiB apart (leading offset), 8-key groups 1024 bytes apart, 16 keys per MMA = 2048 bytes
        const uint64_t v_desc = smem_desc_sw128(v_smem + s * KV_BYTES, KV_CHUNK_BYTES, 1024);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // P: 16 bf16 per K step = 8 TMEM columns at column 8 k
          mma_f16_ts(o_tmem, s_tmem + 8 * k, v_desc + 128 * k, idesc_pv, (j | k) != 0);
        }
        tc_commit(v_empty(s));
        if (j == n_tiles - 1) tc_commit(o_full);
        if (j + 2 < n_tiles) ok = issue_qk(j + 2);
      }
    }
    __syncwarp();
  } else {
    // Two groups of four warps take the key tiles in turn: group g handles tiles g, g + 2, ... out of S buffer g.
    // Inside a group one thread owns one query row.
    const int quad = warp & 3;  // TMEM lanes [32 quad, 32 quad + 32) are the ones this warp may touch
    const int grp = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // row of the tile == TMEM lane
    const int row = m0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + grp * S_COLS;
    const uint32_t o_tmem = tmem_base + lane_addr + O_COL;
    const uint32_t x_ref = xch_smem + r * 4;
    const float beta = p.softmax_scale * 1.4426950408889634f;
    const int row_limit = p.causal ? row + shift : nk - 1;  // last visible key of this row
    // m_ref: reference exponent of the row, fixed by the first tile (O and the sums are in units of 2^-m_ref)
    // l: sum of the exact probabilities over this group's tiles (normaliser of O, lse, pmax)
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    bool met = false;  // the one-time meeting of the two groups has taken place

    for (int j = grp; j < n_tiles; j += 2) {
      const int it = j >> 1;
      if (!mbar_wait_warp(s_full(grp), it & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int key0 = j * BN;
      const bool tile_masked = (key0 + BN > nk) || (p.causal && key0 + BN - 1 > m0 + shift);
      const int limit = min(row_limit, nk - 1) - key0;  // columns > limit are masked

      if (j == 0) {
        // the row reference: maximum of the first tile (every row that sees any key sees one here)
        float t = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t sraw[32];
          tmem_ld32(s_tmem + c * 32, sraw);
          tc_wait_ld();
          if (tile_masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > limit) sraw[i] = 0xff800000u;
          }
          t = fmaxf(t, block_max(sraw) * beta);
        }
        m_ref = t;
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(x_ref), "f"(t) : "memory");
      }
      if (it == 0) {
        // both groups meet once: the second one picks up the reference the first one has just published
        asm volatile("bar.sync 1, 256;" ::: "memory");
        met = true;
        if (grp == 1) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(m_ref) : "r"(x_ref) : "memory");
      }

#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sraw[32];
        tmem_ld32(s_tmem + c * 32, sraw);
        tc_wait_ld();
        if (tile_masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > limit) sraw[i] = 0xff800000u;  // -inf
        }
        const float cm = block_max(sraw) * beta;  // beta > 0 (checked on the host)
        m_true = fmaxf(m_true, cm);
        // masked scores are -inf and give P = 0; a row without a visible key so far has m_ref = -inf
        const float bias = m_ref > -INFINITY ? -m_ref : 0.f;
        uint32_t w[16];
        float sum_exact;
        softmax_block(sraw, beta, bias, w, sum_exact);
        l += sum_exact;
        // the pairs go to the first columns of the buffer, which the scores read so far have left
        uint32_t w_lo[8], w_hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          w_lo[i] = w[i];
          w_hi[i] = w[8 + i];
        }
        tmem_st8(s_tmem + c * 16, w_lo);
        tmem_st8(s_tmem + c * 16 + 8, w_hi);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(grp));
    }
    if (!met) {
      // this group had no tile (or gave up on a wait): it still owes the other group the meeting above
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }

    // epilogue: the groups add up their sums; group g stores head-dim columns [64 g, 64 g + 64)
    if (n_tiles > 0 && ok) ok = mbar_wait_warp(o_full, 0, p.status, WK_ERR_TIMEOUT_MMA);
    const uint32_t x_mine = xch_smem + (1 + 3 * grp) * BM * 4 + r * 4;
    const uint32_t x_other = xch_smem + (1 + 3 * (grp ^ 1)) * BM * 4 + r * 4;
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(x_mine), "f"(l) : "memory");
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(x_mine + 2 * BM * 4), "f"(m_true) : "memory");
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      float l_o, mt_o;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(l_o) : "r"(x_other) : "memory");
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(mt_o) : "r"(x_other + 2 * BM * 4) : "memory");
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(m_ref) : "r"(x_ref) : "memory");
      l += l_o;
      m_true = fmaxf(m_true, mt_o);
    }
    if (grp == 0 && m_true - m_ref > MAX_BLOCK_EXP) {
      // Some key lies more than 2^100 above the first tile's maximum: P has overflowed bf16.  With a flag array the
      // block is computed again (attn_fwd_redo.cu) and what is stored below is overwritten.
      if (p.redo)
        p.redo[attn_fwd_flag_index(b, hq, m_blk, p.Hq, (p.Nq + BM - 1) / BM)] = 1;
      else
        atomicCAS(p.status, 0, WK_ERR_RANGE);
    }
    if (ok) {
      tc_fence_after();
      const bool empty = !(l > 0.f);
      const float inv = empty ? 0.f : 1.f / l;
      const int col0 = (DH / 2) * grp;
      __nv_bfloat16* out_row = p.out + b * p.out_stride_b + hq * p.out_stride_h +
                               static_cast<int64_t>(row) * p.out_stride_n + col0;
#pragma unroll 1
      for (int c = 0; c < DH / 64; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld32(o_tmem + col0 + c * 32, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row < p.Nq) {
          uint4* dst = reinterpret_cast<uint4*>(out_row + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
            dst[i] = w;
          }
        }
      }
      if (p.write_lse && grp == 0 && row < p.Nq) {
        const int64_t off = b * p.lse_stride_b + hq * p.lse_stride_h + row;
        const float lse = empty ? INFINITY : m_ref + log2f(l);
        p.lse[off] = p.lse_natural ? lse * 0.6931471805599453f : lse;
        p.pmax[off] = empty ? 0.f : exp2f(m_true - lse);
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

}  // namespace
}  // namespace wk

extern "C" int wk_attn_fwd_bf16(const wk_attn_fwd_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nk <= 0 || (a->d != 128 && a->d != 64)) return WK_E_ARG;
  if (a->Hq % a->Hkv) return WK_E_ARG;
  if (!a->q || !a->k || !a->v || !a->out) return WK_E_ARG;
  if (a->q_descale || a->k_descale || a->v_descale) return WK_E_ARG;  // descales belong to the fp8 kernels
  if (a->write_lse && (!a->lse || !a->pmax)) return WK_E_ARG;
  if (!(a->softmax_scale > 0.f)) return WK_E_ARG;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) return WK_E_ARG;
  const int64_t* qs = a->q_strides;
  const int64_t* ks = a->k_strides;
  const int64_t* vs = a->v_strides;
  for (int i = 0; i < 3; ++i) {
    if (qs[i] % 8 || ks[i] % 8 || vs[i] % 8 || qs[i] <= 0 || ks[i] <= 0 || vs[i] <= 0) return WK_E_ARG;
    if (a->out_strides[i] % 8 || a->out_strides[i] <= 0) return WK_E_ARG;
  }
  if (a->B > 65535 || a->Hq > 65535) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;

  CUtensorMap tq, tk, tv;
  const uint32_t box[4] = {CHUNK, BM, 1, 1};
  const uint32_t box_kv[4] = {CHUNK, BN, 1, 1};
  {
    const uint64_t dims[4] = {static_cast<uint64_t>(a->d), static_cast<uint64_t>(a->Nq), static_cast<uint64_t>(a->Hq),
                              static_cast<uint64_t>(a->B)};
    const uint64_t str[3] = {static_cast<uint64_t>(qs[2]) * 2, static_cast<uint64_t>(qs[1]) * 2,
                             static_cast<uint64_t>(qs[0]) * 2};
    int r = encode_tmap(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    const uint64_t dims[4] = {static_cast<uint64_t>(a->d), static_cast<uint64_t>(a->Nk), static_cast<uint64_t>(a->Hkv),
                              static_cast<uint64_t>(a->B)};
    const uint64_t strk[3] = {static_cast<uint64_t>(ks[2]) * 2, static_cast<uint64_t>(ks[1]) * 2,
                              static_cast<uint64_t>(ks[0]) * 2};
    const uint64_t strv[3] = {static_cast<uint64_t>(vs[2]) * 2, static_cast<uint64_t>(vs[1]) * 2,
                              static_cast<uint64_t>(vs[0]) * 2};
    int r = encode_tmap(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->k, dims, strk, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
    r = encode_tmap(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->v, dims, strv, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  FwdParams p;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = static_cast<float*>(a->lse);
  p.pmax = static_cast<float*>(a->pmax);
  p.out_stride_b = a->out_strides[0];
  p.out_stride_h = a->out_strides[1];
  p.out_stride_n = a->out_strides[2];
  p.lse_stride_b = a->lse_strides[0];
  p.lse_stride_h = a->lse_strides[1];
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Nq = a->Nq;
  p.Nk = a->Nk;
  p.causal = a->causal;
  p.write_lse = a->write_lse;
  p.lse_natural = a->lse_natural;
  p.seqused_k = a->seqused_k;
  p.softmax_scale = a->softmax_scale;
  p.status = status;
  p.redo = static_cast<int*>(a->workspace);
  if (a->workspace && (a->workspace_bytes < attn_fwd_flag_bytes(a->B, a->Hq, a->Nq) ||
                       (reinterpret_cast<uintptr_t>(a->workspace) & 3)))
    return WK_E_ARG;

  const void* kernel = a->d == 64 ? reinterpret_cast<const void*>(attn_fwd_bf16_kernel<64>)
                                  : reinterpret_cast<const void*>(attn_fwd_bf16_kernel<128>);
  if (allow_smem(kernel, SMEM_BYTES)) return WK_E_CUDA;
  const int num_m = (a->Nq + BM - 1) / BM;
  p.m_first = 0;
  dim3 grid(num_m, a->Hq, a->B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  void* args[] = {&tq, &tk, &tv, &p};
  if (cudaLaunchKernel(kernel, grid, dim3(THREADS), args, SMEM_BYTES, st) != cudaSuccess) return WK_E_CUDA;
  // blocks the kernel flagged as beyond its exponent range are computed again (normally none)
  return p.redo ? launch_attn_fwd_redo(a, true, p.redo, st) : 0;
}
