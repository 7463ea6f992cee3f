// FP8 (e4m3) flash-attention forward for sm_100a, head dimension 128.
//
// Two kernels share the numerics described below.  From 2048 keys on (and on request) the work goes to the wide
// kernel further down: one persistent CTA per SM with four softmax groups.  Shorter sequences, and always the query
// blocks that see at most 512 keys (two-term P), go to the kernel described first:
// one CTA = 128 queries of one (batch, query head), two CTAs per SM, key tiles of 64.
// 320 threads:
//   warp 0      TMA producer: Q tile once, then K and V tiles (64 keys x 128 bytes,
//               128-byte swizzle) into four-stage rings
//   warp 1      allocates 256 TMEM columns (two S buffers of 64 columns, O: 128..255) and
//               issues tcgen05.mma:  S = Q.K^T (kind::f8f6f4, both operands K-major from
//               shared memory) always two tiles ahead, so the softmax never waits for it;
//               O += P.V (kind::mxf8f6f4.block_scale, P read from TMEM, V MN-major from
//               shared memory) as soon as a tile's P is there
//   warps 2-9   softmax in two groups of four warps that take the key tiles in turn (group
//               g owns S buffer g); inside a group one thread per query row: read S from
//               TMEM, write P as MXFP8 back over the S columns (e4m3 codes plus one
//               power-of-two scale per row and 32 keys, both straight into TMEM), row sums;
//               finally O . v_descale / l -> bf16, lse (base 2) and pmax
//
// Numerics follow the reference's forward (warpy_kernels/attn/fwd_base.py:297-360,
// 939-988; fwd_sm120.py:93-136): logits in base 2 with beta = softmax_scale .
// q_descale . k_descale . log2(e), bottom-right aligned causal mask, lse =
// m_ref + log2(l), pmax = 2^(m_true - lse), empty rows give out = 0, lse = +inf,
// pmax = 0.  O is normalised by the exact row sum; the reference sums the rounded P instead
// (fwd_sm120.py:95-118), which measured worse here once the row maximum is stored exactly.
// Where the reference quantises P against each 128-key tile's own maximum
// ("tile_local") and rescales O by the ratio of consecutive references, this kernel
// quantises every block of 32 keys against its own exponent e_blk = m_ref + k, k the
// smallest integer with e_blk >= block maximum,
//   P8 = e4m3(2^(s.beta - e_blk + 8)),   scale = 2^(k - 8),
// and lets the block-scaled MMA apply the scale, so O accumulates in the units of one
// reference m_ref per row.  m_ref is the row maximum of the first tile (its largest
// probability is then stored exactly, 2^8, as in the reference) and never moves: block
// exponents above it are as good as below it.  Scores that outgrow it by more than 2^100
// (69 nats) cannot be represented; the kernel then flags the query block in the call's workspace and the block is
// computed again by attn_fwd_redo.cu with the exact row maximum (without a workspace: WK_ERR_RANGE in the status
// word).  Query blocks that see at most 512 keys carry P as two
// e4m3 terms (value + 2^-4 . residual): with so few keys the rounding of P would not
// average out.
//
// Tensor-core bound: 4 . B . Hq . Nq . Nk . d flops (half of that when causal).
#include <math.h>

#include <type_traits>

#include "attn_fwd_redo.h"
#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

// Cycle probe of the persistent kernel (compile with -DWK_FWD_PROBE; never part of the shipped library): lane 0 of a
// warp adds the cycles it spent between two marks to a global counter.
#ifdef WK_FWD_PROBE
__device__ unsigned long long g_fwd_probe[32];
// per-warp accumulators in shared memory (lane 0 only), flushed to the global counters once at the end
#define PROBE_SMEM __shared__ unsigned long long probe_acc[20][20]
#define PROBE_DECL long long probe_t = clock64()
#define PROBE(slot)                                                                        \
  do {                                                                                     \
    const long long probe_now = clock64();                                                 \
    if ((threadIdx.x & 31) == 0) probe_acc[threadIdx.x >> 5][slot] += probe_now - probe_t; \
    probe_t = probe_now;                                                                   \
  } while (0)
#define PROBE_COUNT(slot) do { if ((threadIdx.x & 31) == 0) probe_acc[threadIdx.x >> 5][slot] += 1; } while (0)
#define PROBE_INIT do { if ((threadIdx.x & 31) == 0) for (int i = 0; i < 20; ++i) probe_acc[threadIdx.x >> 5][i] = 0; } while (0)
#define PROBE_FLUSH do { if ((threadIdx.x & 31) == 0) for (int i = 0; i < 20; ++i) if (probe_acc[threadIdx.x >> 5][i]) atomicAdd(&g_fwd_probe[i], probe_acc[threadIdx.x >> 5][i]); } while (0)
#else
#define PROBE_SMEM
#define PROBE_DECL
#define PROBE(slot)
#define PROBE_COUNT(slot)
#define PROBE_INIT
#define PROBE_FLUSH
#endif

constexpr int BM = 128;       // queries per CTA
constexpr int BN = 64;        // keys per tile
constexpr int D = 128;        // bytes per row of a tile in shared memory: head dimension 128, or head dimension 64
                              // with the upper half of every row zero (filled in by TMA: the tensor maps
                              // describe 64-byte rows, the boxes are 128 bytes wide).  The kernels are
                              // instantiated for DH = 128 and 64; with 64 the products over the head
                              // dimension take two K steps instead of four, P.V has N = 64, and O is 64 columns.
constexpr int KV_STAGES = 4;
constexpr int Q_BYTES = BM * D;     // 16 KiB
constexpr int KV_BYTES = BN * D;    // 8 KiB
constexpr int THREADS = 320;
constexpr int GROUP_THREADS = 128;  // one softmax group
constexpr int TMEM_COLS = 256;
constexpr int S_COLS = 64;    // one S buffer; buffer b starts at column 64 b
constexpr int O_COL = 128;
constexpr int P_OFFSET = 8;          // a block's largest P is stored in (2^7, 2^8]
constexpr float MAX_BLOCK_EXP = 100.f;  // how far (log2) a block may rise above the row reference
// After the softmax the 64 columns of an S buffer are reused: block k of 32 keys keeps its P codes in columns
// [32 k, 32 k + 8) and its residual codes in [32 k + 8, 32 k + 16); the scale factors sit in 16..27.
constexpr int PLO_OFF = 8;
constexpr int SFA_COL = 16;
constexpr int SFB_COL = 20;
constexpr int SFA_LO_COL = 24;
constexpr int RESID_MAX_TILES = 8;   // query blocks that see at most this many key tiles carry the residual term
constexpr int XCH_BYTES = 7 * BM * 4;  // row reference plus (l, lq, m_true) of each group
constexpr int SMEM_BYTES = Q_BYTES + 2 * KV_STAGES * KV_BYTES + XCH_BYTES + 1024 + 256;

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  float* pmax;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  int64_t out_stride_b, out_stride_h, out_stride_n;  // elements
  int64_t lse_stride_b, lse_stride_h;                // elements
  int B, Hq, Hkv, Nq, Nk;
  int d;  // head dimension, 128 or 64 (the persistent kernel reads it at run time; the two-CTA kernel is instantiated)
  int causal;
  int write_lse;
  int lse_natural;
  const int* seqused_k;  // [B] or null
  float softmax_scale;
  int m_first;  // first query block of this launch (the grid covers gridDim.x blocks from here)
  int* status;
  int* redo;    // one flag per query block, or null: blocks whose scores outgrow the row reference are recomputed
};

// Some key of the row lies more than 2^MAX_BLOCK_EXP above the row reference: with a flag array the query block is
// marked for recomputation (attn_fwd_redo.cu) and what this kernel stores for it is overwritten; without one the
// status word says that the result is not to be trusted.
__device__ __noinline__ void report_out_of_range(const FwdParams& p, int b, int hq, int m_blk) {
  if (p.redo)
    p.redo[attn_fwd_flag_index(b, hq, m_blk, p.Hq, (p.Nq + 127) / 128)] = 1;
  else
    atomicCAS(p.status, 0, WK_ERR_RANGE);
}

// One block of 32 keys of one row: P codes (and the residual codes) and the sum of the exact values.
template <bool RESID>
__device__ __forceinline__ void softmax_block(const uint32_t (&sraw)[32], float beta, float bias, uint32_t (&w)[8],
                                              uint32_t (&wl)[8], float& sum_exact) {
  const uint64_t beta2 = pack_f32x2(beta, beta), bias2 = pack_f32x2(bias, bias);
  uint64_t acc01 = 0, acc23 = 0;  // packed fp32 partial sums of the exact values
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
    const uint16_t h01 = cvt_e4m3x2(p0, p1), h23 = cvt_e4m3x2(p2, p3);
    w[i] = static_cast<uint32_t>(h01) | (static_cast<uint32_t>(h23) << 16);
    if (RESID) {
      // second e4m3 term: what the first rounding lost, times 2^4
      float q0, q1, q2, q3;
      unpack_e4m3x2(h01, q0, q1);
      unpack_e4m3x2(h23, q2, q3);
      wl[i] = pack_e4m3x4((p0 - q0) * 16.f, (p1 - q1) * 16.f, (p2 - q2) * 16.f, (p3 - q3) * 16.f);
    }
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

// RESID: this instantiation handles the query blocks that see at most RESID_MAX_TILES key tiles and carries P
// as two e4m3 terms; the other instantiation handles all other blocks.  Both are launched on the full grid and
// a CTA leaves at once when the block is not of its kind.
template <bool RESID, int DH>
__global__ void __launch_bounds__(THREADS, 2)
attn_fwd_fp8_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
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
  // With few keys the e4m3 rounding of P does not average out; such blocks carry P as two e4m3 terms
  // (value + 2^-4 . residual) at the price of a second P.V product.
  // The two-term launch comes first in the stream and lets the main launch start beside it; the main launch in
  // turn does not end before the two-term one has (both write parts of the same output).
  if (RESID) pdl_launch_dependents();
  if ((n_tiles <= RESID_MAX_TILES) != RESID) {
    if (!RESID) pdl_wait();
    return;
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
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_4d(q_smem, &tmap_q, q_full, 0, m0, hq, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(k_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(k_full(s), KV_BYTES);
        tma_load_4d(k_smem + s * KV_BYTES, &tmap_k, k_full(s), 0, j * BN, hkv, b);
        if (!mbar_wait(v_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(v_full(s), KV_BYTES);
        tma_load_4d(v_smem + s * KV_BYTES, &tmap_v, v_full(s), 0, j * BN, hkv, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(0, 0, 0, 0, BM, BN);
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
        for (int k = 0; k < DH / 32; ++k) {
          // 32 e4m3 = 32 bytes along the head dimension inside the 128-byte swizzle span
          mma_f8_ss(s_tmem, q_desc + 2 * k, k_desc + 2 * k, idesc_qk, k != 0);
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
        // V tile: 64 keys (the MMA's K) x 128 bytes of head dim (the MMA's N): MN-major,
        // one 128-byte span wide, 8-key groups 1024 bytes apart, 32 keys per MMA = 4096 bytes
        const uint64_t v_desc = smem_desc_sw128(v_smem + s * KV_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < BN / 32; ++k) {
          // P: 32 e4m3 per K step = 8 TMEM columns at column 32 k; scale byte k of the row's scale word
          mma_mxf8_ts(o_tmem, s_tmem + 32 * k, v_desc + 256 * k, make_idesc_mx_major(BM, DH, k, 0, 0, 1),
                      s_tmem + SFA_COL, s_tmem + SFB_COL, (j | k) != 0);
        }
        if (RESID) {
#pragma unroll
          for (int k = 0; k < BN / 32; ++k) {
            mma_mxf8_ts(o_tmem, s_tmem + 32 * k + PLO_OFF, v_desc + 256 * k,
                        make_idesc_mx_major(BM, DH, k, 0, 0, 1), s_tmem + SFA_LO_COL, s_tmem + SFB_COL, 1);
          }
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
    const int sc = b * p.Hkv + hkv;
    const float beta = p.softmax_scale * p.q_descale[sc] * p.k_descale[sc] * 1.4426950408889634f;
    const float sv = p.v_descale[sc];
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

      uint32_t sf_word = 0, sf_word_lo = 0;
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
        const bool live = cm > -INFINITY;
        float kf = live ? ceilf(cm - m_ref) : 0.f;  // block exponent relative to the row reference
        // scores more than 2^100 above the first tile's maximum are not representable here: clamped, and the
        // epilogue reports the row (m_true - m_ref tells)
        kf = fminf(kf, MAX_BLOCK_EXP);
        const float bias = live ? (static_cast<float>(P_OFFSET) - kf) - m_ref : 0.f;
        uint32_t w[8], wl[8];
        float sum_exact;
        softmax_block<RESID>(sraw, beta, bias, w, wl, sum_exact);
        // the codes go to the first columns of the 32 score columns they were made from
        tmem_st8(s_tmem + c * 32, w);
        if (RESID) tmem_st8(s_tmem + c * 32 + PLO_OFF, wl);
        int sf = live ? 127 + static_cast<int>(kf) - P_OFFSET : 0;
        sf = min(max(sf, 0), 254);
        const float blk_scale = __uint_as_float(static_cast<uint32_t>(sf) << 23);
        if (live) l = fmaf(sum_exact, blk_scale, l);
        sf_word |= static_cast<uint32_t>(sf) << (8 * c);
        sf_word_lo |= static_cast<uint32_t>(max(sf - 4, 0)) << (8 * c);
      }
      // scale factors straight into TMEM: the MMA reads the scale of row r from lane r, column r / 32
      tmem_st1(s_tmem + SFA_COL + quad, sf_word);
      tmem_st4(s_tmem + SFB_COL, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
      if (RESID) tmem_st1(s_tmem + SFA_LO_COL + quad, sf_word_lo);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(grp));
    }
    if (!met) {
      // this group had no tile (or gave up on a wait): it still owes the other group the meeting above
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }

    // epilogue: the groups add up their sums; group g stores head-dim columns [DH / 2 . g, DH / 2 . (g + 1))
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
    if (grp == 0 && m_true - m_ref > MAX_BLOCK_EXP) report_out_of_range(p, b, hq, m_blk);
    if (ok) {
      tc_fence_after();
      const bool empty = !(l > 0.f);
      const float inv = empty ? 0.f : sv / l;
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
  if (!RESID) pdl_wait();
}

// ---------------------------------------------------------------------------------------------------------------
// Wide variant (query blocks that see more than RESID_MAX_TILES key tiles): one persistent CTA per SM, 608 threads,
// each working through a list of query blocks.
//
//   warp 0       TMA producer: Q of a block (two buffers), then its K and V tiles of 128 keys into four-stage rings
//   warp 1       S = Q.K^T for 128 keys at a time (four tcgen05.mma with N = 128: what a thread can issue per unit
//                of time is limited, and a shared-memory operand pair for N = 64 is bandwidth-bound) into one of
//                two 128-column S buffers
//   warp 2       O += P.V, 64 keys at a time as the groups deliver their P
//   warps 3-18   softmax in four groups of four warps: rounds of 128 keys alternate between the two S buffers,
//                the two groups of a buffer take 64 keys each.  A thread reads the 64 scores of its row into
//                registers and the buffer goes straight back to warp 1, so the next S is computed while the
//                exponentials run; P goes to a small TMEM region per group.  (With P written over S, a group
//                waited 1500-2500 cycles after every tile for the round trip P -> P.V -> next S.)  The groups also
//                store a block's output; meanwhile warps 0 and 1 are already at work on the next block.
//   TMEM (512 columns): S buffers 0..255 | group g: P codes 256 + 24 g .. + 15, scale word column + 16 + quad |
//                       unit scales for V 352..355 | O 384..511
//
// Work list: the grid has one CTA per query block (longest blocks of a head first), but a CTA that has finished
// issuing the loads of its block asks the hardware for the index of a CTA that has not started yet
// (clusterlaunchcontrol.try_cancel) and works on that block as well, and so on until none is left: the blocks are
// handed out one by one in launch order, as they would be to fresh CTAs, without the start-up and the drain of a
// CTA in between.  Rounds and blocks are counted through the CTA's whole life: every barrier parity below derives
// from those running counts.
// ---------------------------------------------------------------------------------------------------------------
constexpr int M_BN = 128;          // keys per round
constexpr int M_KV_BYTES = M_BN * D;
constexpr int M_GROUPS = 4;
constexpr int M_SOFTMAX_THREADS = M_GROUPS * GROUP_THREADS;
constexpr int M_THREADS = 96 + M_SOFTMAX_THREADS;
constexpr int M_TMEM_COLS = 512;
constexpr int M_P_COL = 256;       // group g: 256 + 24 g
constexpr int M_P_STRIDE = 24;
constexpr int M_SFA_OFF = 16;      // inside a group's P region
constexpr int M_SFB_COL = 352;
constexpr int M_O_COL = 384;
constexpr int M_XCH_HALF = (1 + 2 * M_GROUPS) * BM * 4;  // row reference plus (l, m_true) of each group
constexpr int M_XCH_BYTES = 2 * M_XCH_HALF;              // blocks alternate between the halves
constexpr int M_FIN_BYTES = M_SOFTMAX_THREADS * 16;  // what a thread remembers of a finished block
constexpr int M_SMEM_BYTES = 2 * Q_BYTES + 2 * KV_STAGES * M_KV_BYTES + M_XCH_BYTES + M_FIN_BYTES + 1024 + 512;

struct WideItem {
  int hq, b, hkv, m0, nk, shift, n_tiles, n_rounds;
};

constexpr int M_SCHED_SLOTS = 4;  // answers of the launch control in flight
constexpr int M_CONSUMERS = 3 + M_SOFTMAX_THREADS;  // threads that read every answer

// The query block of grid index (x, y, z); false if it belongs to the two-term variant's launch.
__device__ __forceinline__ bool wide_item(const FwdParams& p, uint32_t x, uint32_t y, uint32_t z, WideItem& it) {
  const int m_blk = p.m_first + gridDim.x - 1 - x;  // longest (latest) causal blocks first
  it.hq = y;
  it.b = z;
  it.hkv = it.hq / (p.Hq / p.Hkv);
  it.m0 = m_blk * BM;
  it.nk = p.seqused_k ? max(0, min(p.Nk, p.seqused_k[it.b])) : p.Nk;
  it.shift = it.nk - p.Nq;  // key j is visible to query i iff j <= i + shift (causal)
  int n_tiles = (it.nk + BN - 1) / BN;
  if (p.causal) {
    const int last_row = min(it.m0 + BM, p.Nq) - 1;
    const int last_key = last_row + it.shift;  // may be negative
    n_tiles = last_key < 0 ? 0 : min(n_tiles, last_key / BN + 1);
  }
  it.n_tiles = n_tiles;
  it.n_rounds = (n_tiles + 1) / 2;  // 128 keys each; the second half of the last one may be all masked
  return n_tiles > RESID_MAX_TILES;
}

// Stores a finished query block's output (called by every softmax thread: group `grp` stores head-dim columns
// [32 grp, 32 grp + 32) of row `r`) once all groups have published their sums in `xch` and the last P.V product has
// completed; false if a wait gave up.  Kept out of line: it runs once per block, and inlined into the tile loop it
// cost that loop registers.
__device__ __noinline__ bool wide_store_output(const FwdParams& p, uint32_t xch, uint32_t fin_addr, uint32_t sum_meet,
                                               uint32_t o_full, uint32_t o_free, uint32_t o_tmem, int grp, int r,
                                               int fin_ci) {
  int row, b, hq;
  float m_ref;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(row), "=r"(b), "=r"(hq), "=f"(m_ref)
               : "r"(fin_addr)
               : "memory");
  const int sc = b * p.Hkv + hq / (p.Hq / p.Hkv);
  if (!mbar_wait_warp(sum_meet, fin_ci & 1, p.status, WK_ERR_TIMEOUT_P)) return false;
  float l = 0.f, m_true = -INFINITY;
#pragma unroll
  for (int g = 0; g < M_GROUPS; ++g) {  // same order in every group: identical sums
    float l_g, mt_g;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(l_g) : "r"(xch + (1 + 2 * g) * BM * 4 + r * 4) : "memory");
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(mt_g) : "r"(xch + (2 + 2 * g) * BM * 4 + r * 4) : "memory");
    l += l_g;
    m_true = fmaxf(m_true, mt_g);
  }
  if (grp == 0 && m_true - m_ref > MAX_BLOCK_EXP) report_out_of_range(p, b, hq, row / BM);
  if (!mbar_wait_warp(o_full, fin_ci & 1, p.status, WK_ERR_TIMEOUT_MMA)) return false;
  tc_fence_after();
  const bool empty = !(l > 0.f);
  const float inv = empty ? 0.f : p.v_descale[sc] / l;
  const int col0 = 32 * grp;
  __nv_bfloat16* out_row =
      p.out + b * p.out_stride_b + hq * p.out_stride_h + static_cast<int64_t>(row) * p.out_stride_n + col0;
  {
    uint32_t v[32];
    // head dimension 64: the first two groups store it all (the others read columns nobody has written and drop them)
    tmem_ld32(o_tmem + col0, v);
    tc_wait_ld();
    // O is in registers: the next block's first P.V product may overwrite it
    tc_fence_before();
    mbar_arrive(o_free);
    if (col0 < p.d && row < p.Nq) {
      uint4* dst = reinterpret_cast<uint4*>(out_row);
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
  return true;
}

__global__ void __launch_bounds__(M_THREADS, 1)
attn_fwd_fp8_wide_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  PROBE_SMEM;
  PROBE_INIT;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;  // two buffers
  const uint32_t k_smem = q_smem + 2 * Q_BYTES;
  const uint32_t v_smem = k_smem + KV_STAGES * M_KV_BYTES;
  const uint32_t xch_smem = v_smem + KV_STAGES * M_KV_BYTES;  // exchange between the softmax groups
  const uint32_t fin_smem = xch_smem + M_XCH_BYTES;
  const uint32_t bar_base = fin_smem + M_FIN_BYTES;
  auto q_full = [&](int i) { return bar_base + 8u * i; };
  auto q_empty = [&](int i) { return bar_base + 8u * (2 + i); };
  // A thread that issues MMAs pays 100-150 cycles for every barrier operation while shared memory is busy, so a
  // round of 128 keys costs each of the two issuing threads as few of them as possible: K and V of a stage arrive
  // on one barrier, both groups of an S buffer announce their P on one barrier, and one commit per round
  // (round_done) tells the producer that the stage's K and V may be overwritten and the two groups that their P
  // regions may be.
  auto kv_full = [&](int s) { return bar_base + 8u * (4 + s); };                   // K and V of stage s have landed
  auto round_done = [&](int s) { return bar_base + 8u * (4 + KV_STAGES + s); };    // the round's P.V has completed
  const uint32_t misc_bar = bar_base + 8u * (4 + 4 * KV_STAGES);
  auto s_full = [&](int buf) { return misc_bar + 8u * buf; };        // S buffer `buf` holds a round's scores
  auto s_free = [&](int buf) { return misc_bar + 8u * (2 + buf); };  // both of its groups have read them
  auto p_full = [&](int buf) { return misc_bar + 8u * (4 + buf); };  // both groups of buffer `buf` have written P
  const uint32_t o_full = misc_bar + 8u * 12;    // the block's last P.V product has completed
  const uint32_t o_free = misc_bar + 8u * 13;    // every softmax thread has read its part of O
  const uint32_t ref_full = misc_bar + 8u * 14;  // the block's row references are published
  const uint32_t sum_meet = misc_bar + 8u * 15;  // every group has published its sums
  auto sched_full = [&](int i) { return misc_bar + 8u * (16 + i); };                   // answer i has landed
  auto sched_empty = [&](int i) { return misc_bar + 8u * (16 + M_SCHED_SLOTS + i); };  // and everybody has read it
  const uint32_t tmem_slot = misc_bar + 8u * (16 + 2 * M_SCHED_SLOTS);
  auto sched_resp = [&](int i) { return misc_bar + 8u * (18 + 2 * M_SCHED_SLOTS) + 16u * i; };  // 16-byte answers

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full(i), 1);
      mbar_init(q_empty(i), 1);
    }
    for (int i = 0; i < M_SCHED_SLOTS; ++i) {
      mbar_init(sched_full(i), 1);
      mbar_init(sched_empty(i), M_CONSUMERS);
    }
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(round_done(s), 1);
    }
    for (int buf = 0; buf < 2; ++buf) {
      mbar_init(s_full(buf), 1);
      mbar_init(s_free(buf), 2 * GROUP_THREADS);
      mbar_init(p_full(buf), 2 * GROUP_THREADS);
    }
    mbar_init(o_full, 1);
    mbar_init(o_free, M_SOFTMAX_THREADS);
    mbar_init(ref_full, GROUP_THREADS);
    mbar_init(sum_meet, M_SOFTMAX_THREADS);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, M_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  WideItem it;
  bool ok = true;
  bool valid = wide_item(p, blockIdx.x, blockIdx.y, blockIdx.z, it);  // false: nothing to do for this block here
  uint32_t n_blocks = 0;  // answers read so far
  // Reads the next answer of the launch control: false if no block was left (or the wait gave up: ok is false then).
  auto next_block = [&]() {
    const int slot = n_blocks % M_SCHED_SLOTS;
    if (!mbar_wait(sched_full(slot), (n_blocks / M_SCHED_SLOTS) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
      ok = false;
      return false;
    }
    uint32_t x, y, z;
    const bool got = launch_control_answer(sched_resp(slot), x, y, z);
    // the slot's next answer is written through the async proxy: order this read before it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(sched_empty(slot));
    ++n_blocks;
    if (got) valid = wide_item(p, x, y, z, it);
    return got;
  };
  if (warp == 0) {
    if (lane == 0) {
      int ci = -1;
      uint32_t gr = 0;  // rounds so far
      for (;;) {
        if (valid) {
        ++ci;
        const int qb = ci & 1;
        // the S products of the block before the previous one have read this Q buffer
        if (ci >= 2 && !mbar_wait(q_empty(qb), ((ci >> 1) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(q_full(qb), Q_BYTES);
        tma_load_4d(q_smem + qb * Q_BYTES, &tmap_q, q_full(qb), 0, it.m0, it.hq, it.b);
        for (int R = 0; R < it.n_rounds; ++R, ++gr) {
          const int s = gr % KV_STAGES;
          const uint32_t ph = (gr / KV_STAGES) & 1;
          // the stage is free when the P.V product of the round that used it last has completed
          if (!mbar_wait(round_done(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(kv_full(s), 2 * M_KV_BYTES);
          tma_load_4d(k_smem + s * M_KV_BYTES, &tmap_k, kv_full(s), 0, R * M_BN, it.hkv, it.b);
          tma_load_4d(v_smem + s * M_KV_BYTES, &tmap_v, kv_full(s), 0, R * M_BN, it.hkv, it.b);
        }
        }
        if (!ok) break;
        // this block's loads are on their way: ask for another block (the MMAs have rounds in hand meanwhile)
        const int slot = n_blocks % M_SCHED_SLOTS;
        if (n_blocks >= M_SCHED_SLOTS &&
            !mbar_wait(sched_empty(slot), ((n_blocks / M_SCHED_SLOTS) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY))
          break;
        mbar_expect_tx(sched_full(slot), 16);
        launch_control_try_cancel(sched_resp(slot), sched_full(slot));
        if (!next_block()) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- S = Q.K^T, a round of 128 keys at a time ---------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(0, 0, 0, 0, BM, M_BN);
      int ci = -1;
      uint32_t gr = 0;
      PROBE_DECL;
      for (;;) {
        if (valid) {
        ++ci;
        const int qb = ci & 1;
        const uint64_t q_desc = smem_desc_sw128(q_smem + qb * Q_BYTES, 16, 1024);
        PROBE(16);
        if (!mbar_wait(q_full(qb), (ci >> 1) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        PROBE(17);
        for (int R = 0; R < it.n_rounds; ++R, ++gr) {
          const int s = gr % KV_STAGES;
          const uint32_t ph = (gr / KV_STAGES) & 1;
          const int buf = gr & 1;
          // the buffer is free when both groups have the scores of the round before the previous one in registers
          PROBE(16);
          if (gr >= 2 && !mbar_wait(s_free(buf), ((gr >> 1) - 1) & 1, p.status, WK_ERR_TIMEOUT_P)) {
            ok = false;
            break;
          }
          PROBE(14);
          // K of the round, and its V on behalf of warp 2 (what that one does with V comes after this S, the
          // softmax and the hand-over of P)
          if (!mbar_wait(kv_full(s), ph, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          tc_fence_after();
          PROBE(15);
          const uint64_t k_desc = smem_desc_sw128(k_smem + s * M_KV_BYTES, 16, 1024);
          const uint32_t s_tmem = tmem_base + 128 * buf;
#pragma unroll
          for (int k = 0; k < D / 32; ++k) {
            // 32 e4m3 = 32 bytes along the head dimension inside the 128-byte swizzle span (two steps for d = 64)
            if (32 * k < p.d) mma_f8_ss(s_tmem, q_desc + 2 * k, k_desc + 2 * k, idesc_qk, k != 0);
          }
          tc_commit(s_full(buf));
        }
        if (ok) tc_commit(q_empty(qb));
        }
        if (!ok || !next_block()) break;
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ---- O += P.V, 64 keys at a time ------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t o_tmem = tmem_base + M_O_COL;
      // N = head dimension; the scale-factor id of A (the byte of the row's scale word) is added per K step
      const uint32_t idesc_pv = make_idesc_mx_major(BM, p.d, 0, 0, 0, 1);
      int ci = -1;
      uint32_t gr = 0;
      PROBE_DECL;
      for (;;) {
        if (valid) {
        ++ci;
        PROBE(11);
        // the softmax threads have read the previous block's O
        if (ci >= 1 && !mbar_wait(o_free, (ci - 1) & 1, p.status, WK_ERR_TIMEOUT_TMEM)) break;
        tc_fence_after();
        PROBE(12);
        for (int R = 0; ok && R < it.n_rounds; ++R, ++gr) {
          const int s = gr % KV_STAGES;
          const int buf = gr & 1;
          PROBE(11);
          // V tile: 128 keys (the MMA's K) x 128 bytes of head dim (the MMA's N): MN-major,
          // one 128-byte span wide, 8-key groups 1024 bytes apart, 32 keys per MMA = 4096 bytes
          const uint64_t v_desc = smem_desc_sw128(v_smem + s * M_KV_BYTES, 16, 1024);
          if (!mbar_wait(p_full(buf), (gr >> 1) & 1, p.status, WK_ERR_TIMEOUT_P)) {
            ok = false;
            break;
          }
          tc_fence_after();
          PROBE(10);
          PROBE_COUNT(13);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t p_tmem = tmem_base + M_P_COL + M_P_STRIDE * (2 * buf + h);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              // P: 32 e4m3 per K step = 8 TMEM columns; scale byte k of the row's scale word
              mma_mxf8_ts(o_tmem, p_tmem + 8 * k, v_desc + 256 * (2 * h + k), idesc_pv | (k << 29),
                          p_tmem + M_SFA_OFF, tmem_base + M_SFB_COL, (R | h | k) != 0);
            }
          }
          tc_commit(round_done(s));
        }
        if (ok) tc_commit(o_full);
        }
        if (!ok || !next_block()) break;
      }
    }
    __syncwarp();
  } else {
    // Group g works on S buffer g >> 1 (every second round) and there on keys [64 (g & 1), + 64).
    // Inside a group one thread owns one query row.
    const int quad = warp & 3;  // TMEM lanes [32 quad, 32 quad + 32) are the ones this warp may touch
    const int grp = (warp - 3) >> 2;
    const int buf = grp >> 1, half = grp & 1;
    const int r = quad * 32 + lane;  // row of the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + 128 * buf + 64 * half;
    const uint32_t p_tmem = tmem_base + lane_addr + M_P_COL + M_P_STRIDE * grp;
    const uint32_t o_tmem = tmem_base + lane_addr + M_O_COL;
    int ci = -1;
    uint32_t gr0 = 0;  // rounds of the blocks before this one
    bool unit_scales_set = false;
    // A barrier operation costs 100-300 cycles of latency while shared memory feeds the MMAs, and a thread's tile has
    // four of them.  Two are taken off its critical path: whether the next S and the P region are ready is asked
    // early (test_wait, answer used later), and the hand-over of a tile's P (wait for the TMEM stores, arrive) is
    // put off until the loads of the next tile's scores are on their way.
    bool s_ready = false;   // the scores of this group's next tile were already there when last asked
    bool handing_over = false;  // P of the last tile is stored but not yet announced
    auto hand_over = [&]() {
      if (handing_over) {
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(p_full(buf));
        handing_over = false;
      }
    };
    PROBE_DECL;

    // The output of a block is stored by the groups while they are already at work on the next block: its last P.V
    // products are still running when a group has finished its last tile, so the group first does its first tile of
    // the next block and stores the finished block's output after that (wide_store_output; what it needs of the
    // finished block waits in shared memory, not in registers of the tile loop).
    const uint32_t my_fin = fin_smem + (threadIdx.x - 96) * 16;
    bool pending = false;
    auto store_output = [&](int fin_ci) {
      return wide_store_output(p, xch_smem + (fin_ci & 1) * M_XCH_HALF, my_fin, sum_meet, o_full, o_free, o_tmem, grp, r,
                               fin_ci);
    };

    for (;;) {
      if (valid) {
      ++ci;
      const uint32_t xch = xch_smem + (ci & 1) * M_XCH_HALF;
      const uint32_t x_ref = xch + r * 4;
      const int row = it.m0 + r;
      const int sc = it.b * p.Hkv + it.hkv;
      const float beta = p.softmax_scale * p.q_descale[sc] * p.k_descale[sc] * 1.4426950408889634f;
      const int row_limit = p.causal ? row + it.shift : it.nk - 1;  // last visible key of this row
      // m_ref: reference exponent of the row, fixed by the first tile (O and the sums are in units of 2^-m_ref)
      // l: sum of the exact probabilities over this group's tiles (normaliser of O, lse, pmax)
      float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
      bool have_ref = false;

      for (uint32_t gr = gr0 + ((buf ^ gr0) & 1); gr < gr0 + it.n_rounds; gr += 2) {
        const uint32_t n = gr >> 1;  // this group's tiles so far
        const int j = 2 * static_cast<int>(gr - gr0) + half;  // the 64-key tile
        PROBE(7);
        if (!__all_sync(0xffffffffu, s_ready) &&
            !mbar_wait_warp(s_full(buf), n & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        PROBE(1);
        // the whole row of the tile into registers, then the S buffer goes back to the MMA thread
        uint32_t sraw[2][32];
        tmem_ld32(s_tmem, sraw[0]);
        tmem_ld32(s_tmem + 32, sraw[1]);
        hand_over();  // the previous tile's P, while the loads are in flight
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(s_free(buf));
        // is this group's P region free (the P.V product of its previous tile completed)?  Needed after the
        // exponentials; asked now so that the answer is there by then.
        const bool p_free = n == 0 || mbar_test_wait(round_done((gr - 2) % KV_STAGES), ((gr - 2) / KV_STAGES) & 1);
        PROBE(2);

        const int key0 = j * BN;
        const bool tile_masked = (key0 + BN > it.nk) || (p.causal && key0 + BN - 1 > it.m0 + it.shift);
        const int limit = min(row_limit, it.nk - 1) - key0;  // columns > limit are masked
        if (tile_masked) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > limit) sraw[c][i] = 0xff800000u;  // -inf
        }
        float cm[2];
        cm[0] = block_max(sraw[0]) * beta;  // beta > 0 (checked on the host)
        cm[1] = block_max(sraw[1]) * beta;
        PROBE(3);
        if (j == 0) {
          // the row reference: maximum of the first tile (every row that sees any key sees one here)
          m_ref = fmaxf(cm[0], cm[1]);
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(x_ref), "f"(m_ref) : "memory");
          mbar_arrive(ref_full);
          have_ref = true;
        } else if (!have_ref) {
          // this group's first tile of the block: pick up the reference the first group has published
          if (!mbar_wait_warp(ref_full, ci & 1, p.status, WK_ERR_TIMEOUT_P)) {
            ok = false;
            break;
          }
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(m_ref) : "r"(x_ref) : "memory");
          have_ref = true;
        }
        PROBE(4);
        // The codes of both 32-key blocks are computed into registers first; the group's P region is only needed
        // when they are stored, and by then the P.V product of the previous tile has long completed.
        uint32_t sf_word = 0;
        uint32_t w[2][8];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          m_true = fmaxf(m_true, cm[c]);
          const bool live = cm[c] > -INFINITY;
          float kf = live ? ceilf(cm[c] - m_ref) : 0.f;  // block exponent relative to the row reference
          // scores more than 2^100 above the first tile's maximum are not representable here: clamped, and
          // wide_store_output reports the row (m_true - m_ref tells)
          kf = fminf(kf, MAX_BLOCK_EXP);
          const float bias = live ? (static_cast<float>(P_OFFSET) - kf) - m_ref : 0.f;
          uint32_t wl[8];
          float sum_exact;
          softmax_block<false>(sraw[c], beta, bias, w[c], wl, sum_exact);
          int sf = live ? 127 + static_cast<int>(kf) - P_OFFSET : 0;
          sf = min(max(sf, 0), 254);
          const float blk_scale = __uint_as_float(static_cast<uint32_t>(sf) << 23);
          if (live) l = fmaf(sum_exact, blk_scale, l);
          sf_word |= static_cast<uint32_t>(sf) << (8 * c);
        }
        PROBE(5);
        if (!__all_sync(0xffffffffu, p_free)) {
          if (!mbar_wait_warp(round_done((gr - 2) % KV_STAGES), ((gr - 2) / KV_STAGES) & 1, p.status,
                              WK_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        PROBE(6);
        PROBE_COUNT(9);
        tmem_st8(p_tmem, w[0]);
        tmem_st8(p_tmem + 8, w[1]);
        // scale factors straight into TMEM: the MMA reads the scale of row r from lane r, column r / 32
        tmem_st1(p_tmem + M_SFA_OFF + quad, sf_word);
        if (!unit_scales_set) {
          tmem_st4(tmem_base + lane_addr + M_SFB_COL, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
          unit_scales_set = true;
        }
        handing_over = true;
        hand_over();
        s_ready = mbar_test_wait(s_full(buf), (n + 1) & 1);  // this group's next tile, in this block or the next
        if (pending) {
          // first tile after a finished block: its P is handed over (the P.V product waits for O to be read
          // anyway), now that block's output
          pending = false;
          PROBE(7);
          if (!store_output(ci - 1)) {
            ok = false;
            break;
          }
          PROBE(8);
        }
      }
      gr0 += it.n_rounds;
      if (!ok) break;
      hand_over();  // the block's last tile

      // the groups' sums; each group stores head-dim columns [32 g, 32 g + 32) of the output later (store_output)
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(xch + (1 + 2 * grp) * BM * 4 + r * 4), "f"(l) : "memory");
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(xch + (2 + 2 * grp) * BM * 4 + r * 4), "f"(m_true) : "memory");
      mbar_arrive(sum_meet);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_fin), "r"(row), "r"(it.b), "r"(it.hq), "f"(m_ref)
                   : "memory");
      pending = true;
      }
      if (!ok || !next_block()) break;
    }
    if (ok && pending) store_output(ci);
  }

  PROBE_FLUSH;
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, M_TMEM_COLS);
  }
  pdl_wait();  // does not end before the two-term launch, which started before this one, has
}

}  // namespace
}  // namespace wk

#ifdef WK_FWD_PROBE
extern "C" int wk_fwd_probe_read(unsigned long long* out, int clear) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpyFromSymbol(out, wk::g_fwd_probe, 32 * sizeof(unsigned long long)) != cudaSuccess) return -2;
  if (clear) {
    unsigned long long zero[32] = {};
    if (cudaMemcpyToSymbol(wk::g_fwd_probe, zero, sizeof(zero)) != cudaSuccess) return -2;
  }
  return 0;
}
#endif

extern "C" int wk_attn_fwd_fp8(const wk_attn_fwd_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nk <= 0 || (a->d != 128 && a->d != 64)) return WK_E_ARG;
  if (a->Hq % a->Hkv) return WK_E_ARG;
  if (!a->q || !a->k || !a->v || !a->out || !a->q_descale || !a->k_descale || !a->v_descale) return WK_E_ARG;
  if (a->write_lse && (!a->lse || !a->pmax)) return WK_E_ARG;
  if (!(a->softmax_scale > 0.f)) return WK_E_ARG;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) return WK_E_ARG;
  const int64_t* qs = a->q_strides;
  const int64_t* ks = a->k_strides;
  const int64_t* vs = a->v_strides;
  for (int i = 0; i < 3; ++i) {
    if (qs[i] % 16 || ks[i] % 16 || vs[i] % 16 || qs[i] <= 0 || ks[i] <= 0 || vs[i] <= 0) return WK_E_ARG;
    if (a->out_strides[i] % 8 || a->out_strides[i] <= 0) return WK_E_ARG;
  }
  if (a->B > 65535 || a->Hq > 65535) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;

  CUtensorMap tq, tk, tv, tk128, tv128;  // K and V in tiles of 64 keys and, for the wide variant, of 128
  const uint32_t box[4] = {D, BM, 1, 1};
  const uint32_t box_kv[4] = {D, BN, 1, 1};
  {
    // rows of a->d bytes under boxes of 128: with head dimension 64 TMA fills the upper half of every row with zeros
    const uint64_t dims[4] = {static_cast<uint64_t>(a->d), static_cast<uint64_t>(a->Nq), static_cast<uint64_t>(a->Hq),
                              static_cast<uint64_t>(a->B)};
    const uint64_t str[3] = {static_cast<uint64_t>(qs[2]), static_cast<uint64_t>(qs[1]),
                             static_cast<uint64_t>(qs[0])};
    int r = encode_tmap(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    const uint64_t dims[4] = {static_cast<uint64_t>(a->d), static_cast<uint64_t>(a->Nk), static_cast<uint64_t>(a->Hkv),
                              static_cast<uint64_t>(a->B)};
    const uint64_t strk[3] = {static_cast<uint64_t>(ks[2]), static_cast<uint64_t>(ks[1]),
                              static_cast<uint64_t>(ks[0])};
    const uint64_t strv[3] = {static_cast<uint64_t>(vs[2]), static_cast<uint64_t>(vs[1]),
                              static_cast<uint64_t>(vs[0])};
    int r = encode_tmap(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->k, dims, strk, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
    r = encode_tmap(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->v, dims, strv, box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
    const uint32_t box_kv128[4] = {D, M_BN, 1, 1};
    r = encode_tmap(&tk128, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->k, dims, strk, box_kv128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
    r = encode_tmap(&tv128, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->v, dims, strv, box_kv128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  FwdParams p;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = static_cast<float*>(a->lse);
  p.pmax = static_cast<float*>(a->pmax);
  p.q_descale = static_cast<const float*>(a->q_descale);
  p.k_descale = static_cast<const float*>(a->k_descale);
  p.v_descale = static_cast<const float*>(a->v_descale);
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
  p.d = a->d;
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

  const bool d64 = a->d == 64;
  const void* k_main = d64 ? reinterpret_cast<const void*>(attn_fwd_fp8_kernel<false, 64>)
                           : reinterpret_cast<const void*>(attn_fwd_fp8_kernel<false, 128>);
  const void* k_resid = d64 ? reinterpret_cast<const void*>(attn_fwd_fp8_kernel<true, 64>)
                            : reinterpret_cast<const void*>(attn_fwd_fp8_kernel<true, 128>);
  const void* k_wide = reinterpret_cast<const void*>(attn_fwd_fp8_wide_kernel);
  if (allow_smem(k_main, SMEM_BYTES) || allow_smem(k_resid, SMEM_BYTES) || allow_smem(k_wide, M_SMEM_BYTES))
    return WK_E_CUDA;
  // ctas_per_sm: 0 picks by the number of keys.  Measured with equal work (causal / full, TFLOP/s), the wide kernel
  // against the two-CTA kernel: 1024 keys 723 / 1066 against 723 / 1070, 2048 keys 1012 / 1289 against 989 / 1253,
  // 4096 keys 1215 / 1412 against 1149 / 1342, 8192 keys 1321 / 1488 against 1192 / 1348, 16384 keys (causal) 1417
  // against 1140
  if (a->ctas_per_sm < 0 || a->ctas_per_sm > 2) return WK_E_ARG;
  const bool wide = a->ctas_per_sm == 1 || (a->ctas_per_sm == 0 && a->Nk >= 2048);
  const int num_m = (a->Nq + BM - 1) / BM;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Query blocks that see few key tiles run the two-term variant.  The tile count never decreases with the
  // block index, so without per-batch key lengths the two variants get disjoint block ranges; with seqused_k
  // both cover the whole grid and every CTA picks its variant itself.
  int m_split = 0;
  if (!a->seqused_k) {
    const int shift = a->Nk - a->Nq;
    const int all_tiles = (a->Nk + BN - 1) / BN;
    for (int m = 0; m < num_m; ++m) {
      int n = all_tiles;
      if (a->causal) {
        const int last_key = (m * BM + BM < a->Nq ? m * BM + BM : a->Nq) - 1 + shift;
        n = last_key < 0 ? 0 : (last_key / BN + 1 < all_tiles ? last_key / BN + 1 : all_tiles);
      }
      if (n <= RESID_MAX_TILES) m_split = m + 1;
    }
  }
  const int main_first = a->seqused_k ? 0 : m_split;
  const int resid_count = a->seqused_k ? num_m : m_split;
  // The short blocks first: their CTAs are many and brief, and the main launch, allowed to start while they still
  // run (programmatic stream serialisation), fills the SMs as they leave instead of waiting for the last of them.
  if (resid_count > 0) {
    p.m_first = 0;
    void* args[] = {&tq, &tk, &tv, &p};
    if (cudaLaunchKernel(k_resid, dim3(resid_count, a->Hq, a->B), dim3(THREADS), args, SMEM_BYTES, st) != cudaSuccess)
      return WK_E_CUDA;
  }
  if (num_m - main_first > 0) {
    p.m_first = main_first;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_m - main_first, a->Hq, a->B);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = resid_count > 0 ? 1 : 0;
    // wide: one CTA per query block in the grid; the CTAs that start take over the blocks of those that have not yet
    cfg.blockDim = dim3(wide ? M_THREADS : THREADS);
    cfg.dynamicSmemBytes = wide ? M_SMEM_BYTES : SMEM_BYTES;
    void* args[] = {&tq, wide ? &tk128 : &tk, wide ? &tv128 : &tv, &p};
    if (cudaLaunchKernelExC(&cfg, wide ? k_wide : k_main, args) != cudaSuccess) return WK_E_CUDA;
  }
  if (cudaGetLastError() != cudaSuccess) return WK_E_CUDA;
  // blocks the kernels above flagged as beyond their exponent range are computed again (normally none)
  return p.redo ? launch_attn_fwd_redo(a, false, p.redo, st) : 0;
}


