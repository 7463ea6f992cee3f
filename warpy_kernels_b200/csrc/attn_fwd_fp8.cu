// FP8 (e4m3) flash-attention forward for sm_100a, head dimension 128.
//
// One CTA = 128 queries of one (batch, query head); two CTAs share an SM so that
// one CTA's softmax overlaps the other's tensor-core work.
//   warp 0      TMA producer: Q tile once, then K and V tiles (128 keys x 128 bytes,
//               128-byte swizzle) into two-stage rings
//   warp 1      allocates 256 TMEM columns (S: 0..127, O: 128..255) and issues
//               tcgen05.mma kind::f8f6f4:  S = Q.K^T (both K-major from shared memory),
//               O += P.V (P read from TMEM, V MN-major from shared memory)
//   warps 2-5   softmax, one thread per query row: read S from TMEM, running maximum
//               with a lazily refreshed reference (O and the row sum are rescaled
//               only when the maximum grew by more than 2^4), P = 2^(S.beta - m_ref + 4)
//               rounded to e4m3 and written back over the S columns, fp32 row sums;
//               finally O . v_descale / l -> bf16, lse (base 2) and pmax
//
// Numerics follow the reference's forward (warpy_kernels/attn/fwd_base.py:297-360,
// 939-988; fwd_sm120.py:93-136): logits in base 2 with beta = softmax_scale .
// q_descale . k_descale . log2(e), bottom-right aligned causal mask, P stored with a
// power-of-two offset so that small probabilities stay above e4m3 subnormals, lse =
// m_ref + log2(l) - offset, pmax = 2^(m_true - lse), empty rows give out = 0,
// lse = +inf, pmax = 0.  The offset here is 2^4 instead of the reference's 2^8: the
// stale reference maximum may trail the true one by 2^4, and 2^(4+4) <= 448.
//
// Tensor-core bound: 4 . B . Hq . Nq . Nk . d flops (half of that when causal).
#include <math.h>

#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

constexpr int BM = 128;       // queries per CTA
constexpr int BN = 128;       // keys per tile
constexpr int D = 128;        // head dimension (bytes per row in e4m3)
constexpr int KV_STAGES = 2;
constexpr int TILE_BYTES = BN * D;  // 16 KiB
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0;
constexpr int O_COL = 128;
constexpr float P_OFFSET = 4.0f;   // log2 of the factor P is stored with
constexpr float RESCALE_TAU = 4.0f;  // refresh the reference maximum when it trails by more than this
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + 1024 + 256;

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
  int causal;
  int write_lse;
  int lse_natural;
  const int* seqused_k;  // [B] or null
  float softmax_scale;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 2)
attn_fwd_fp8_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = smem_base + TILE_BYTES;
  const uint32_t v_smem = k_smem + KV_STAGES * TILE_BYTES;
  const uint32_t bar_base = v_smem + KV_STAGES * TILE_BYTES;
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (1 + KV_STAGES + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (1 + 2 * KV_STAGES + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (1 + 3 * KV_STAGES + s); };
  const uint32_t s_full = bar_base + 8u * (1 + 4 * KV_STAGES);
  const uint32_t p_full = s_full + 8;
  const uint32_t o_full = s_full + 16;
  const uint32_t tmem_slot = s_full + 24;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int m_blk = gridDim.x - 1 - blockIdx.x;  // longest (latest) causal blocks first
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
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
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
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_4d(q_smem, &tmap_q, q_full, 0, m0, hq, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(k_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(k_full(s), TILE_BYTES);
        tma_load_4d(k_smem + s * TILE_BYTES, &tmap_k, k_full(s), 0, j * BN, hkv, b);
        if (!mbar_wait(v_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(v_full(s), TILE_BYTES);
        tma_load_4d(v_smem + s * TILE_BYTES, &tmap_v, v_full(s), 0, j * BN, hkv, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(0, 0, 0, 0, BM, BN);
      constexpr uint32_t idesc_pv = make_idesc(0, 0, 0, 1, BM, D);
      const uint32_t s_tmem = tmem_base + S_COL;
      const uint32_t o_tmem = tmem_base + O_COL;
      bool ok = mbar_wait(q_full, 0, p.status, WK_ERR_TIMEOUT_LOAD);
      const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(k_full(s), ph, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        tc_fence_after();
        const uint64_t k_desc = smem_desc_sw128(k_smem + s * TILE_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < D / 32; ++k) {
          // 32 e4m3 = 32 bytes along the head dimension inside the 128-byte swizzle span
          mma_f8_ss(s_tmem, q_desc + 2 * k, k_desc + 2 * k, idesc_qk, k != 0);
        }
        tc_commit(k_empty(s));
        tc_commit(s_full);
        if (!mbar_wait(p_full, j & 1, p.status, WK_ERR_TIMEOUT_P)) break;
        if (!mbar_wait(v_full(s), ph, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        tc_fence_after();
        // V tile: 128 keys (the MMA's K) x 128 bytes of head dim (the MMA's N): MN-major,
        // one 128-byte span wide, 8-key groups 1024 bytes apart, 32 keys per MMA = 4096 bytes
        const uint64_t v_desc = smem_desc_sw128(v_smem + s * TILE_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < BN / 32; ++k) {
          // P: 32 e4m3 per K step = 8 TMEM columns
          mma_f8_ts(o_tmem, s_tmem + 8 * k, v_desc + 256 * k, idesc_pv, (j | k) != 0);
        }
        tc_commit(v_empty(s));
        if (j == n_tiles - 1) tc_commit(o_full);
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row of the tile == TMEM lane
    const int row = m0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + S_COL;
    const uint32_t o_tmem = tmem_base + lane_addr + O_COL;
    const int sc = b * p.Hkv + hkv;
    const float beta = p.softmax_scale * p.q_descale[sc] * p.k_descale[sc] * 1.4426950408889634f;
    const float sv = p.v_descale[sc];
    const int row_limit = p.causal ? row + shift : nk - 1;  // last visible key of this row
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait_warp(s_full, j & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int key0 = j * BN;
      const bool tile_masked = (key0 + BN > nk) || (p.causal && key0 + BN - 1 > m0 + shift);
      const int limit = min(row_limit, nk - 1) - key0;  // columns > limit are masked

      // pass 1: row maximum of the raw scores
      float tmax = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_tmem + c * 32, v);
        tc_wait_ld();
        if (tile_masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i <= limit) tmax = fmaxf(tmax, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) tmax = fmaxf(tmax, __uint_as_float(v[i]));
        }
      }
      const float t = beta >= 0.f ? tmax * beta : -INFINITY;  // beta < 0 is rejected on the host
      m_true = fmaxf(m_true, t);
      const bool need = t > m_ref + RESCALE_TAU || (m_ref == -INFINITY && t > -INFINITY);
      float corr = 1.f;
      if (need) {
        corr = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - t);
        l *= corr;
        m_ref = t;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // the previous P.V has completed (s_full tracks every earlier MMA), so O is quiescent
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(o_tmem + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_st32(o_tmem + c * 32, v);
        }
        tc_wait_st();
      }

      // pass 2: P = 2^(s.beta - m_ref + offset) -> e4m3, written over the S columns already consumed
      const float bias = (m_ref == -INFINITY ? 0.f : -m_ref) + P_OFFSET;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_tmem + c * 32, v);
        tc_wait_ld();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = ex2_approx(fmaf(__uint_as_float(v[i]), beta, bias));
          if (tile_masked && c * 32 + i > limit) e = 0.f;
          pr[i] = e;
          l += e;
        }
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = pack_e4m3x4(pr[4 * i], pr[4 * i + 1], pr[4 * i + 2], pr[4 * i + 3]);
        tmem_st8(s_tmem + c * 8, w);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }

    // epilogue
    if (n_tiles > 0 && ok) ok = mbar_wait_warp(o_full, 0, p.status, WK_ERR_TIMEOUT_MMA);
    if (ok) {
      tc_fence_after();
      const bool empty = !(l > 0.f);
      const float inv = empty ? 0.f : sv / l;
      __nv_bfloat16* out_row =
          p.out + b * p.out_stride_b + hq * p.out_stride_h + static_cast<int64_t>(row) * p.out_stride_n;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld32(o_tmem + c * 32, v);
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
      if (p.write_lse && row < p.Nq) {
        const int64_t off = b * p.lse_stride_b + hq * p.lse_stride_h + row;
        const float lse = empty ? INFINITY : m_ref + log2f(l) - P_OFFSET;
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

extern "C" int wk_attn_fwd_fp8(const wk_attn_fwd_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nk <= 0 || a->d != D) return WK_E_ARG;
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
  int* status = status_word();
  if (!status) return WK_E_CUDA;

  CUtensorMap tq, tk, tv;
  const uint32_t box[4] = {D, BM, 1, 1};
  {
    const uint64_t dims[4] = {D, static_cast<uint64_t>(a->Nq), static_cast<uint64_t>(a->Hq),
                              static_cast<uint64_t>(a->B)};
    const uint64_t str[3] = {static_cast<uint64_t>(qs[2]), static_cast<uint64_t>(qs[1]),
                             static_cast<uint64_t>(qs[0])};
    int r = encode_tmap(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    const uint64_t dims[4] = {D, static_cast<uint64_t>(a->Nk), static_cast<uint64_t>(a->Hkv),
                              static_cast<uint64_t>(a->B)};
    const uint64_t strk[3] = {static_cast<uint64_t>(ks[2]), static_cast<uint64_t>(ks[1]),
                              static_cast<uint64_t>(ks[0])};
    const uint64_t strv[3] = {static_cast<uint64_t>(vs[2]), static_cast<uint64_t>(vs[1]),
                              static_cast<uint64_t>(vs[0])};
    int r = encode_tmap(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->k, dims, strk, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
    r = encode_tmap(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, a->v, dims, strv, box, CU_TENSOR_MAP_SWIZZLE_128B);
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
  p.causal = a->causal;
  p.write_lse = a->write_lse;
  p.lse_natural = a->lse_natural;
  p.seqused_k = a->seqused_k;
  p.softmax_scale = a->softmax_scale;
  p.status = status;

  if (allow_smem(reinterpret_cast<const void*>(attn_fwd_fp8_kernel), SMEM_BYTES)) return WK_E_CUDA;
  dim3 grid((a->Nq + BM - 1) / BM, a->Hq, a->B);
  attn_fwd_fp8_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}
