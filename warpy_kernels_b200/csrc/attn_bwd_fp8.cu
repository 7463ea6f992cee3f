// FP8 (e4m3) flash-attention backward for sm_100a, head dimension 128 or 64 (64: tiles keep their 128-byte rows in
// shared memory with the upper half zero -- the tensor maps describe 64-byte rows under 128-byte boxes and TMA fills
// in the rest -- while the products over the head dimension take two K steps instead of four and dQ / dK / dV are
// 64 columns wide; the two main kernels are instantiated per head dimension, the prep kernels read it at run time).
//
// Gradients with respect to the dequantised q, k, v (q = q_descale . q8 and so on):
//   S = alpha . q k^T,  P = softmax(S) = 2^(S . log2e - L)   (L: the forward's base-2 lse)
//   dV = P^T dO,  dP = dO v^T,  D = rowsum(dO * O),  dS = P * (dP - D),
//   dQ = alpha . dS k,  dK = alpha . dS^T q
// as in the reference's backward (warpy_kernels/attn/bwd_common.py:88-304, bwd_sm120.py:253-512):
// every product runs on the tensor core in e4m3.  Three kernels:
//
//  1. attn_bwd_prep4_kernel (HBM-bound; attn_bwd_prep_kernel for rows that do not start on 16-byte
//     boundaries): per query row, dO -> e4m3 with a power-of-two row
//     scale g (as the MXFP8 quantiser picks it) and the two numbers per row the main kernels
//     read, log2(g) - L and -sum(dO8 . O).  The reference scales dO per
//     (batch, kv head) and carries a second residual term (bwd_common.py:133-266); a scale per
//     row keeps small rows precise without it.
//  2. attn_bwd_dkdv_kernel: a key block = 128 keys of one (batch, kv head), K and V resident in shared
//     memory, loop over the group's query heads and query tiles.  The grid has one CTA per key block; the
//     CTAs that start take over the blocks of those that have not (launch control, common.cuh), with K and V
//     double-buffered and the next block's first scores under way while dK and dV are stored.  Per 64 queries:
//       S^T = K Q^T and dP^T = V dO8^T            (tcgen05.mma kind::f8f6f4, into one score buffer in TMEM)
//       threads (four per key): scores into registers (the buffer is free again), then P^T . g and dS^T as
//                              MXFP8: e4m3 codes and one power-of-two scale per key and 32 queries into TMEM
//                              columns of their own
//       dV += (P g)^T dO8 and dK += dS^T Q8       (kind::mxf8f6f4, A from TMEM, B = the same
//                                                  Q / dO8 tiles read MN-major)
//     dV and dK stay in TMEM for the whole CTA (484 of 512 columns in use).
//  3. attn_bwd_dq_kernel: a query block = 128 queries of one (batch, query head), loop over key tiles,
//     recomputes S and dP, dQ += dS K in TMEM; the grid has one CTA per query block and the CTAs that start
//     take over the blocks of those that have not, as in the dK/dV kernel.  Recomputing instead of reducing dQ
//     across key blocks costs two more products but needs no atomics, no fp32 dQ buffer, no
//     post-pass, and is deterministic (the reference: bwd_sm120.py:742-756 red.global.add /
//     bwd_common.py:307-403 post kernel).
//
// Tensor-core bound: 10 . B . Hq . Nq . Nk . d flops of algorithmic work (half when causal).
#include <math.h>

#include <type_traits>

#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

// Cycle probe of the two main kernels (compile with -DWK_BWD_PROBE; never part of the shipped library): lane 0 of a
// warp adds the cycles it spent between two marks to a counter, slots 0..23 for the dK/dV kernel and 24..47 for the
// dQ kernel.
#ifdef WK_BWD_PROBE
__device__ unsigned long long g_bwd_probe[48];
// per-warp accumulators in shared memory (lane 0 only), flushed to the global counters once at the end
#define PROBE_SMEM __shared__ unsigned long long probe_acc[18][24]
#define PROBE_DECL long long probe_t = clock64()
// With -DWK_BWD_TRACE as well, the CTA with grid index (0, 0, 0) also writes the time of every mark (first 256 per warp).
#ifdef WK_BWD_TRACE
__device__ unsigned long long g_bwd_trace[2][20][256];
#define TRACE_VARS(which)                                                                \
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0; \
  const int trace_which = which;                                                         \
  int trace_n = 0
#define TRACE(slot)                                                                      \
  if (trace_on && trace_n < 256)                                                         \
  g_bwd_trace[trace_which][threadIdx.x >> 5][trace_n++] =                                \
      (static_cast<unsigned long long>(slot) << 56) | (static_cast<unsigned long long>(probe_now) & 0xffffffffffffffull)
#else
#define TRACE_VARS(which)
#define TRACE(slot)
#endif
#define PROBE(slot)                                                                        \
  do {                                                                                     \
    const long long probe_now = clock64();                                                 \
    if ((threadIdx.x & 31) == 0) probe_acc[threadIdx.x >> 5][slot] += probe_now - probe_t; \
    probe_t = probe_now;                                                                   \
    TRACE(slot);                                                                           \
  } while (0)
#define PROBE_COUNT(slot) do { if ((threadIdx.x & 31) == 0) probe_acc[threadIdx.x >> 5][slot] += 1; } while (0)
#define PROBE_INIT do { if ((threadIdx.x & 31) == 0) for (int i = 0; i < 24; ++i) probe_acc[threadIdx.x >> 5][i] = 0; } while (0)
#define PROBE_FLUSH(base) do { if ((threadIdx.x & 31) == 0) for (int i = 0; i < 24; ++i) if (probe_acc[threadIdx.x >> 5][i]) atomicAdd(&g_bwd_probe[(base) + i], probe_acc[threadIdx.x >> 5][i]); } while (0)
#else
#define PROBE_SMEM
#define TRACE_VARS(which)
#define PROBE_DECL
#define PROBE(slot)
#define PROBE_COUNT(slot)
#define PROBE_INIT
#define PROBE_FLUSH(base)
#endif

constexpr int BM = 128;  // queries per tile
constexpr int BN = 128;  // keys per tile
constexpr int D = 128;  // bytes per row of a tile in shared memory (the largest head dimension)
constexpr int TILE_BYTES = 128 * 128;
constexpr int SF_BYTES = 512;
constexpr int THREADS = 640;          // four warps with one working thread each (loads, MMAs), 16 element-wise warps
constexpr int FIRST_EW_WARP = 4;
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
  const float* v_descale;     // [B,Hkv]
  uint8_t* do8;               // [B,Hq,Nq,D] contiguous
  float* qstat;               // [B,Hq,Nq_pad/128][2][128]: per 128 rows the arrays log2(g) - L and -D / sv
  int64_t do_sb, do_sh, do_sn;
  int64_t o_sb, o_sh, o_sn;
  int64_t lse_sb, lse_sh;
  int B, Hq, Hkv, Nq, nq_pad, d;
};

// one warp per query row, 4 consecutive elements per lane
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const PrepParams p) {
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
  const bool mine = lane * 4 < p.d;  // head dimension 64: half the lanes hold zeros and only join the reductions
  const uint2 draw = mine ? *reinterpret_cast<const uint2*>(dsrc) : make_uint2(0, 0);
  const uint2 oraw = mine ? *reinterpret_cast<const uint2*>(osrc) : make_uint2(0, 0);
  float dv[4], ov[4];
  dv[0] = __uint_as_float(draw.x << 16);
  dv[1] = __uint_as_float(draw.x & 0xffff0000u);
  dv[2] = __uint_as_float(draw.y << 16);
  dv[3] = __uint_as_float(draw.y & 0xffff0000u);
  ov[0] = __uint_as_float(oraw.x << 16);
  ov[1] = __uint_as_float(oraw.x & 0xffff0000u);
  ov[2] = __uint_as_float(oraw.y << 16);
  ov[3] = __uint_as_float(oraw.y & 0xffff0000u);
  uint32_t amax = 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) amax = max(amax, __float_as_uint(dv[c]) & 0x7fffffffu);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  // the MXFP8 quantiser's scale: the row peak lands in (224, 448]
  int e = static_cast<int>((amax + 0x1fffffu) >> 23) - 8;
  e = min(max(e, 0), 254);
  const float inv = __uint_as_float(static_cast<uint32_t>(max(254 - e, 1)) << 23);
  const float log2_g = static_cast<float>(e - 127);  // g = 2^(e - 127) is the scale the e4m3 codes carry
  const uint16_t c01 = cvt_e4m3x2(dv[0] * inv, dv[1] * inv);
  const uint16_t c23 = cvt_e4m3x2(dv[2] * inv, dv[3] * inv);
  float q0, q1, q2, q3;
  unpack_e4m3x2(c01, q0, q1);
  unpack_e4m3x2(c23, q2, q3);
  float dsum = (q0 * ov[0] + q1 * ov[1]) + (q2 * ov[2] + q3 * ov[3]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
  uint8_t* dst = p.do8 + ((static_cast<int64_t>(b) * p.Hq + h) * p.Nq + i) * p.d + lane * 4;
  if (mine) *reinterpret_cast<uint32_t*>(dst) = static_cast<uint32_t>(c01) | (static_cast<uint32_t>(c23) << 16);
  if (lane == 0) {
    const float sv = p.v_descale[b * p.Hkv + h / (p.Hq / p.Hkv)];
    const float L = p.lse[b * p.lse_sb + h * p.lse_sh + i];
    // With dO = g . dO8:  P g = 2^(s . beta - L + log2 g),  dV += (P g) dO8,  dS = (P g) . (sv . dP8 - sum(dO8 . O)),
    // so the main kernels need two numbers per query and no multiplication by g
    stat[0] = log2_g - L;
    stat[128] = -dsum;
  }
}

// The same for tensors whose strides are multiples of 8 elements: four query rows per warp, 8 lanes per row and 16
// consecutive elements per lane, read with 16-byte loads (64 bytes in flight per thread instead of 16: the kernel is
// HBM-bound and the one-row-per-warp form reached a third of the copy bandwidth).
__global__ void __launch_bounds__(256) attn_bwd_prep4_kernel(const PrepParams p) {
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
  const bool mine = sub * 16 < p.d;  // head dimension 64: half the lanes hold zeros and only join the reductions
  uint4 draw[2] = {}, oraw[2] = {};
  if (live && mine) {
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
  uint32_t amax = 0;
#pragma unroll
  for (int c = 0; c < 8; ++c) amax = max(amax, max((dw[c] << 16) & 0x7fffffffu, dw[c] & 0x7fff0000u));
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  // the MXFP8 quantiser's scale: the row peak lands in (224, 448]
  int e = static_cast<int>((amax + 0x1fffffu) >> 23) - 8;
  e = min(max(e, 0), 254);
  const float inv = __uint_as_float(static_cast<uint32_t>(max(254 - e, 1)) << 23);
  const float log2_g = static_cast<float>(e - 127);  // g = 2^(e - 127) is the scale the e4m3 codes carry
  uint32_t codes[4];
  float dsum = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint16_t cc = cvt_e4m3x2(__uint_as_float(dw[c] << 16) * inv, __uint_as_float(dw[c] & 0xffff0000u) * inv);
    float q0, q1;
    unpack_e4m3x2(cc, q0, q1);
    dsum += q0 * __uint_as_float(ow[c] << 16) + q1 * __uint_as_float(ow[c] & 0xffff0000u);
    if (c & 1) codes[c >> 1] |= static_cast<uint32_t>(cc) << 16;
    else codes[c >> 1] = cc;
  }
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
  // the two values of row i sit 128 floats apart inside the row's tile of 128
  float* stat = p.qstat + ((static_cast<int64_t>(b) * p.Hq + h) * p.nq_pad + (i & ~127)) * 2 + (i & 127);
  if (!live) {
    // padding rows: lse = +inf makes every probability zero
    if (sub < 2) stat[sub * 128] = sub == 0 ? -INFINITY : 0.f;
    return;
  }
  uint8_t* dst = p.do8 + ((static_cast<int64_t>(b) * p.Hq + h) * p.Nq + i) * p.d + sub * 16;
  if (mine) *reinterpret_cast<uint4*>(dst) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
  if (sub == 0) {
    const float L = p.lse[b * p.lse_sb + h * p.lse_sh + i];
    stat[0] = log2_g - L;
    stat[128] = -dsum;
  }
}

// ---------------------------------------------------------------------------
// helpers shared by the two main kernels
// ---------------------------------------------------------------------------
// Power-of-two scale for a block whose largest magnitude has the fp32 bit pattern `amax_bits`:
// the scaled peak lands in [128, 256).  Returns the ue8m0 byte; `inv` is the multiplier.
__device__ __forceinline__ uint32_t block_scale(uint32_t amax_bits, float& inv) {
  const int eb = static_cast<int>(amax_bits >> 23);
  const int sf = max(eb - 7, 0);
  inv = __uint_as_float(static_cast<uint32_t>(254 - sf) << 23);
  return static_cast<uint32_t>(sf);
}

// Four consecutive floats from shared memory (the row records: every thread reads the same address, a broadcast).
__device__ __forceinline__ float4 lds_f4(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}

// The element-wise code keeps a block of 32 values as 16 packed fp32 pairs (fma/mul.f32x2 work on two at once).
__device__ __forceinline__ void quantize_block_to_tmem(const uint64_t (&x)[16], uint32_t taddr, float inv) {
  const uint64_t inv2 = pack_f32x2(inv, inv);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float a, b, c, d;
    unpack_f32x2(mul_f32x2(x[2 * i], inv2), a, b);
    unpack_f32x2(mul_f32x2(x[2 * i + 1], inv2), c, d);
    w[i] = pack_e4m3x4(a, b, c, d);
  }
  tmem_st8(taddr, w);
}

// Largest magnitude of 32 values, as an fp32 bit pattern.
__device__ __forceinline__ uint32_t absmax_bits(const uint64_t (&x)[16]) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    float v0, v1, v2, v3, v4, v5, v6, v7;
    unpack_f32x2(x[i + 0], v0, v1);
    unpack_f32x2(x[i + 1], v2, v3);
    unpack_f32x2(x[i + 2], v4, v5);
    unpack_f32x2(x[i + 3], v6, v7);
    a0 = max3_abs(a0, v0, v1);
    a1 = max3_abs(a1, v2, v3);
    a2 = max3_abs(a2, v4, v5);
    a3 = max3_abs(a3, v6, v7);
  }
  return __float_as_uint(fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)));
}

// Largest of 32 values that are all >= 0, as an fp32 bit pattern.
__device__ __forceinline__ uint32_t max_bits_nonneg(const uint64_t (&x)[16]) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    float v0, v1, v2, v3, v4, v5, v6, v7;
    unpack_f32x2(x[i + 0], v0, v1);
    unpack_f32x2(x[i + 1], v2, v3);
    unpack_f32x2(x[i + 2], v4, v5);
    unpack_f32x2(x[i + 3], v6, v7);
    a0 = max3(a0, v0, v1);
    a1 = max3(a1, v2, v3);
    a2 = max3(a2, v4, v5);
    a3 = max3(a3, v6, v7);
  }
  return __float_as_uint(fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)));
}

struct BwdParams {
  const float* qstat;    // [B,Hq,nq_pad/128][2][128]: log2(g) - L and -sum(dO8 . O) of 128 rows
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
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
constexpr int A_STAGES = 4;
constexpr int A_STAT_BYTES = BM * 8;
constexpr int A_STAGE_BYTES = 2 * TILE_BYTES + A_STAT_BYTES;
constexpr int SCHED_SLOTS = 4;  // answers of the launch control in flight
// More than half an SM's shared memory: each CTA allocates all 512 TMEM columns, so a second resident CTA could
// only spin in tcgen05.alloc.
constexpr int A_SMEM_BYTES = 4 * TILE_BYTES + A_STAGES * A_STAGE_BYTES + 1024 + 512;
static_assert(A_SMEM_BYTES > 120 * 1024 && A_SMEM_BYTES <= 227 * 1024, "one CTA per SM");
static_assert(A_STAGE_BYTES % 1024 == 0, "tiles of a stage start on swizzle-atom boundaries");
// TMEM columns.  One buffer for the scores of 64 queries (S^T and dP^T), which the two groups of element-wise
// threads take turns on; the e4m3 codes they produce and the codes' scale words live apart from it, so that the
// buffer is free for the next product as soon as its scores are in registers.  Unit = 64 queries of a tile (h = 0,
// 1); block k = 0, 1 of a unit = 32 queries = the K extent of one block-scaled product.
constexpr int A_ST_COL = 0, A_DPT_COL = 64;
constexpr int A_PC_COL = 128;   // (P g)^T codes: 8 columns per (h, k)
constexpr int A_DSC_COL = 160;  // dS^T codes, the same
constexpr int A_SF_COL = 192;   // per (h, k) 8 columns: the P scales in 0..3, the dS scales in 4..7
constexpr int A_SF_UNIT_COL = 224;  // scale 1 for the B operands, written once
constexpr int A_DV_COL = 256, A_DK_COL = 384;

template <int DH>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // K and V of a key block: two buffers, the blocks of the CTA's list alternate between them
  auto k_smem = [&](int kb) { return smem_base + kb * 2 * TILE_BYTES; };
  auto v_smem = [&](int kb) { return smem_base + kb * 2 * TILE_BYTES + TILE_BYTES; };
  const uint32_t stage_smem = smem_base + 4 * TILE_BYTES;  // per stage: Q tile, dO tile, row records
  const uint32_t bar_base = stage_smem + A_STAGES * A_STAGE_BYTES;
  auto kv_full = [&](int kb) { return bar_base + 8u * kb; };
  auto kv_empty = [&](int kb) { return bar_base + 8u * (2 + kb); };  // the S products of the block have read K and V
  auto q_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto q_empty = [&](int s) { return bar_base + 8u * (4 + A_STAGES + s); };
  // per group of element-wise threads (h = 0, 1: the group takes the units with that h)
  const uint32_t unit_bars = bar_base + 8u * (4 + 2 * A_STAGES);
  auto s_full = [&](int h) { return unit_bars + 8u * h; };         // the unit's S^T and dP^T are in the buffer
  auto s_free = [&](int h) { return unit_bars + 8u * (2 + h); };   // ... and now in the group's registers
  auto p_full = [&](int h) { return unit_bars + 8u * (4 + h); };   // the unit's codes and scales are in TMEM
  auto ts_done = [&](int h) { return unit_bars + 8u * (6 + h); };  // ... and the dV / dK products have read them
  const uint32_t acc_full = unit_bars + 8u * 8;  // dK and dV of the block are complete
  const uint32_t acc_free = acc_full + 8;        // and every element-wise thread has read its part
  auto sched_full = [&](int i) { return acc_free + 8u * (1 + i); };                  // answer i has landed
  auto sched_empty = [&](int i) { return acc_free + 8u * (1 + SCHED_SLOTS + i); };  // and everybody has read it
  const uint32_t tmem_slot = acc_free + 8u * (1 + 2 * SCHED_SLOTS);
  auto sched_resp = [&](int i) { return acc_free + 8u * (3 + 2 * SCHED_SLOTS) + 16u * i; };  // 16-byte answers

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  PROBE_SMEM;
  PROBE_INIT;
  TRACE_VARS(0);
  const int group = p.Hq / p.Hkv;
  const int shift = p.Nk - p.Nq;
  const int num_m = (p.Nq + BM - 1) / BM;

  if (threadIdx.x == 0) {
    for (int kb = 0; kb < 2; ++kb) {
      mbar_init(kv_full(kb), 1);
      mbar_init(kv_empty(kb), 2);  // both score threads
    }
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full(h), 2);  // S^T and dP^T come from two threads
      mbar_init(s_free(h), HALF_THREADS);
      mbar_init(p_full(h), HALF_THREADS);
      mbar_init(ts_done(h), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_free, 2 * HALF_THREADS);
    for (int i = 0; i < SCHED_SLOTS; ++i) {
      mbar_init(sched_full(i), 1);
      mbar_init(sched_empty(i), 4 + 2 * HALF_THREADS);  // the TMA thread, three MMA threads, the element-wise threads
    }
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

  // The CTA's list of key blocks: its own grid index first, then the indices of CTAs that have not started, handed
  // out by the launch control (common.cuh) one at a time.  Tiles and blocks are counted through the CTA's whole life;
  // every barrier parity below derives from those running counts.
  struct KeyBlock {
    int n0, hkv, b, m_first, tiles_per_head, n_iter;
  } blk;
  auto set_block = [&](uint32_t x, uint32_t y, uint32_t z) {
    blk.n0 = x * BN;
    blk.hkv = y;
    blk.b = z;
    // first query tile that sees a key of this block (bottom-right aligned causal mask)
    blk.m_first = p.causal ? min(num_m, max(0, blk.n0 - shift) / BM) : 0;
    blk.tiles_per_head = num_m - blk.m_first;
    blk.n_iter = group * blk.tiles_per_head;
  };
  set_block(blockIdx.x, blockIdx.y, blockIdx.z);
  bool ok = true;
  uint32_t n_answers = 0;  // answers read so far
  // Reads the next answer of the launch control: false if no block was left (or the wait gave up: ok is false then).
  auto next_block = [&]() {
    const int slot = n_answers % SCHED_SLOTS;
    if (!mbar_wait(sched_full(slot), (n_answers / SCHED_SLOTS) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
      ok = false;
      return false;
    }
    uint32_t x, y, z;
    const bool got = launch_control_answer(sched_resp(slot), x, y, z);
    // the slot's next answer is written through the async proxy: order this read before it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(sched_empty(slot));
    ++n_answers;
    if (got) set_block(x, y, z);
    return got;
  };

  if (warp == 0) {
    if (lane == 0) {
      int ci = -1;      // blocks with work so far
      uint32_t gt = 0;  // tiles so far
      for (;;) {
        if (blk.n_iter > 0) {
          ++ci;
          const int kb = ci & 1;
          // the S products of the block before the previous one have read this pair of buffers
          if (ci >= 2 && !mbar_wait(kv_empty(kb), ((ci >> 1) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(kv_full(kb), 2 * TILE_BYTES);
          tma_load_4d(k_smem(kb), &tmap_k, kv_full(kb), 0, blk.n0, blk.hkv, blk.b);
          tma_load_4d(v_smem(kb), &tmap_v, kv_full(kb), 0, blk.n0, blk.hkv, blk.b);
          for (int it = 0; it < blk.n_iter; ++it, ++gt) {
            const int s = gt % A_STAGES;
            const uint32_t ph = (gt / A_STAGES) & 1;
            const int hq = blk.hkv * group + it / blk.tiles_per_head;
            const int m0 = (blk.m_first + it % blk.tiles_per_head) * BM;
            if (!mbar_wait(q_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) {
              ok = false;
              break;
            }
            const uint32_t base = stage_smem + s * A_STAGE_BYTES;
            mbar_expect_tx(q_full(s), A_STAGE_BYTES);
            tma_load_4d(base, &tmap_q, q_full(s), 0, m0, hq, blk.b);
            tma_load_4d(base + TILE_BYTES, &tmap_do, q_full(s), 0, m0, hq, blk.b);
            bulk_load(base + 2 * TILE_BYTES,
                      p.qstat + ((static_cast<int64_t>(blk.b) * p.Hq + hq) * p.nq_pad + m0) * 2, A_STAT_BYTES,
                      q_full(s));
          }
          if (!ok) break;
        }
        // this block's loads are on their way: ask for another block
        const int slot = n_answers % SCHED_SLOTS;
        if (n_answers >= SCHED_SLOTS &&
            !mbar_wait(sched_empty(slot), ((n_answers / SCHED_SLOTS) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY))
          break;
        mbar_expect_tx(sched_full(slot), 16);
        launch_control_try_cancel(sched_resp(slot), sched_full(slot));
        if (!next_block()) break;
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 2) {
    if (lane == 0) {
      // The CTA's work is a sequence of units: 64 queries (h = 0, 1) of a query tile of a key block, block after
      // block.  Unit n = 2 g + h (g: tiles so far) goes to element-wise group h.  The scores of a unit go into the
      // one score buffer as soon as the other group holds the unit before it in registers: S^T = K Q^T from this
      // thread in warp 1, dP^T = V dO8^T from the one in warp 2, side by side (the time from the buffer's release
      // to its next scores is on every unit's critical path, and one thread needs ~90 cycles per MMA it issues
      // here); a third thread (warp 3) issues the sums.
      const int which = warp - 1;  // 0: S^T, 1: dP^T
      constexpr uint32_t idesc_ss = make_idesc(0, 0, 0, 0, BN, BM / 2);
      const uint32_t d_tmem = tmem_base + (which == 0 ? A_ST_COL : A_DPT_COL);
      // Descriptors as (low word, shared high word): the tiles' low words are set up once, a K step or a row block
      // is one 32-bit add.
      const uint32_t desc_hi = smem_desc_sw128_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(which == 0 ? k_smem(0) : v_smem(0), 16);
      const uint32_t a_lo1 = smem_desc_lo(which == 0 ? k_smem(1) : v_smem(1), 16);
      // B: the Q tile of the stage for S^T, the dO8 tile behind it for dP^T
      const uint32_t b_lo0 = smem_desc_lo(stage_smem, 16) + (which == 0 ? 0 : (TILE_BYTES >> 4));
      bool have = blk.n_iter > 0;
      while (ok && !have && next_block()) have = blk.n_iter > 0;
      int ci = 0;      // blocks with work so far
      uint32_t g = 0;  // tiles so far
      PROBE_DECL;
      while (ok && have) {
        const int kb = ci & 1, n_iter = blk.n_iter;
        const uint32_t a_lo = kb ? a_lo1 : a_lo0;
        if (!mbar_wait(kv_full(kb), (ci >> 1) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        for (int it = 0; ok && it < n_iter; ++it, ++g) {
          const int s = g % A_STAGES;
          if (!mbar_wait(q_full(s), (g / A_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          PROBE(0);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            // the unit before this one (the other group's) has left the score buffer
            const uint32_t n = 2 * g + h;
            if (n >= 1 && !mbar_wait(s_free(h ^ 1), ((n - 1) >> 1) & 1, p.status, WK_ERR_TIMEOUT_P)) {
              ok = false;
              break;
            }
            PROBE(1);
            tc_fence_after();
            // queries [64 h, 64 h + 64) of the tile: rows 64 h.. of the Q and dO8 tiles are 64 x 128 bytes further on
            // (+512 in descriptor units)
            const uint32_t b_lo = b_lo0 + s * (A_STAGE_BYTES >> 4) + 512 * h;
#pragma unroll
            for (int k = 0; k < DH / 32; ++k) mma_f8_ss_w(d_tmem, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc_ss, k != 0);
            tc_commit(s_full(h));
            PROBE(2);
            PROBE_COUNT(6);
          }
        }
        if (!ok) break;
        tc_commit(kv_empty(kb));  // this thread's products of the block have all been issued
        ++ci;
        have = false;
        while (ok && !have && next_block()) have = blk.n_iter > 0;
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    if (lane == 0) {
      // dV += (P g)^T dO8 and dK += dS^T Q8, unit after unit, each as soon as its group has written the codes.
      // B operands: the dO8 / Q8 tiles again, now read MN-major (K = queries, 32 per step = 4096 bytes, N = head
      // dimension)
      const uint32_t desc_hi = smem_desc_sw128_hi(1024);
      const uint32_t q_lo0 = smem_desc_lo(stage_smem, 16);
      const uint32_t idesc_ts = make_idesc_mx_major(BN, DH, 0, 0, 0, 1);
      const uint32_t unit_sf = tmem_base + A_SF_UNIT_COL;
      bool have = blk.n_iter > 0;
      while (ok && !have && next_block()) have = blk.n_iter > 0;
      int ci = 0;
      uint32_t g = 0;
      PROBE_DECL;
      while (ok && have) {
        const int n_iter = blk.n_iter;
        for (int it = 0; ok && it < n_iter; ++it, ++g) {
          const int s = g % A_STAGES;
          const uint32_t q_lo = q_lo0 + s * (A_STAGE_BYTES >> 4);
          const uint32_t do_lo = q_lo + (TILE_BYTES >> 4);
          // the tile has landed (the score threads saw that long ago; this thread reads the tile too)
          if (!mbar_wait(q_full(s), (g / A_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          PROBE(0);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(p_full(h), g & 1, p.status, WK_ERR_TIMEOUT_P)) {
              ok = false;
              break;
            }
            PROBE(3);
            // the element-wise threads have read the previous block's dK and dV
            if (it == 0 && h == 0 && ci >= 1 && !mbar_wait(acc_free, (ci - 1) & 1, p.status, WK_ERR_TIMEOUT_TMEM)) {
              ok = false;
              break;
            }
            PROBE(4);
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 2; ++k)
              mma_mxf8_ts_w(tmem_base + A_DV_COL, tmem_base + A_PC_COL + 8 * (2 * h + k), do_lo + 256 * (2 * h + k),
                            desc_hi, idesc_ts, tmem_base + A_SF_COL + 8 * (2 * h + k), unit_sf, (it | h | k) != 0);
#pragma unroll
            for (int k = 0; k < 2; ++k)
              mma_mxf8_ts_w(tmem_base + A_DK_COL, tmem_base + A_DSC_COL + 8 * (2 * h + k), q_lo + 256 * (2 * h + k),
                            desc_hi, idesc_ts, tmem_base + A_SF_COL + 8 * (2 * h + k) + 4, unit_sf, (it | h | k) != 0);
            tc_commit(ts_done(h));
            PROBE(5);
            PROBE_COUNT(6);
          }
          // every product that reads the stage is complete when this fires (the scores were read long ago)
          tc_commit(q_empty(s));
        }
        if (!ok) break;
        tc_commit(acc_full);
        ++ci;
        have = false;
        while (ok && !have && next_block()) have = blk.n_iter > 0;
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int c = (warp - FIRST_EW_WARP) >> 2;  // which block of 32 of the tile's 128 queries this thread handles
    const int half = c >> 1;         // the unit (and the group) the block belongs to
    const int r = quad * 32 + lane;  // key row of the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    // the block's scores in the buffer; where its codes and scale words go
    const uint32_t st_tmem = tmem_base + lane_addr + A_ST_COL + 32 * (c & 1);
    const uint32_t dpt_tmem = tmem_base + lane_addr + A_DPT_COL + 32 * (c & 1);
    const uint32_t pc_tmem = tmem_base + lane_addr + A_PC_COL + 8 * c;
    const uint32_t dsc_tmem = tmem_base + lane_addr + A_DSC_COL + 8 * c;
    const uint32_t sf_tmem = tmem_base + lane_addr + A_SF_COL + 8 * c + quad;
    if (c == 0) tmem_st4(tmem_base + lane_addr + A_SF_UNIT_COL, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
    int ci = -1;     // key blocks with work so far
    uint32_t g = 0;  // tiles so far
    PROBE_DECL;

    for (;;) {
    const int n0 = blk.n0, n_iter = blk.n_iter;
    const int key = n0 + r;
    const int sc = blk.b * p.Hkv + blk.hkv;
    const float beta = p.softmax_scale * p.q_descale[sc] * p.k_descale[sc] * LOG2E;
    const uint64_t sv2 = pack_f32x2(p.v_descale[sc], p.v_descale[sc]);
    if (n_iter > 0) ++ci;

    int mt = blk.m_first;  // the query tile, restarting with every query head of the group
    for (int it = 0; it < n_iter; ++it, ++g) {
      const int s = g % A_STAGES;
      const int m0 = mt * BM;
      if (++mt == num_m) mt = blk.m_first;
      if (!mbar_wait_warp(s_full(half), g & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      PROBE(8);
      tc_fence_after();
      // the tile's row records: arrays log2(g) - L and -sum(dO8 . O) of 128 queries each, read four at a time
      const uint32_t stat = stage_smem + s * A_STAGE_BYTES + 2 * TILE_BYTES;
      // query column c is visible to this key iff key < Nk and (not causal or key <= m0 + c + shift)
      const int first_col = key >= p.Nk ? BM : (p.causal ? max(0, key - shift - m0) : 0);
      // uniform over the CTA: does this (key block, query tile) pair contain any masked score?
      const bool tile_masked = (n0 + BN > p.Nk) || (p.causal && n0 + BN - 1 > m0 + shift);
      uint32_t sf_p, sf_d;
      {
        uint32_t sraw[32], draw[32];
        tmem_ld32(st_tmem, sraw);
        tmem_ld32(dpt_tmem, draw);
        tc_wait_ld();
        // the scores are in registers: the buffer may take the next unit
        tc_fence_before();
        mbar_arrive(s_free(half));
        PROBE(9);
        uint64_t pt[16], ds[16];  // (P g)^T and dS^T of this key for 32 queries, as packed pairs
        const uint64_t beta2 = pack_f32x2(beta, beta);
        // two copies of the loop, with and without the mask, behind one branch per tile (as predicated code the
        // comparisons and selects take two issue slots per score in every tile)
        auto scores_to_ds = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // the same addresses for every thread: shared-memory broadcasts
          const float4 el = lds_f4(stat + 16 * (c * 8 + i)), nd = lds_f4(stat + 16 * (32 + c * 8 + i));
          float x0, x1, x2, x3;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i]), __uint_as_float(sraw[4 * i + 1])), beta2,
                                 pack_f32x2(el.x, el.y)), x0, x1);
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[4 * i + 2]), __uint_as_float(sraw[4 * i + 3])), beta2,
                                 pack_f32x2(el.z, el.w)), x2, x3);
          float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
          if constexpr (decltype(masked)::value) {
            if (c * 32 + 4 * i + 0 < first_col) p0 = 0.f;
            if (c * 32 + 4 * i + 1 < first_col) p1 = 0.f;
            if (c * 32 + 4 * i + 2 < first_col) p2 = 0.f;
            if (c * 32 + 4 * i + 3 < first_col) p3 = 0.f;
          }
          pt[2 * i] = pack_f32x2(p0, p1);
          pt[2 * i + 1] = pack_f32x2(p2, p3);
          ds[2 * i] = mul_f32x2(pt[2 * i], fma_f32x2(pack_f32x2(__uint_as_float(draw[4 * i]), __uint_as_float(draw[4 * i + 1])),
                                                     sv2, pack_f32x2(nd.x, nd.y)));
          ds[2 * i + 1] =
              mul_f32x2(pt[2 * i + 1], fma_f32x2(pack_f32x2(__uint_as_float(draw[4 * i + 2]), __uint_as_float(draw[4 * i + 3])),
                                                 sv2, pack_f32x2(nd.z, nd.w)));
        }
        };
        if (tile_masked) scores_to_ds(std::true_type{});
        else scores_to_ds(std::false_type{});
        float inv_p, inv_d;
        const uint32_t bp = block_scale(max_bits_nonneg(pt), inv_p);  // P >= 0 and g > 0
        const uint32_t bd = block_scale(absmax_bits(ds), inv_d);
        PROBE(10);
        // the products of the group's previous unit have read its codes and scale words
        if (g >= 1 && !mbar_wait_warp(ts_done(half), (g - 1) & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        PROBE(11);
        tc_fence_after();
        quantize_block_to_tmem(pt, pc_tmem, inv_p);
        quantize_block_to_tmem(ds, dsc_tmem, inv_d);
        sf_p = bp;
        sf_d = bd;
      }
      // scale factors straight into TMEM: the MMA reads the scale of row r from lane r, column r / 32
      tmem_st1(sf_tmem, sf_p);
      tmem_st1(sf_tmem + 4, sf_d);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full(half));
      PROBE(12);
      PROBE_COUNT(15);
    }

    if (n_iter > 0 && ok) ok = mbar_wait_warp(acc_full, ci & 1, p.status, WK_ERR_TIMEOUT_MMA);
    PROBE(13);
    if (ok) {
      tc_fence_after();
      const float dk_scale = p.softmax_scale * p.q_descale[sc];
      const int64_t row_off = ((static_cast<int64_t>(blk.b) * p.Hkv + blk.hkv) * p.Nk + key) * DH;
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
            if (which == 1) {
              // dK and dV are in registers: the next block's first products may overwrite them
              tc_fence_before();
              mbar_arrive(acc_free);
            }
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
    PROBE(14);
    if (!ok || !next_block()) break;
    PROBE(16);
    }
  }
  PROBE_FLUSH(0);

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
constexpr int B_STAGES = 4;
constexpr int B_STAGE_BYTES = 2 * TILE_BYTES;  // K tile, V tile
constexpr int B_SMEM_BYTES = 4 * TILE_BYTES + B_STAGES * B_STAGE_BYTES + 1024 + 512;
static_assert(B_SMEM_BYTES > 120 * 1024 && B_SMEM_BYTES <= 227 * 1024, "one CTA per SM");
// TMEM columns: the scores of a whole key tile, dQ, and apart from the scores the dS codes and their scale words,
// twice each (tiles alternate), so that the score columns are free for the next tile's products as soon as the
// element-wise threads hold the scores in registers.
constexpr int B_S_COL = 0, B_DP_COL = 128, B_DQ_COL = 256;
constexpr int B_DSC_COL = 384;      // dS codes: per tile buffer 32 columns, 8 per block of 32 keys
constexpr int B_SF_COL = 448;       // their scales: per tile buffer 16 columns, 4 per block of 32 keys
constexpr int B_SF_UNIT_COL = 480;  // scale 1 for the B operand, written once
constexpr int EW_THREADS = 2 * HALF_THREADS;

template <int DH>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // Q and dO8 of a query block: two buffers, the blocks of the CTA's list alternate between them
  auto q_smem = [&](int qb) { return smem_base + qb * 2 * TILE_BYTES; };
  auto do_smem = [&](int qb) { return smem_base + qb * 2 * TILE_BYTES + TILE_BYTES; };
  const uint32_t stage_smem = smem_base + 4 * TILE_BYTES;
  const uint32_t bar_base = stage_smem + B_STAGES * B_STAGE_BYTES;
  auto q_full = [&](int qb) { return bar_base + 8u * qb; };
  auto q_empty = [&](int qb) { return bar_base + 8u * (2 + qb); };  // every product of the block has read Q and dO8
  auto kv_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (4 + B_STAGES + s); };
  const uint32_t s_full = bar_base + 8u * (4 + 2 * B_STAGES);  // S and dP of a tile are in TMEM
  const uint32_t s_free = s_full + 8;                          // ... and now in the element-wise threads' registers
  const uint32_t p_full = s_full + 16;                         // the tile's dS codes and scales are in TMEM
  auto ts_done = [&](int i) { return s_full + 24 + 8u * i; };  // ... and the dQ products have read them (buffer i)
  const uint32_t acc_full = s_full + 40;                       // dQ of the block is complete
  const uint32_t acc_free = s_full + 48;                       // and every element-wise thread has read its part
  auto sched_full = [&](int i) { return acc_free + 8u * (1 + i); };                  // answer i has landed
  auto sched_empty = [&](int i) { return acc_free + 8u * (1 + SCHED_SLOTS + i); };  // and everybody has read it
  const uint32_t tmem_slot = acc_free + 8u * (1 + 2 * SCHED_SLOTS);
  auto sched_resp = [&](int i) { return acc_free + 8u * (4 + 2 * SCHED_SLOTS) + 16u * i; };  // 16-byte answers, 16-byte aligned

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  PROBE_SMEM;
  PROBE_INIT;
  TRACE_VARS(1);
  PROBE_DECL;
  const int shift = p.Nk - p.Nq;
  const int group = p.Hq / p.Hkv;

  if (threadIdx.x == 0) {
    for (int qb = 0; qb < 2; ++qb) {
      mbar_init(q_full(qb), 1);
      mbar_init(q_empty(qb), 1);
    }
    for (int s = 0; s < B_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    mbar_init(s_full, 2);  // S and dP come from two threads
    mbar_init(s_free, EW_THREADS);
    mbar_init(p_full, EW_THREADS);
    mbar_init(ts_done(0), 1);
    mbar_init(ts_done(1), 1);
    mbar_init(acc_full, 1);
    mbar_init(acc_free, EW_THREADS);
    for (int i = 0; i < SCHED_SLOTS; ++i) {
      mbar_init(sched_full(i), 1);
      mbar_init(sched_empty(i), 4 + EW_THREADS);  // the TMA thread, three MMA threads, the element-wise threads
    }
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
  PROBE(20);
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  // The CTA's list of query blocks: its own grid index first, then the indices of CTAs that have not started, handed
  // out by the launch control (common.cuh) one at a time, in launch order (the blocks with the most key tiles
  // first).  Tiles and blocks are counted through the CTA's whole life; every barrier parity below derives from
  // those running counts.
  struct QueryBlock {
    int m0, hq, b, hkv, n_tiles;
  } blk;
  auto set_block = [&](uint32_t x, uint32_t y, uint32_t z) {
    blk.m0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(x)) * BM;
    blk.hq = y;
    blk.b = z;
    blk.hkv = blk.hq / group;
    int n = (p.Nk + BN - 1) / BN;
    if (p.causal) {
      const int last_key = min(blk.m0 + BM, p.Nq) - 1 + shift;
      n = last_key < 0 ? 0 : min(n, last_key / BN + 1);
    }
    blk.n_tiles = n;
  };
  set_block(blockIdx.x, blockIdx.y, blockIdx.z);
  bool ok = true;
  uint32_t n_answers = 0;  // answers read so far
  // Reads the next answer of the launch control: false if no block was left (or the wait gave up: ok is false then).
  auto next_block = [&]() {
    const int slot = n_answers % SCHED_SLOTS;
    if (!mbar_wait(sched_full(slot), (n_answers / SCHED_SLOTS) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
      ok = false;
      return false;
    }
    uint32_t x, y, z;
    const bool got = launch_control_answer(sched_resp(slot), x, y, z);
    // the slot's next answer is written through the async proxy: order this read before it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(sched_empty(slot));
    ++n_answers;
    if (got) set_block(x, y, z);
    return got;
  };

  if (warp == 0) {
    if (lane == 0) {
      int ci = -1;      // blocks with work so far
      uint32_t jt = 0;  // tiles so far
      for (;;) {
        if (blk.n_tiles > 0) {
          ++ci;
          const int qb = ci & 1;
          // the products of the block before the previous one have read this pair of buffers
          if (ci >= 2 && !mbar_wait(q_empty(qb), ((ci >> 1) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(q_full(qb), 2 * TILE_BYTES);
          tma_load_4d(q_smem(qb), &tmap_q, q_full(qb), 0, blk.m0, blk.hq, blk.b);
          tma_load_4d(do_smem(qb), &tmap_do, q_full(qb), 0, blk.m0, blk.hq, blk.b);
          for (int j = 0; j < blk.n_tiles; ++j, ++jt) {
            const int s = jt % B_STAGES;
            const uint32_t ph = (jt / B_STAGES) & 1;
            if (!mbar_wait(kv_empty(s), ph ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) {
              ok = false;
              break;
            }
            const uint32_t base = stage_smem + s * B_STAGE_BYTES;
            mbar_expect_tx(kv_full(s), B_STAGE_BYTES);
            tma_load_4d(base, &tmap_k, kv_full(s), 0, j * BN, blk.hkv, blk.b);
            tma_load_4d(base + TILE_BYTES, &tmap_v, kv_full(s), 0, j * BN, blk.hkv, blk.b);
          }
          if (!ok) break;
        }
        // this block's loads are on their way: ask for another block
        const int slot = n_answers % SCHED_SLOTS;
        if (n_answers >= SCHED_SLOTS &&
            !mbar_wait(sched_empty(slot), ((n_answers / SCHED_SLOTS) - 1) & 1, p.status, WK_ERR_TIMEOUT_EMPTY))
          break;
        mbar_expect_tx(sched_full(slot), 16);
        launch_control_try_cancel(sched_resp(slot), sched_full(slot));
        if (!next_block()) break;
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 3) {
    if (lane == 0) {
      // The scores of a key tile, issued as soon as the element-wise threads hold the tile before it in registers
      // (across query blocks too), so that the next tile's scores are waiting when they are done with the current
      // one: S = Q K^T from this thread in warp 1, dP = dO8 V^T from the one in warp 3, side by side (the time from
      // the columns' release to the next scores is on the critical path, and one thread needs ~90 cycles per MMA
      // it issues here).  The dQ products come from a third thread (warp 2).
      const int which = warp == 1 ? 0 : 1;  // 0: S, 1: dP
      constexpr uint32_t idesc_ss = make_idesc(0, 0, 0, 0, BM, BN);
      const uint32_t d_tmem = tmem_base + (which == 0 ? B_S_COL : B_DP_COL);
      // descriptors as (low word, shared high word), as in the dK/dV kernel
      const uint32_t desc_hi = smem_desc_sw128_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(which == 0 ? q_smem(0) : do_smem(0), 16);
      const uint32_t a_lo1 = smem_desc_lo(which == 0 ? q_smem(1) : do_smem(1), 16);
      // B: the K tile of the stage for S, the V tile behind it for dP
      const uint32_t b_lo0 = smem_desc_lo(stage_smem, 16) + (which == 0 ? 0 : (TILE_BYTES >> 4));
      bool have = blk.n_tiles > 0;
      while (ok && !have && next_block()) have = blk.n_tiles > 0;
      int ci = 0;
      uint32_t jt = 0;
      while (ok && have) {
        const int qb = ci & 1, n_tiles = blk.n_tiles;
        const uint32_t a_lo = qb ? a_lo1 : a_lo0;
        if (!mbar_wait(q_full(qb), (ci >> 1) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) break;
        for (int j = 0; j < n_tiles; ++j, ++jt) {
          const int s = jt % B_STAGES;
          if (!mbar_wait(kv_full(s), (jt / B_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          PROBE(0);
          if (jt >= 1 && !mbar_wait(s_free, (jt - 1) & 1, p.status, WK_ERR_TIMEOUT_P)) {
            ok = false;
            break;
          }
          // The dQ products of the tile before the previous one have read their codes: whoever sees this tile's
          // scores may overwrite that buffer of codes (the element-wise threads do not ask again)
          if (jt >= 2 && !mbar_wait(ts_done(jt & 1), ((jt >> 1) - 1) & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          PROBE(1);
          tc_fence_after();
          const uint32_t b_lo = b_lo0 + s * (B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < DH / 32; ++k) mma_f8_ss_w(d_tmem, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc_ss, k != 0);
          tc_commit(s_full);
          PROBE(2);
        }
        if (!ok) break;
        ++ci;
        have = false;
        while (ok && !have && next_block()) have = blk.n_tiles > 0;
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    if (lane == 0) {
      // dQ += dS K over a tile, as soon as the tile's codes are written: A = the dS codes, B = the K tile read
      // MN-major (32 keys per step = 4096 bytes)
      const uint32_t desc_hi = smem_desc_sw128_hi(1024);
      const uint32_t idesc_ts = make_idesc_mx_major(BM, DH, 0, 0, 0, 1);
      const uint32_t k_lo0 = smem_desc_lo(stage_smem, 16);
      bool have = blk.n_tiles > 0;
      while (ok && !have && next_block()) have = blk.n_tiles > 0;
      int ci = 0;
      uint32_t jt = 0;
      while (ok && have) {
        const int qb = ci & 1, n_tiles = blk.n_tiles;
        for (int j = 0; j < n_tiles; ++j, ++jt) {
          const int s = jt % B_STAGES;
          // the tile has landed (the score thread saw that long ago; this thread reads the tile too)
          if (!mbar_wait(kv_full(s), (jt / B_STAGES) & 1, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          PROBE(17);
          if (!mbar_wait(p_full, jt & 1, p.status, WK_ERR_TIMEOUT_P)) {
            ok = false;
            break;
          }
          PROBE(3);
          // the element-wise threads have read the previous block's dQ
          if (j == 0 && ci >= 1 && !mbar_wait(acc_free, (ci - 1) & 1, p.status, WK_ERR_TIMEOUT_TMEM)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t k_lo = k_lo0 + s * (B_STAGE_BYTES >> 4);
          const uint32_t codes = tmem_base + B_DSC_COL + 32 * (jt & 1), sf = tmem_base + B_SF_COL + 16 * (jt & 1);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_mxf8_ts_w(tmem_base + B_DQ_COL, codes + 8 * k, k_lo + 256 * k, desc_hi, idesc_ts, sf + 4 * k,
                          tmem_base + B_SF_UNIT_COL, (j | k) != 0);
          tc_commit(ts_done(jt & 1));
          // every product that reads the stage is complete when this fires (the scores were read long ago)
          tc_commit(kv_empty(s));
          PROBE(5);
          PROBE_COUNT(6);
        }
        if (!ok) break;
        tc_commit(acc_full);
        tc_commit(q_empty(qb));  // and every product that reads the block's Q and dO8
        ++ci;
        have = false;
        while (ok && !have && next_block()) have = blk.n_tiles > 0;
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int c = (warp - FIRST_EW_WARP) >> 2;  // which block of 32 of the tile's 128 keys this thread handles
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    // this thread's block: scores in columns [32 c, 32 c + 32) of both buffers
    const uint32_t s_tmem = tmem_base + lane_addr + B_S_COL + 32 * c;
    const uint32_t dp_tmem = tmem_base + lane_addr + B_DP_COL + 32 * c;
    const uint32_t dsc_tmem = tmem_base + lane_addr + B_DSC_COL + 8 * c;
    const uint32_t sf_tmem = tmem_base + lane_addr + B_SF_COL + 4 * c + quad;
    if (c == 0) tmem_st4(tmem_base + lane_addr + B_SF_UNIT_COL, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
    int ci = -1;      // query blocks with work so far
    uint32_t jt = 0;  // tiles so far

    for (;;) {
    const int m0 = blk.m0, n_tiles = blk.n_tiles, hq = blk.hq, b = blk.b;
    const int row = m0 + r;
    const int sc = b * p.Hkv + blk.hkv;
    const float sq = p.q_descale[sc], sk = p.k_descale[sc];
    const float beta = p.softmax_scale * sq * sk * LOG2E;
    const float* rec = p.qstat + ((static_cast<int64_t>(b) * p.Hq + hq) * p.nq_pad + m0) * 2 + r;
    const float neg_l = rec[0], neg_d = rec[128];  // log2(g) - L and -sum(dO8 . O) of this query
    const float gsv = p.v_descale[sc];  // dP = sv . dP8 in units of g
    const int row_limit = min(p.causal ? row + shift : p.Nk - 1, p.Nk - 1);
    if (n_tiles > 0) ++ci;

    for (int j = 0; j < n_tiles; ++j, ++jt) {
      if (!mbar_wait_warp(s_full, jt & 1, p.status, WK_ERR_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      PROBE(8);
      tc_fence_after();
      const int limit = row_limit - j * BN;  // columns > limit are masked
      // uniform over the CTA: does this tile contain any masked score?
      const bool tile_masked = (j * BN + BN > p.Nk) || (p.causal && j * BN + BN - 1 > m0 + shift);
      uint32_t sf_d;
      {
        uint32_t sraw[32], draw[32];
        tmem_ld32(s_tmem, sraw);
        tmem_ld32(dp_tmem, draw);
        tc_wait_ld();
        // the scores are in registers: the columns may take the next tile
        tc_fence_before();
        mbar_arrive(s_free);
        PROBE(9);
        uint64_t ds[16];  // dS of this query for 32 keys, as packed pairs
        const uint64_t beta2 = pack_f32x2(beta, beta), nl2 = pack_f32x2(neg_l, neg_l), z2 = pack_f32x2(gsv, gsv),
                       nd2 = pack_f32x2(neg_d, neg_d);
        // two copies of the loop, with and without the mask, behind one branch per tile
        auto scores_to_ds = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sraw[2 * i]), __uint_as_float(sraw[2 * i + 1])), beta2, nl2),
                       x0, x1);
          float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          if constexpr (decltype(masked)::value) {
            if (c * 32 + 2 * i > limit) p0 = 0.f;
            if (c * 32 + 2 * i + 1 > limit) p1 = 0.f;
          }
          ds[i] = mul_f32x2(pack_f32x2(p0, p1),
                            fma_f32x2(pack_f32x2(__uint_as_float(draw[2 * i]), __uint_as_float(draw[2 * i + 1])), z2, nd2));
        }
        };
        if (tile_masked) scores_to_ds(std::true_type{});
        else scores_to_ds(std::false_type{});
        float inv_d;
        const uint32_t bd = block_scale(absmax_bits(ds), inv_d);
        PROBE(10);
        // the products of the tile before the previous one have read this buffer of codes and scale words: the
        // score thread waited for them before it issued this tile's scores
        quantize_block_to_tmem(ds, dsc_tmem + 32 * (jt & 1), inv_d);
        sf_d = bd;
      }
      tmem_st1(sf_tmem + 16 * (jt & 1), sf_d);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
      PROBE(12);
      PROBE_COUNT(15);
    }

    if (n_tiles > 0 && ok) ok = mbar_wait_warp(acc_full, ci & 1, p.status, WK_ERR_TIMEOUT_MMA);
    PROBE(13);
    if (ok) {
      tc_fence_after();
      const float scale = p.softmax_scale * sk;
      __nv_bfloat16* dst_row = p.dq + ((static_cast<int64_t>(b) * p.Hq + hq) * p.Nq + row) * DH;
#pragma unroll 1
      {
        uint32_t v[32];
        if (n_tiles > 0) {  // uniform: TMEM loads are warp-wide
          tmem_ld32(tmem_base + lane_addr + B_DQ_COL + c * 32, v);
          tc_wait_ld();
          // dQ is in registers: the next block's first product may overwrite it
          tc_fence_before();
          mbar_arrive(acc_free);
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
    PROBE(14);
    PROBE_COUNT(21);
    if (!ok || !next_block()) break;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  PROBE_FLUSH(24);
}

// Rows of `d` bytes under boxes of 128: with head dimension 64 TMA fills the upper half of every row with zeros.
int make_map4(CUtensorMap* m, const void* base, int d, int n, int h, int b, const int64_t* strides) {
  const uint64_t dims[4] = {static_cast<uint64_t>(d), static_cast<uint64_t>(n), static_cast<uint64_t>(h), static_cast<uint64_t>(b)};
  const uint64_t str[3] = {static_cast<uint64_t>(strides[2]), static_cast<uint64_t>(strides[1]),
                           static_cast<uint64_t>(strides[0])};
  const uint32_t box[4] = {D, 128, 1, 1};
  return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace
}  // namespace wk

#ifdef WK_BWD_TRACE
extern "C" int wk_bwd_trace_read(unsigned long long* out) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpyFromSymbol(out, wk::g_bwd_trace, sizeof(unsigned long long) * 2 * 20 * 256) != cudaSuccess) return -2;
  unsigned long long* zero = static_cast<unsigned long long*>(calloc(2 * 20 * 256, sizeof(unsigned long long)));
  cudaMemcpyToSymbol(wk::g_bwd_trace, zero, sizeof(unsigned long long) * 2 * 20 * 256);
  free(zero);
  return 0;
}
#endif
#ifdef WK_BWD_PROBE
extern "C" int wk_bwd_probe_read(unsigned long long* out, int clear) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpyFromSymbol(out, wk::g_bwd_probe, 48 * sizeof(unsigned long long)) != cudaSuccess) return -2;
  if (clear) {
    unsigned long long zero[48] = {};
    if (cudaMemcpyToSymbol(wk::g_bwd_probe, zero, sizeof(zero)) != cudaSuccess) return -2;
  }
  return 0;
}
#endif

extern "C" int64_t wk_attn_bwd_fp8_workspace_bytes(int B, int Hq, int Nq) {
  if (B < 0 || Hq < 0 || Nq < 0) return WK_E_ARG;
  const int64_t nq_pad = (static_cast<int64_t>(Nq) + 127) / 128 * 128;
  return static_cast<int64_t>(B) * Hq * (static_cast<int64_t>(Nq) * 128 + nq_pad * 16) + 256;
}

extern "C" int wk_attn_bwd_fp8(const wk_attn_bwd_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Nq <= 0 || a->Nk <= 0 || (a->d != 128 && a->d != 64)) return WK_E_ARG;
  if (a->Hq % a->Hkv || a->B > 65535 || a->Hq > 65535) return WK_E_ARG;
  if (!a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv) return WK_E_ARG;
  if (!a->q_descale || !a->k_descale || !a->v_descale || !a->workspace) return WK_E_ARG;
  if (!(a->softmax_scale > 0.f)) return WK_E_ARG;
  const void* ptrs[] = {a->q, a->k, a->v, a->dq, a->dk, a->dv, a->workspace};
  for (const void* ptr : ptrs)
    if (!aligned16(ptr)) return WK_E_ARG;
  if ((reinterpret_cast<uintptr_t>(a->out) & 7) || (reinterpret_cast<uintptr_t>(a->dout) & 7)) return WK_E_ARG;
  for (int i = 0; i < 3; ++i) {
    if (a->q_strides[i] % 16 || a->k_strides[i] % 16 || a->v_strides[i] % 16) return WK_E_ARG;
    if (a->q_strides[i] <= 0 || a->k_strides[i] <= 0 || a->v_strides[i] <= 0) return WK_E_ARG;
    if (a->out_strides[i] % 4 || a->dout_strides[i] % 4 || a->out_strides[i] <= 0 || a->dout_strides[i] <= 0)
      return WK_E_ARG;
  }
  if (a->workspace_bytes < wk_attn_bwd_fp8_workspace_bytes(a->B, a->Hq, a->Nq)) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int nq_pad = (a->Nq + 127) / 128 * 128;
  uint8_t* do8 = static_cast<uint8_t*>(a->workspace);
  const int64_t do8_bytes = (static_cast<int64_t>(a->B) * a->Hq * a->Nq * a->d + 255) / 256 * 256;
  float* qstat = reinterpret_cast<float*>(do8 + do8_bytes);

  PrepParams pp;
  pp.dout = static_cast<const __nv_bfloat16*>(a->dout);
  pp.out = static_cast<const __nv_bfloat16*>(a->out);
  pp.lse = a->lse;
  pp.v_descale = a->v_descale;
  pp.do8 = do8;
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
  pp.Hkv = a->Hkv;
  pp.Nq = a->Nq;
  pp.nq_pad = nq_pad;
  pp.d = a->d;
  {
    const int64_t rows = static_cast<int64_t>(a->B) * a->Hq * nq_pad;
    bool wide_loads = aligned16(a->out) && aligned16(a->dout);  // 16-byte loads: rows on 16-byte boundaries
    for (int i = 0; i < 3; ++i) wide_loads = wide_loads && a->out_strides[i] % 8 == 0 && a->dout_strides[i] % 8 == 0;
    if (wide_loads) {
      attn_bwd_prep4_kernel<<<static_cast<unsigned>((rows + 31) / 32), 256, 0, st>>>(pp);
    } else {
      const int64_t blocks = (rows + 7) / 8;
      attn_bwd_prep_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(pp);
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
  const int64_t do_str[3] = {static_cast<int64_t>(a->Hq) * a->Nq * a->d, static_cast<int64_t>(a->Nq) * a->d, a->d};
  r = make_map4(&tdo, do8, a->d, a->Nq, a->Hq, a->B, do_str);
  if (r) return r;

  BwdParams p;
  p.qstat = qstat;
  p.q_descale = a->q_descale;
  p.k_descale = a->k_descale;
  p.v_descale = a->v_descale;
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

  if (allow_smem((a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<128>)), A_SMEM_BYTES)) return WK_E_CUDA;
  if (allow_smem((a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_dq_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_dq_kernel<128>)), B_SMEM_BYTES)) return WK_E_CUDA;
  {
    dim3 grid((a->Nk + BN - 1) / BN, a->Hkv, a->B);
    void* args[] = {&tq, &tk, &tv, &tdo, &p};
    const void* kernel = a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<128>);
    if (cudaLaunchKernel(kernel, grid, dim3(THREADS), args, A_SMEM_BYTES, st) != cudaSuccess) return WK_E_CUDA;
  }
  {
    dim3 grid((a->Nq + BM - 1) / BM, a->Hq, a->B);
    void* args[] = {&tq, &tk, &tv, &tdo, &p};
    const void* kernel = a->d == 64 ? reinterpret_cast<const void*>(attn_bwd_dq_kernel<64>) : reinterpret_cast<const void*>(attn_bwd_dq_kernel<128>);
    if (cudaLaunchKernel(kernel, grid, dim3(THREADS), args, B_SMEM_BYTES, st) != cudaSuccess) return WK_E_CUDA;
  }
  return 0;
}
