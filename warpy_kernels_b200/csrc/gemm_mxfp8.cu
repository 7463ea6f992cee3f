// MXFP8 block-scaled GEMM for sm_100a:
//   out[M,N] = alpha . (a8 . 2^(sa-127)) . (b8 . 2^(sb-127))^T      bf16 output, fp32 accumulation
// a8 [M,K], b8 [N,K] e4m3; sa [M,K/32], sb [N,K/32] ue8m0 bytes (one per row and 32
// elements along K); either scale tensor may be absent (unit scales).  Optionally the
// fp32 results are also written as MXFP8 (codes + scale byte per 32 columns) before
// they are rounded to bf16.
//
// Two kernels:
//  1. swizzle_scales_kernel re-tiles the row-major scale bytes into the 512-byte
//     atoms tcgen05.mma reads them in (128 rows x 4 K-blocks: byte offset
//     (row % 32) * 16 + (row / 32 % 4) * 4 + kblock % 4), one atom per 128 rows and 128
//     K elements, atoms ordered [row block][K block].  This is the kernel's scratch.
//  2. gemm_mxfp8_kernel: persistent, warp-specialised, 128 x 256 tile, 128 K-bytes per
//     stage.  Warp 0: TMA for A/B (128-byte swizzle) plus bulk copies of the scale
//     atoms.  Warp 1: tcgen05.cp of the atoms into TMEM, then four
//     tcgen05.mma kind::mxf8f6f4.block_scale (K = 32 each; the scale-factor id selects
//     the byte of the K block).  Warps 2-5: epilogue from TMEM.
//     TMEM: two 256-column accumulators that share 64 columns ([0,256) and [192,448)) plus the
//     scale-factor columns.  The epilogue drains the shared columns of a tile first and then
//     lets the next tile's main loop start while it drains the rest.
//
// Arithmetic follows the reference's block-scaled path (warpy_kernels/gemm/sm120.py:121-146:
// e4m3 products scaled by 2^(sfa-127) per row and 32-element K block, fp32 accumulate)
// and its MX output epilogue (warpy_kernels/gemm/sm89.py:65-93).
//
// Tensor-core bound: 2*M*N*K flops per launch.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "host_common.h"
#include "gemm_mxfp8.h"

namespace wk {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes == e4m3 elements
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int SF_ATOM = 512;
constexpr int SFA_BYTES = SF_ATOM;
constexpr int SFB_BYTES = 2 * SF_ATOM;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 192;    // accumulator slot a lives in columns [192 a, 192 a + 256)
constexpr int SF_COL = 448;        // scale-factor columns start here
constexpr int SF_SLOTS = 4;        // one slot per smem stage
constexpr int SF_SLOT_COLS = 12;   // 4 (A: 128 rows) + 8 (B: 256 rows)

// ---------------------------------------------------------------------------
// scale pre-swizzle
// ---------------------------------------------------------------------------
// One thread per (row, 128-element K block): reads 4 scale bytes, writes one 32-bit word.
__global__ void swizzle_scales_kernel(const uint8_t* __restrict__ s, uint32_t* __restrict__ out,
                                      int rows, int kblocks128) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(rows) * kblocks128;
  if (idx >= total) return;
  const int kb = static_cast<int>(idx % kblocks128);
  const int row = static_cast<int>(idx / kblocks128);
  uint32_t w = 0x7f7f7f7fu;  // unit scales when the caller gave none
  if (s) w = *reinterpret_cast<const uint32_t*>(s + static_cast<int64_t>(row) * kblocks128 * 4 + kb * 4);
  const int rb = row / 128;
  const int r = row % 128;
  const int64_t atom = static_cast<int64_t>(rb) * kblocks128 + kb;
  out[atom * (SF_ATOM / 4) + (r % 32) * 4 + (r / 32)] = w;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t ovl_bar = bar_base + 8u * (2 * STAGES + 4);  // the shared columns of the last tile are drained
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 5);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int num_m = p.M / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K / BK;
  const int n_atoms_total = p.N / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_init(ovl_bar, 4);
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
      // The launch may overlap the end of the kernel that re-tiles the scales (programmatic stream serialisation):
      // nothing is loaded before that kernel has completed.
      pdl_wait();
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m);
        const int nb_atoms = min(2, n_atoms_total - tc.n_blk * 2);  // 1 on a 128-wide edge tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.status, WK_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t ssfa = sb + B_BYTES;
          const uint32_t ssfb = ssfa + SFA_BYTES;
          mbar_expect_tx(full_bar(stage), A_BYTES + B_BYTES + SFA_BYTES + nb_atoms * SF_ATOM);
          tma_load_2d(sa, &tmap_a, full_bar(stage), kb * BK, tc.m_blk * BM);
          tma_load_2d(sb, &tmap_b, full_bar(stage), kb * BK, tc.n_blk * BN);
          bulk_load(ssfa, p.sfa + (static_cast<int64_t>(tc.m_blk) * num_kb + kb) * SF_ATOM, SF_ATOM,
                    full_bar(stage));
          for (int a = 0; a < nb_atoms; ++a) {
            bulk_load(ssfb + a * SF_ATOM,
                      p.sfb + (static_cast<int64_t>(tc.n_blk * 2 + a) * num_kb + kb) * SF_ATOM, SF_ATOM,
                      full_bar(stage));
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
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      // descriptors of stage 0; a later stage only moves the 16-byte-granular start address field
      constexpr uint64_t kStageStep = STAGE_BYTES / 16;
      static_assert(STAGE_BYTES % 16 == 0, "stage size must keep descriptors 16-byte granular");
      const uint64_t a_desc0 = smem_desc_sw128(smem_base, 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_base + A_BYTES, 16, 1024);
      const uint64_t sfa_desc0 = smem_desc_plain(smem_base + A_BYTES + B_BYTES, 16, 128);
      const uint64_t sfb_desc0 = smem_desc_plain(smem_base + A_BYTES + B_BYTES + SFA_BYTES, 16, 128);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        // this slot was drained two tiles ago, and the previous tile has given up the columns it shares
        if (!mbar_wait(tempty_bar(acc), ((local >> 1) & 1) ^ 1, p.status, WK_ERR_TIMEOUT_TMEM)) break;
        if (local > 0 && !mbar_wait(ovl_bar, (local - 1) & 1, p.status, WK_ERR_TIMEOUT_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, WK_ERR_TIMEOUT_LOAD)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t step = static_cast<uint64_t>(stage) * kStageStep;
          const uint32_t sf_tmem = tmem_base + SF_COL + stage * SF_SLOT_COLS;
          // 32 rows x 16 bytes per copy; the shared-memory source is a plain (unswizzled) block
          tmem_cp_32x128b_warpx4(sf_tmem + 0, sfa_desc0 + step);
          tmem_cp_32x128b_warpx4(sf_tmem + 4, sfb_desc0 + step);
          tmem_cp_32x128b_warpx4(sf_tmem + 8, sfb_desc0 + step + SF_ATOM / 16);
          const uint64_t a_desc = a_desc0 + step;
          const uint64_t b_desc = b_desc0 + step;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            mma_mxf8_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, make_idesc_mx(BM, BN, k, k), sf_tmem,
                        sf_tmem + 4, (kb | k) != 0);
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
    const int quad = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m);
      const int acc = local & 1;
      if (!mbar_wait_warp(tfull_bar(acc), (local >> 1) & 1, p.status, WK_ERR_TIMEOUT_MMA)) break;
      tc_fence_after();
      // column chunks in the order they are drained: the 64 columns shared with the other slot first
      const int first_chunk = acc == 0 ? 6 : 0;
      const int row = tc.m_blk * BM + quad * 32 + lane;
      const float row_scale = epilogue_row_scale(p.epi, row);
#pragma unroll 1
      for (int ci = 0; ci < BN / 32; ++ci) {
        const int c = (ci + first_chunk) & 7;
        uint32_t v[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * ACC_STRIDE + c * 32, v);
        tc_wait_ld();
        if (ci == 1) {
          // both shared chunks are in registers: the next tile's main loop may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(ovl_bar);
        }
        const int col = tc.n_blk * BN + c * 32;
        if (col < p.N) epilogue_chunk(p.epi, v, row_scale, row, col, p.N, p.out);
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

Epilogue epilogue_of(const wk_gemm_mx_args* a) {
  Epilogue e;
  e.scale_a = a->scale_a;
  e.scale_b = a->scale_b;
  e.scale_a_rows = a->scale_a_rows;
  e.scale_b_cols = a->scale_b_cols;
  e.accum = a->accum;
  e.act = a->act;
  e.out_f16 = a->out_f16;
  e.pre_out = a->pre_out;
  e.pre_in = a->pre_in;
  e.q_mx = static_cast<uint8_t*>(a->q_mx);
  e.s_mx = static_cast<uint8_t*>(a->s_mx);
  return e;
}

bool epilogue_args_ok(const wk_gemm_mx_args* a) {
  if (a->act < 0 || a->act > 2 || (a->act == ACT_DGELU && !a->pre_in)) return false;
  if ((a->pre_out && !aligned16(a->pre_out)) || (a->pre_in && !aligned16(a->pre_in))) return false;
  if (a->scale_b && a->scale_b_cols && !aligned16(a->scale_b)) return false;
  return true;
}

int swizzle(const void* s, void* dst, int rows, int k, cudaStream_t st) {
  const int kb128 = k / 128;
  const int64_t total = static_cast<int64_t>(rows) * kb128;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  swizzle_scales_kernel<<<static_cast<unsigned>(blocks), threads, 0, st>>>(
      static_cast<const uint8_t*>(s), static_cast<uint32_t*>(dst), rows, kb128);
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}

}  // namespace
}  // namespace wk

extern "C" int64_t wk_gemm_mxfp8_workspace_bytes(int m, int n, int k) {
  if (m < 0 || n < 0 || k < 0) return WK_E_ARG;
  return (static_cast<int64_t>(m) + n) * (k / 32) + 32;
}

extern "C" int64_t wk_mx_scales_tiled_bytes(int rows, int k) {
  if (rows < 0 || k < 0 || rows % 128 || k % 128) return WK_E_ARG;
  return static_cast<int64_t>(rows) * (k / 32);
}

extern "C" int wk_tile_mx_scales(const void* s, int rows, int k, void* dst, void* stream) {
  using namespace wk;
  if (rows < 0 || k < 0 || rows % 128 || k % 128 || !dst || !aligned16(dst)) return WK_E_ARG;
  if (s && (reinterpret_cast<uintptr_t>(s) & 3)) return WK_E_ARG;
  if (rows == 0 || k == 0) return 0;
  if (int unsupported = require_sm100()) return unsupported;
  return swizzle(s, dst, rows, k, static_cast<cudaStream_t>(stream));
}

extern "C" int wk_gemm_mxfp8(const wk_gemm_mx_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  const int m = a->m, n = a->n, k = a->k;
  if (m < 0 || n < 0 || k < 0 || m % BM || n % 128 || k % BK) return WK_E_ARG;
  if (m == 0 || n == 0) return 0;
  if (k == 0) return WK_E_ARG;
  if (!a->a || !a->b || !a->out) return WK_E_ARG;
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->out) || !aligned16(a->workspace)) return WK_E_ARG;
  const bool a_tiled = a->a_scale_tiled != 0, b_tiled = a->b_scale_tiled != 0;
  if (!a->workspace && !(a_tiled && b_tiled)) return WK_E_ARG;  // scratch for whatever is still row-major
  if (a_tiled && (!a->a_scale_mx || !aligned16(a->a_scale_mx))) return WK_E_ARG;
  if (b_tiled && (!a->b_scale_mx || !aligned16(a->b_scale_mx))) return WK_E_ARG;
  if (a->a_scale_mx && (reinterpret_cast<uintptr_t>(a->a_scale_mx) & 3)) return WK_E_ARG;
  if (a->b_scale_mx && (reinterpret_cast<uintptr_t>(a->b_scale_mx) & 3)) return WK_E_ARG;
  if ((a->q_mx == nullptr) != (a->s_mx == nullptr)) return WK_E_ARG;
  if (a->q_mx && !aligned16(a->q_mx)) return WK_E_ARG;
  if (!epilogue_args_ok(a)) return WK_E_ARG;
  if (a->cta_pair < 0 || a->cta_pair > 2) return WK_E_ARG;
  if (a->workspace && a->workspace_bytes < wk_gemm_mxfp8_workspace_bytes(m, n, k)) return WK_E_ARG;
  if (int unsupported = require_sm100()) return unsupported;
  int* status = status_word();
  if (!status) return WK_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // scale tensors the caller has already tiled (wk_tile_mx_scales) are read where they are; the others are
  // re-tiled into the workspace first
  const uint8_t* sfa = static_cast<const uint8_t*>(a->a_scale_mx);
  const uint8_t* sfb = static_cast<const uint8_t*>(a->b_scale_mx);
  int r = 0;
  if (!a_tiled) {
    uint8_t* dst = static_cast<uint8_t*>(a->workspace);
    r = swizzle(a->a_scale_mx, dst, m, k, st);
    if (r) return r;
    sfa = dst;
  }
  if (!b_tiled) {
    uint8_t* dst = static_cast<uint8_t*>(a->workspace) + ((static_cast<int64_t>(m) * (k / 32) + 15) / 16) * 16;
    r = swizzle(a->b_scale_mx, dst, n, k, st);
    if (r) return r;
    sfb = dst;
  }

  GemmParams p;
  p.out = a->out;
  p.sfa = sfa;
  p.sfb = sfb;
  p.epi = epilogue_of(a);
  p.M = m;
  p.N = n;
  p.K = k;
  if (a->group_m < 0) return WK_E_ARG;
  p.group_m = a->group_m ? a->group_m : 8;
  p.status = status;
  if (a->cta_pair == 1) return launch_gemm_mxfp8_2sm(a->a, a->b, p, st, !(a_tiled && b_tiled));

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {BK, BM};
    r = encode_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {BK, BN};
    r = encode_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  if (allow_smem(reinterpret_cast<const void*>(gemm_mxfp8_kernel), SMEM_BYTES)) return WK_E_CUDA;
  const int num_tiles = (m / BM) * ((n + BN - 1) / BN);
  const int sms = sm_count();
  if (sms <= 0) return WK_E_CUDA;
  const int grid = num_tiles < sms ? num_tiles : sms;
  // after a re-tiling launch: start under its tail (the producer waits for it before the first load)
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = (a_tiled && b_tiled) ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_mxfp8_kernel, ta, tb, p) == cudaSuccess ? 0 : WK_E_CUDA;
}

// ---------------------------------------------------------------------------
// Variant for callers that must not allocate device memory.
// ---------------------------------------------------------------------------
// The re-tiled scale factors live in a fixed array that is part of the loaded
// module instead of a caller-provided workspace, and the status word is a module
// variable too, so this entry point never calls cudaMalloc / cudaFree or any
// allocating library routine.  Every GPU that loads the library carries the array
// (WK_NOALLOC_SCRATCH_BYTES) until the process exits.
//
// In host code the names below are only handles for the runtime, not device
// addresses; the real addresses are looked up once per device with
// cudaGetSymbolAddress while that device is current, and those pointers are what
// the kernels receive.
namespace wk {
namespace {

constexpr int64_t kNoAllocScratchBytes = WK_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ int g_noalloc_status;

constexpr int kNoAllocMaxDevices = 64;
uint8_t* g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {};
int* g_noalloc_status_ptr[kNoAllocMaxDevices] = {};

// Looks the two device addresses up on the first call made on a device.
int noalloc_setup(int dev) {
  if (g_noalloc_scratch_ptr[dev] && g_noalloc_status_ptr[dev]) return 0;
  void* scratch = nullptr;
  void* status = nullptr;
  if (cudaGetSymbolAddress(&scratch, g_noalloc_scratch) != cudaSuccess || !scratch) return WK_E_CUDA;
  if (cudaGetSymbolAddress(&status, g_noalloc_status) != cudaSuccess || !status) return WK_E_CUDA;
  g_noalloc_scratch_ptr[dev] = static_cast<uint8_t*>(scratch);
  g_noalloc_status_ptr[dev] = static_cast<int*>(status);
  return 0;
}

}  // namespace
}  // namespace wk

extern "C" int64_t wk_gemm_mxfp8_noalloc_max_bytes(void) { return wk::kNoAllocScratchBytes; }

extern "C" int wk_gemm_mxfp8_noalloc(const wk_gemm_mx_args* a, void* stream) {
  using namespace wk;
  if (!a) return WK_E_ARG;
  const int m = a->m, n = a->n, k = a->k;
  if (m < 0 || n < 0 || k < 0 || m % BM || n % 128 || k % BK) return WK_E_ARG;
  if (m == 0 || n == 0) return 0;
  if (k == 0) return WK_E_ARG;
  if (!a->a || !a->b || !a->out) return WK_E_ARG;
  if (!aligned16(a->a) || !aligned16(a->b) || !aligned16(a->out)) return WK_E_ARG;
  if (a->a_scale_mx && (reinterpret_cast<uintptr_t>(a->a_scale_mx) & 3)) return WK_E_ARG;
  if (a->b_scale_mx && (reinterpret_cast<uintptr_t>(a->b_scale_mx) & 3)) return WK_E_ARG;
  if ((a->q_mx == nullptr) != (a->s_mx == nullptr)) return WK_E_ARG;
  if (a->q_mx && !aligned16(a->q_mx)) return WK_E_ARG;
  if (!epilogue_args_ok(a)) return WK_E_ARG;
  // scales that are already tiled need no scratch at all: such a caller uses wk_gemm_mxfp8 with a NULL workspace
  if (a->a_scale_tiled || a->b_scale_tiled) return WK_E_ARG;
  // the fixed array bounds the problem size: (M + N) * K / 32 scale bytes must fit
  if (wk_gemm_mxfp8_workspace_bytes(m, n, k) > kNoAllocScratchBytes) return WK_E_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return WK_E_CUDA;
  if (int unsupported = require_sm100()) return unsupported;
  int r = noalloc_setup(dev);
  if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  uint8_t* sfa = g_noalloc_scratch_ptr[dev];
  uint8_t* sfb = sfa + ((static_cast<int64_t>(m) * (k / 32) + 15) / 16) * 16;
  // every atom the GEMM will read is rewritten here, so nothing of the previous call survives into this one
  r = swizzle(a->a_scale_mx, sfa, m, k, st);
  if (r) return r;
  r = swizzle(a->b_scale_mx, sfb, n, k, st);
  if (r) return r;

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {BK, BM};
    r = encode_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {BK, BN};
    r = encode_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  GemmParams p;
  p.out = a->out;
  p.sfa = sfa;
  p.sfb = sfb;
  p.epi = epilogue_of(a);
  p.M = m;
  p.N = n;
  p.K = k;
  p.group_m = 8;
  p.status = g_noalloc_status_ptr[dev];
  if (cudaFuncSetAttribute(reinterpret_cast<const void*>(gemm_mxfp8_kernel),
                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return WK_E_CUDA;
  const int num_tiles = (m / BM) * ((n + BN - 1) / BN);
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return WK_E_CUDA;
  const int grid = num_tiles < sms ? num_tiles : sms;
  gemm_mxfp8_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}

extern "C" int wk_gemm_mxfp8_noalloc_status(void) {
  using namespace wk;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return WK_E_CUDA;
  if (noalloc_setup(dev)) return WK_E_CUDA;
  if (cudaDeviceSynchronize() != cudaSuccess) return WK_E_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, g_noalloc_status_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return WK_E_CUDA;
  if (v != 0 && cudaMemset(g_noalloc_status_ptr[dev], 0, sizeof(int)) != cudaSuccess) return WK_E_CUDA;
  return v;
}
