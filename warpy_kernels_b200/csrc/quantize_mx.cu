// MXFP8 quantiser: rows of bf16 / fp32 values -> e4m3 codes plus one ue8m0 scale
// byte per block of 32 consecutive elements.
//
// Arithmetic (bit-exact with the reference's GEMM epilogue quantiser,
// warpy_kernels/gemm/sm89.py:65-93 with warpy_kernels/ptx/common.py:539-565 and
// warpy_kernels/ptx/sm89.py:85-93):
//   A    = max_i (bits(x_i) & 0x7fffffff)                  integer max of |x| bit patterns
//   e    = clamp(((A + 0x1fffff) >> 23) - 8, 0, 254)        scale byte, value 2^(e-127)
//   inv  = float_from_bits(max(254 - e, 1) << 23)           2^(127-e)
//   code = cvt.rn.satfinite.e4m3(x_i * inv)
//
// HBM-bound: 2 (bf16) or 4 (fp32) bytes in, 1 + 1/32 bytes out per element.  Four
// consecutive threads own one block of 32 elements (8 each: one 16-byte load for
// bf16, two for fp32), so a warp reads 512 / 1024 contiguous bytes and writes 256.
#include "common.cuh"
#include "host_common.h"

namespace wk {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// The scale byte and the multiplier for one block's integer amax.
__device__ __forceinline__ void mx_scale(uint32_t amax_bits, uint32_t& e, float& inv) {
  int t = static_cast<int>((amax_bits + 0x1fffffu) >> 23) - 8;
  t = max(t, 0);
  t = min(t, 254);
  e = static_cast<uint32_t>(t);
  inv = __uint_as_float(static_cast<uint32_t>(max(254 - t, 1)) << 23);
}

// CONTIG: rows are back to back (ld_x == cols), so input, code and scale offsets are all linear in the group
// index and no division is needed.
template <typename T, bool CONTIG>
__global__ void __launch_bounds__(kThreads)
quantize_mx_kernel(const T* __restrict__ x, int64_t ld_x, uint8_t* __restrict__ q,
                   uint8_t* __restrict__ s, int64_t total_groups, int groups_per_row) {
  // one "group" = 8 consecutive elements; 4 groups = one scale block
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; base - threadIdx.x % 32 < total_groups; base += stride * kUnroll) {
    float v[kUnroll][8];
    bool ok[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = base + u * stride;
      ok[u] = g < total_groups;
      if (ok[u]) {
        int64_t off = g * 8;
        if (!CONTIG) {
          const uint32_t row = static_cast<uint32_t>(g / groups_per_row);
          off = row * ld_x + (g - static_cast<int64_t>(row) * groups_per_row) * 8;
        }
        load8(x + off, v[u]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = base + u * stride;
      uint32_t amax = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max(amax, __float_as_uint(v[u][i]) & 0x7fffffffu);
      amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      uint32_t e;
      float inv;
      mx_scale(amax, e, inv);
      if (ok[u]) {
        uint2 codes;
        codes.x = pack_e4m3x4(__fmul_rn(v[u][0], inv), __fmul_rn(v[u][1], inv),
                              __fmul_rn(v[u][2], inv), __fmul_rn(v[u][3], inv));
        codes.y = pack_e4m3x4(__fmul_rn(v[u][4], inv), __fmul_rn(v[u][5], inv),
                              __fmul_rn(v[u][6], inv), __fmul_rn(v[u][7], inv));
        // the outputs are contiguous [rows, cols] and [rows, cols / 32]: linear in g whatever ld_x is
        __stcs(reinterpret_cast<uint2*>(q + g * 8), codes);
        if ((g & 3) == 0) s[g >> 2] = static_cast<uint8_t>(e);
      }
    }
  }
}

template <typename T>
int launch(const T* x, int64_t rows, int64_t cols, int64_t ld_x, uint8_t* q, uint8_t* s,
           cudaStream_t stream) {
  const int64_t total = rows * (cols / 8);
  const int sms = sm_count();
  if (sms <= 0) return WK_E_CUDA;
  const int64_t want = (total + static_cast<int64_t>(kThreads) * kUnroll - 1) / (kThreads * kUnroll);
  // 8 resident CTAs of 256 threads fill an SM; more CTAs than that only add tail.
  int64_t grid = want < static_cast<int64_t>(sms) * 8 ? want : static_cast<int64_t>(sms) * 8;
  if (grid < 1) grid = 1;
  if (ld_x == cols) {
    quantize_mx_kernel<T, true><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
        x, ld_x, q, s, total, static_cast<int>(cols / 8));
  } else {
    quantize_mx_kernel<T, false><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
        x, ld_x, q, s, total, static_cast<int>(cols / 8));
  }
  return cudaGetLastError() == cudaSuccess ? 0 : WK_E_CUDA;
}

}  // namespace
}  // namespace wk

extern "C" int wk_quantize_mx(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                              void* q, void* s, void* stream) {
  if (rows < 0 || cols < 0 || cols % 32 != 0 || ld_x < cols || ld_x % 8 != 0) return WK_E_ARG;
  if (cols / 8 > 0x7fffffff || rows > 0x7fffffff) return WK_E_ARG;
  if (rows == 0 || cols == 0) return 0;
  if (!x || !q || !s || !wk::aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7)) return WK_E_ARG;
  if (int unsupported = wk::require_sm100()) return unsupported;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == WK_BF16)
    return wk::launch(static_cast<const __nv_bfloat16*>(x), rows, cols, ld_x,
                      static_cast<uint8_t*>(q), static_cast<uint8_t*>(s), st);
  if (dtype == WK_F32)
    return wk::launch(static_cast<const float*>(x), rows, cols, ld_x, static_cast<uint8_t*>(q),
                      static_cast<uint8_t*>(s), st);
  return WK_E_ARG;
}
