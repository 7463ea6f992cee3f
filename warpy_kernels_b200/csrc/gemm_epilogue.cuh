// Fused GEMM epilogue shared by the BF16/FP16 and the MXFP8 kernel.
//
// Order of operations as in the reference's epilogue (warpy_kernels/gemm/base.py:436-497):
//   v = acc . scale_a[row or 0] . scale_b[col or 0]      scalar or per-row / per-column fp32 scales
//   v += out[row, col]                                    accum
//   pre_out[row, col] = v                                 store_pre (with act = gelu)
//   v = gelu(v)        or        v = v . gelu'(pre_in[row, col])
//   out[row, col] = round16(v);  optional MXFP8 copy of v (warpy_kernels/gemm/sm89.py:65-93)
// GELU is the exact erf form and its derivative cdf + x . pdf (warpy_kernels/utils/math.py:7-21).
//
// One thread owns one output row of the tile and walks it in chunks of 32 consecutive columns (the
// layout tcgen05.ld 32x32b delivers), so a chunk is exactly one MX block.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace wk {

enum : int { ACT_NONE = 0, ACT_GELU = 1, ACT_DGELU = 2 };

struct Epilogue {
  const float* scale_a;  // null = 1
  const float* scale_b;  // null = 1
  int scale_a_rows;      // 1: scale_a has one entry per output row
  int scale_b_cols;      // 1: scale_b has one entry per output column
  int accum;             // add the values `out` already holds
  int act;               // ACT_*
  int out_f16;           // 0: bf16 output (and pre buffers), 1: fp16
  void* pre_out;         // optional [M, N]: the value before the activation
  const void* pre_in;    // [M, N] for ACT_DGELU
  uint8_t* q_mx;         // optional [M, N] e4m3
  uint8_t* s_mx;         // optional [M, N / 32] ue8m0
};

__device__ __forceinline__ float gelu_exact(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float dgelu_exact(float x) {
  return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * __expf(-0.5f * x * x) * 0.39894228040143268f;
}

template <bool F16>
__device__ __forceinline__ uint32_t pack_half16x2(float lo, float hi) {
  if (F16) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  return pack_bf16x2(lo, hi);
}
template <bool F16>
__device__ __forceinline__ void unpack_half16x2(uint32_t w, float& lo, float& hi) {
  if (F16) {
    f16x2_to_float2(w, lo, hi);
  } else {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
}

// Loads 32 consecutive 16-bit values of a row as fp32.
template <bool F16>
__device__ __forceinline__ void load_row32(const void* base, int64_t off, float (&x)[32]) {
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 w = src[i];
    unpack_half16x2<F16>(w.x, x[8 * i + 0], x[8 * i + 1]);
    unpack_half16x2<F16>(w.y, x[8 * i + 2], x[8 * i + 3]);
    unpack_half16x2<F16>(w.z, x[8 * i + 4], x[8 * i + 5]);
    unpack_half16x2<F16>(w.w, x[8 * i + 6], x[8 * i + 7]);
  }
}
template <bool F16>
__device__ __forceinline__ void store_row32(void* base, int64_t off, const float (&x)[32]) {
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    w.x = pack_half16x2<F16>(x[8 * i + 0], x[8 * i + 1]);
    w.y = pack_half16x2<F16>(x[8 * i + 2], x[8 * i + 3]);
    w.z = pack_half16x2<F16>(x[8 * i + 4], x[8 * i + 5]);
    w.w = pack_half16x2<F16>(x[8 * i + 6], x[8 * i + 7]);
    dst[i] = w;
  }
}

// F16: fp16 instead of bf16 storage.  PLAIN: no column scales, no accumulation and no activation (the common
// case, kept free of the tests for those options because the epilogue sits on the kernels' critical path).
template <bool F16, bool PLAIN>
__device__ __forceinline__ void epilogue_chunk_impl(const Epilogue& e, const uint32_t (&acc)[32], float row_scale,
                                                    int row, int col, int N, void* out) {
  const int64_t off = static_cast<int64_t>(row) * N + col;
  float f[32];
  if (!PLAIN && e.scale_b_cols) {
    const float4* sb = reinterpret_cast<const float4*>(e.scale_b + col);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 s4 = __ldg(sb + i);
      f[4 * i + 0] = __uint_as_float(acc[4 * i + 0]) * row_scale * s4.x;
      f[4 * i + 1] = __uint_as_float(acc[4 * i + 1]) * row_scale * s4.y;
      f[4 * i + 2] = __uint_as_float(acc[4 * i + 2]) * row_scale * s4.z;
      f[4 * i + 3] = __uint_as_float(acc[4 * i + 3]) * row_scale * s4.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(acc[i]) * row_scale;
  }
  if (!PLAIN && e.accum) {
    float c[32];
    load_row32<F16>(out, off, c);
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] += c[i];
  }
  if (!PLAIN && e.act == ACT_GELU) {
    if (e.pre_out) store_row32<F16>(e.pre_out, off, f);
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = gelu_exact(f[i]);
  } else if (!PLAIN && e.act == ACT_DGELU) {
    float pre[32];
    load_row32<F16>(e.pre_in, off, pre);
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] *= dgelu_exact(pre[i]);
  }
  store_row32<F16>(out, off, f);
  if (e.q_mx) {
    // this thread's 32 consecutive columns are exactly one MX block
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = max(amax, __float_as_uint(f[i]) & 0x7fffffffu);
    int ex = static_cast<int>((amax + 0x1fffffu) >> 23) - 8;
    ex = min(max(ex, 0), 254);
    const float inv = __uint_as_float(static_cast<uint32_t>(max(254 - ex, 1)) << 23);
    uint4* qdst = reinterpret_cast<uint4*>(e.q_mx + off);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 w;
      w.x = pack_e4m3x4(__fmul_rn(f[16 * i + 0], inv), __fmul_rn(f[16 * i + 1], inv), __fmul_rn(f[16 * i + 2], inv),
                        __fmul_rn(f[16 * i + 3], inv));
      w.y = pack_e4m3x4(__fmul_rn(f[16 * i + 4], inv), __fmul_rn(f[16 * i + 5], inv), __fmul_rn(f[16 * i + 6], inv),
                        __fmul_rn(f[16 * i + 7], inv));
      w.z = pack_e4m3x4(__fmul_rn(f[16 * i + 8], inv), __fmul_rn(f[16 * i + 9], inv),
                        __fmul_rn(f[16 * i + 10], inv), __fmul_rn(f[16 * i + 11], inv));
      w.w = pack_e4m3x4(__fmul_rn(f[16 * i + 12], inv), __fmul_rn(f[16 * i + 13], inv),
                        __fmul_rn(f[16 * i + 14], inv), __fmul_rn(f[16 * i + 15], inv));
      qdst[i] = w;
    }
    e.s_mx[static_cast<int64_t>(row) * (N / 32) + col / 32] = static_cast<uint8_t>(ex);
  }
}

// acc: 32 fp32 accumulators (bit patterns) of row `row`, columns [col, col + 32).  `row_scale` = scalar scales and
// the row's scale_a entry already multiplied together.  The branches are uniform over the grid.
__device__ __forceinline__ void epilogue_chunk(const Epilogue& e, const uint32_t (&acc)[32], float row_scale, int row,
                                               int col, int N, void* out) {
  const bool plain = !e.scale_b_cols && !e.accum && e.act == ACT_NONE;
  if (e.out_f16) {
    epilogue_chunk_impl<true, false>(e, acc, row_scale, row, col, N, out);
  } else if (plain) {
    epilogue_chunk_impl<false, true>(e, acc, row_scale, row, col, N, out);
  } else {
    epilogue_chunk_impl<false, false>(e, acc, row_scale, row, col, N, out);
  }
}

// Scalar part of the scales plus this row's scale_a entry.
__device__ __forceinline__ float epilogue_row_scale(const Epilogue& e, int row) {
  float s = 1.f;
  if (e.scale_a) s *= e.scale_a_rows ? e.scale_a[row] : e.scale_a[0];
  if (e.scale_b && !e.scale_b_cols) s *= e.scale_b[0];
  return s;
}

}  // namespace wk
