// Recomputation of flagged query blocks of the attention forward (FP8 and BF16 inputs), head dimension 128 or 64.
//
// The tensor-core forward kernels keep one reference exponent per query row, fixed by the row's first 64 keys, and
// can represent scores up to 2^100 above it.  A query block in which some row meets a later key beyond that range
// is flagged in the call's workspace (one int per block of 128 queries) and computed again here with the exact row
// maximum: a plain two-pass softmax in fp32 on the CUDA cores -- pass one finds each row's maximum over all visible
// keys, pass two accumulates exp2(s - max) and P.V.  The reference reaches the same result by moving its reference
// with every 128-key tile and rescaling O (warpy_kernels/attn/fwd_base.py:337-360); inputs that need it are
// pathological (one key more than 69 nats above the start of the row), so this path is written for clarity, not speed.
//
// One CTA of 512 threads per flagged block: four threads per query row, each owning 32 of the 128 head-dim
// elements (with head dimension 64 two of the four hold zeros and only join the reductions); K and V pass through
// shared memory 64 keys at a time.  A launch covers every block of the call: each CTA reads its share of the
// flags in one go, so with nothing flagged it costs one small launch that reads the flags and leaves.
#include <math.h>

#include "attn_fwd_redo.h"
#include "common.cuh"

namespace wk {
namespace {

constexpr int R_BM = 128;    // queries per block (the forward kernels' block)
constexpr int R_D = 128;     // largest head dimension
constexpr int R_KEYS = 64;   // keys per shared-memory chunk
constexpr int R_THREADS = 512;
constexpr int R_PART = 32;   // head-dim elements per thread

struct RedoParams {
  const uint8_t* q;
  const uint8_t* k;
  const uint8_t* v;
  __nv_bfloat16* out;
  float* lse;
  float* pmax;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  int64_t q_strides[3], k_strides[3], v_strides[3], out_strides[3];  // elements, dims (B, H, N)
  int64_t lse_stride_b, lse_stride_h;
  int B, Hq, Hkv, Nq, Nk, d, causal, write_lse, lse_natural;
  const int* seqused_k;
  float softmax_scale;
  int* flags;
};

// 32 consecutive elements at `src` (16-byte aligned) as fp32.
template <bool BF16>
__device__ __forceinline__ void load32(const uint8_t* src, float (&x)[R_PART]) {
  if (BF16) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 w = s4[i];
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[8 * i + 2 * j] = __uint_as_float(ws[j] << 16);
        x[8 * i + 2 * j + 1] = __uint_as_float(ws[j] & 0xffff0000u);
      }
    }
  } else {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 w = s4[i];
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        unpack_e4m3x2(static_cast<uint16_t>(ws[j] & 0xffffu), x[16 * i + 4 * j], x[16 * i + 4 * j + 1]);
        unpack_e4m3x2(static_cast<uint16_t>(ws[j] >> 16), x[16 * i + 4 * j + 2], x[16 * i + 4 * j + 3]);
      }
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(R_THREADS) attn_fwd_redo_kernel(const RedoParams p) {
  constexpr int ES = BF16 ? 2 : 1;                 // bytes per element
  __shared__ __align__(16) uint8_t k_s[R_KEYS * R_D * ES];
  __shared__ __align__(16) uint8_t v_s[R_KEYS * R_D * ES];
  const int ROW_BYTES = p.d * ES;
  const int CHUNK_VECS = R_KEYS * ROW_BYTES / 16;  // 16-byte vectors per chunk

  const int tid = threadIdx.x;
  const int r = tid >> 2;     // query row of the block
  const int part = tid & 3;   // which 32 head-dim elements
  const bool part_ok = part * R_PART < p.d;
  const int num_m = (p.Nq + R_BM - 1) / R_BM;
  const int total = p.B * p.Hq * num_m;

  // launched with programmatic stream serialisation: the launch itself overlaps the end of the forward kernel, and
  // the flags are read only once that kernel has completed
  pdl_wait();
  // Every CTA owns a contiguous range of flags and looks at all of them at once, one per thread: with nothing
  // flagged (the normal case) the kernel is one load per thread and a barrier.
  const int per_cta = (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int first = static_cast<int>(blockIdx.x) * per_cta;
  const int last = min(total, first + per_cta);
  int any = 0;
  for (int i = first + tid; i < last; i += R_THREADS) any |= p.flags[i];
  if (!__syncthreads_or(any)) return;

  for (int blk = first; blk < last; ++blk) {
    const int flagged = p.flags[blk];  // the same word for every thread: the branch is uniform
    if (!flagged) continue;
    __syncthreads();  // everybody has read the flag
    if (tid == 0) p.flags[blk] = 0;  // the workspace is handed back all zero

    const int m_blk = blk % num_m;
    const int hq = (blk / num_m) % p.Hq;
    const int b = blk / (num_m * p.Hq);
    const int hkv = hq / (p.Hq / p.Hkv);
    const int nk = p.seqused_k ? max(0, min(p.Nk, p.seqused_k[b])) : p.Nk;
    const int shift = nk - p.Nq;  // key j is visible to query i iff j <= i + shift (causal)
    const int m0 = m_blk * R_BM;
    const int row = m0 + r;
    const bool row_ok = row < p.Nq;
    int limit = p.causal ? min(row + shift, nk - 1) : nk - 1;  // last visible key of this row
    if (!row_ok) limit = -1;
    int n_keys = nk;  // keys any row of the block can see
    if (p.causal) n_keys = max(0, min(nk, min(m0 + R_BM, p.Nq) - 1 + shift + 1));
    const int sc = b * p.Hkv + hkv;
    const float beta =
        p.softmax_scale * (BF16 ? 1.f : p.q_descale[sc] * p.k_descale[sc]) * 1.4426950408889634f;
    const float sv = BF16 ? 1.f : p.v_descale[sc];

    float qf[R_PART];
    if (row_ok && part_ok) {
      load32<BF16>(p.q + (b * p.q_strides[0] + hq * p.q_strides[1] + static_cast<int64_t>(row) * p.q_strides[2] +
                          part * R_PART) * ES, qf);
    } else {
#pragma unroll
      for (int i = 0; i < R_PART; ++i) qf[i] = 0.f;
    }
    const uint8_t* k_base = p.k + (b * p.k_strides[0] + hkv * p.k_strides[1]) * ES;
    const uint8_t* v_base = p.v + (b * p.v_strides[0] + hkv * p.v_strides[1]) * ES;

    // the chunk of keys [c0, c0 + 64) into shared memory; rows past the end are zero
    auto stage = [&](const uint8_t* base, int64_t stride_n, uint8_t* dst, int c0) {
      for (int vec = tid; vec < CHUNK_VECS; vec += R_THREADS) {
        const int key = c0 + vec / (ROW_BYTES / 16);
        const int off = (vec % (ROW_BYTES / 16)) * 16;
        uint4 w = make_uint4(0, 0, 0, 0);
        if (key < nk) w = *reinterpret_cast<const uint4*>(base + static_cast<int64_t>(key) * stride_n * ES + off);
        *reinterpret_cast<uint4*>(dst + (key - c0) * ROW_BYTES + off) = w;
      }
    };
    // score of this thread's row against key j of the staged chunk (the four threads of a row each hold a quarter)
    auto score = [&](int j) {
      float acc = 0.f;
      if (part_ok) {
        float kf[R_PART];
        load32<BF16>(k_s + j * ROW_BYTES + part * R_PART * ES, kf);
#pragma unroll
        for (int i = 0; i < R_PART; ++i) acc = fmaf(qf[i], kf[i], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      return acc * beta;
    };

    // pass 1: the exact row maximum
    float m = -INFINITY;
    for (int c0 = 0; c0 < n_keys; c0 += R_KEYS) {
      __syncthreads();
      stage(k_base, p.k_strides[2], k_s, c0);
      __syncthreads();
      const int jn = min(R_KEYS, n_keys - c0);
      for (int j = 0; j < jn; ++j) {
        const float s = score(j);
        if (c0 + j <= limit) m = fmaxf(m, s);
      }
    }
    // pass 2: sums and P.V against that maximum
    float l = 0.f;
    float o[R_PART];
#pragma unroll
    for (int i = 0; i < R_PART; ++i) o[i] = 0.f;
    for (int c0 = 0; c0 < n_keys; c0 += R_KEYS) {
      __syncthreads();
      stage(k_base, p.k_strides[2], k_s, c0);
      stage(v_base, p.v_strides[2], v_s, c0);
      __syncthreads();
      const int jn = min(R_KEYS, n_keys - c0);
      for (int j = 0; j < jn; ++j) {
        const float s = score(j);
        if (c0 + j <= limit) {
          const float pj = exp2f(s - m);
          l += pj;
          if (part_ok) {
            float vf[R_PART];
            load32<BF16>(v_s + j * ROW_BYTES + part * R_PART * ES, vf);
#pragma unroll
            for (int i = 0; i < R_PART; ++i) o[i] = fmaf(pj, vf[i], o[i]);
          }
        }
      }
    }

    if (row_ok) {
      const bool empty = !(l > 0.f);
      const float inv = empty ? 0.f : sv / l;
      __nv_bfloat16* out_row = p.out + b * p.out_strides[0] + hq * p.out_strides[1] +
                               static_cast<int64_t>(row) * p.out_strides[2] + part * R_PART;
      uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
      for (int i = 0; part_ok && i < 4; ++i) {
        uint4 w;
        w.x = pack_bf16x2(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
        w.y = pack_bf16x2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
        w.z = pack_bf16x2(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
        w.w = pack_bf16x2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
        dst[i] = w;
      }
      if (p.write_lse && part == 0) {
        const int64_t off = b * p.lse_stride_b + hq * p.lse_stride_h + row;
        const float lse = empty ? INFINITY : m + log2f(l);
        p.lse[off] = p.lse_natural ? lse * 0.6931471805599453f : lse;
        p.pmax[off] = empty ? 0.f : exp2f(m - lse);
      }
    }
  }
}

}  // namespace

int64_t attn_fwd_flag_bytes(int B, int Hq, int Nq) {
  const int64_t blocks = static_cast<int64_t>(B) * Hq * ((Nq + R_BM - 1) / R_BM);
  return (blocks * 4 + 15) / 16 * 16;
}

int launch_attn_fwd_redo(const wk_attn_fwd_args* a, bool bf16, int* flags, cudaStream_t st) {
  RedoParams p;
  p.q = static_cast<const uint8_t*>(a->q);
  p.k = static_cast<const uint8_t*>(a->k);
  p.v = static_cast<const uint8_t*>(a->v);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.pmax = a->pmax;
  p.q_descale = a->q_descale;
  p.k_descale = a->k_descale;
  p.v_descale = a->v_descale;
  for (int i = 0; i < 3; ++i) {
    p.q_strides[i] = a->q_strides[i];
    p.k_strides[i] = a->k_strides[i];
    p.v_strides[i] = a->v_strides[i];
    p.out_strides[i] = a->out_strides[i];
  }
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
  p.flags = flags;
  const int64_t blocks = static_cast<int64_t>(a->B) * a->Hq * ((a->Nq + R_BM - 1) / R_BM);
  if (blocks > 0x7fffffff) return WK_E_ARG;
  int sms = sm_count();
  if (sms <= 0) return WK_E_CUDA;
  const int grid = static_cast<int>(blocks < sms ? blocks : sms);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(R_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = bf16 ? cudaLaunchKernelEx(&cfg, attn_fwd_redo_kernel<true>, p)
                             : cudaLaunchKernelEx(&cfg, attn_fwd_redo_kernel<false>, p);
  return e == cudaSuccess ? 0 : WK_E_CUDA;
}

}  // namespace wk

extern "C" int64_t wk_attn_fwd_workspace_bytes(int B, int Hq, int Nq) {
  if (B <= 0 || Hq <= 0 || Nq <= 0) return 0;
  return wk::attn_fwd_flag_bytes(B, Hq, Nq);
}
