// Recomputation of query blocks the tensor-core forward kernels flagged as out of their exponent range
// (attn_fwd_redo.cu), shared by the FP8 and BF16 forward entry points.
#pragma once
#include "host_common.h"

namespace wk {

// Bytes of the flag array for a call: one int per block of 128 queries of every (batch, query head).
int64_t attn_fwd_flag_bytes(int B, int Hq, int Nq);

// Flag index of query block m_blk of (b, hq); the forward kernels and the recomputation agree on it.
__host__ __device__ inline int attn_fwd_flag_index(int b, int hq, int m_blk, int Hq, int num_m) {
  return (b * Hq + hq) * num_m + m_blk;
}

// Enqueues the recomputation of every flagged block of the call described by `a` (q, k, v e4m3, or bf16 when
// `bf16`) on `st`, after the forward kernels; clears the flags it finds.  0 or a negative WK_E_* code.
int launch_attn_fwd_redo(const wk_attn_fwd_args* a, bool bf16, int* flags, cudaStream_t st);

}  // namespace wk
