/* C ABI of libwarpy_b200.so: the sm_100a kernels behind the warpy_kernels Python
 * surface (attn_fwd, attn_bwd, gemm, MXFP8 quantiser).
 *
 * Conventions
 *  - Every pointer is a device pointer of the CUDA device that is current when the
 *    call is made, unless stated otherwise.  No torch types cross this boundary.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *  - Calls only enqueue work; they never synchronise.  Return value: 0 on success,
 *    a negative WK_E_* code when an argument is rejected (nothing was launched) or
 *    the CUDA runtime refused the launch.
 *  - Kernels never spin without a limit: a wait that exceeds two seconds makes the
 *    kernel record a positive code in a per-device status word and leave.
 *    wk_status() synchronises the device and returns (and clears) that word.
 *
 * In the reference every kernel is reached through one generic TVM-FFI call,
 *   warpy_kernels/utils/__init__.py:44-52 (compile_cached -> compiled(*targs, *sargs)),
 * fed by the argument lists built in attn/fwd_api.py:344-353, attn/bwd_api.py:232-380
 * and gemm/api.py:216-234.  Each entry point below replaces that call for one
 * kernel family and takes the same tensors as plain pointers, sizes and strides.
 */
#ifndef WARPY_B200_H
#define WARPY_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* argument / launch errors (negative) */
#define WK_E_ARG (-1)       /* a size, stride, alignment or pointer was rejected */
#define WK_E_CUDA (-2)      /* the CUDA runtime or driver returned an error */
#define WK_E_UNSUPPORTED (-3) /* the device is not compute capability 10.x */
#define WK_E_TOO_LARGE (-4) /* the problem does not fit the fixed scratch of a no-allocation entry point */

/* Size of the scratch array built into the library for wk_gemm_mxfp8_noalloc. */
#define WK_NOALLOC_SCRATCH_BYTES (8ll << 20)

/* dtype codes */
#define WK_BF16 0
#define WK_F32 1

/* Replaces warpy_kernels/arch.py:69-94 (supports): 1 if `feature` ("gemm",
 * "gemm_fp8", "gemm_mx", "gemm_mx_out", "attn_fwd_fp8", "attn_bwd_fp8", ...) has a
 * kernel in this library, 0 if not, WK_E_ARG for an unknown name.  Host only. */
int wk_query(const char* feature);

/* Replaces warpy_kernels/arch.py:29-60 (device_arch): 100 if CUDA device `device` (-1 = the current one)
 * is compute capability 10.x, WK_E_UNSUPPORTED if it is anything else, WK_E_CUDA if there is no such
 * device.  Every compute entry point below makes the same check on the current device before it
 * launches anything.  Host only. */
int wk_device_arch(int device);

/* Synchronises the current device, returns its status word (0 = no kernel gave up
 * on a wait) and clears it.  Negative on a CUDA error. */
int wk_status(void);

/* Human-readable text for a return code or status word.  Host only. */
const char* wk_error_string(int code);

/* MXFP8 quantiser.  Replaces the reference's GEMM epilogue helper
 * warpy_kernels/gemm/sm89.py:65-93 (_store_mx) with warpy_kernels/ptx/common.py:539-565
 * (abs_bits, mx_scale) and warpy_kernels/ptx/sm89.py:85-93 (pack_e4m3x2) as a
 * standalone pass.
 *   x      [rows, cols] row-major, leading dimension ld_x elements, dtype WK_BF16 or WK_F32
 *   q      [rows, cols] e4m3 codes, contiguous
 *   s      [rows, cols/32] ue8m0 scale bytes, contiguous
 * cols % 32 == 0; x and q 16-byte aligned; ld_x % 8 == 0. */
int wk_quantize_mx(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x, void* q,
                   void* s, void* stream);

/* BF16 GEMM, out[M,N] = a[M,K] @ b[N,K]^T with fp32 accumulation, bf16 output.
 * Replaces the launch of GemmSm120 for 16-bit inputs, warpy_kernels/gemm/api.py:216-267
 * (kernel: warpy_kernels/gemm/base.py:382-423).
 * a, b, out contiguous row-major and 16-byte aligned; M % 128 == 0, N % 128 == 0,
 * K % 64 == 0. */
int wk_gemm_bf16(const void* a, const void* b, void* out, int m, int n, int k, void* stream);

/* 16-bit GEMM with the reference's fused epilogue (warpy_kernels/gemm/base.py:436-497):
 *   out = act((a @ b^T) . scale_a . scale_b [+ out])
 * a, b, out (and the pre buffers) are bf16, or fp16 when f16 != 0.  Other fields as in
 * wk_gemm_mx_args.  wk_gemm_bf16 is this call with every option off. */
typedef struct {
  const void* a;
  const void* b;
  void* out;
  int32_t m, n, k;
  int32_t f16;
  const float* scale_a;
  const float* scale_b;
  int32_t scale_a_rows;
  int32_t scale_b_cols;
  int32_t accum;
  int32_t act;
  void* pre_out;
  const void* pre_in;
  void* q_mx; /* optional [M, N] e4m3 copy of out, with s_mx [M, N/32]; N % 32 == 0 */
  void* s_mx;
  int32_t a_trans; /* a is stored [K, M] (warpy_kernels/gemm/api.py:103-104, gemm/base.py:127-135) */
  int32_t b_trans; /* b is stored [K, N] */
  int32_t cta_pair; /* 1: the CTA-pair kernel (tcgen05 cta_group::2, one 256 x 256 tile per two SMs).  2: never pairs.
                       0: the library's choice (pairs when the 256 x 256 tiles fill the GPU about as well as
                       128 x 256 ones).  The results are bit-identical either way. */
  int32_t group_m;  /* the reference's tuning option of that name (warpy_kernels/gemm/api.py:55, base.py:87-103):
                       output tiles are visited in groups of group_m tile rows that sweep all tile columns, so the
                       CTAs running at the same time share operand rows in L2.  0 = 8.  Any value gives the same bits. */
} wk_gemm16_args;

int wk_gemm_16bit(const wk_gemm16_args* args, void* stream);

/* MXFP8 block-scaled GEMM,
 *   out[M,N] = scale_a . scale_b . (a . 2^(a_scale_mx-127)) @ (b . 2^(b_scale_mx-127))^T,
 * e4m3 operands, fp32 accumulation, bf16 output.  Replaces the launch of GemmSm120 for
 * fp8 inputs, warpy_kernels/gemm/api.py:216-267 (block-scaled MMA path:
 * warpy_kernels/gemm/sm120.py:121-146; MX output epilogue: warpy_kernels/gemm/sm89.py:65-93).
 *   a [M,K], b [N,K]           e4m3 bytes, contiguous, 16-byte aligned
 *   a_scale_mx [M,K/32]        ue8m0 bytes, contiguous, 4-byte aligned, or NULL for unit scales
 *   b_scale_mx [N,K/32]        same for b (the reference scales only a; NULL reproduces it)
 *   scale_a, scale_b           optional device pointers to fp32 scales (NULL = 1): one entry, or one per
 *                              output row / column when scale_a_rows / scale_b_cols is set
 *   out [M,N] bf16 (fp16 when out_f16)   contiguous, 16-byte aligned
 *   q_mx [M,N] e4m3, s_mx [M,N/32] ue8m0   optional (both or neither): the fp32 results
 *                              quantised per row and 32 columns before the bf16 rounding
 *   workspace                  scratch of at least wk_gemm_mxfp8_workspace_bytes(M,N,K) bytes,
 *                              16-byte aligned; holds the re-tiled scale factors of this call
 * M % 128 == 0, N % 128 == 0, K % 128 == 0. */
typedef struct {
  const void* a;
  const void* b;
  const void* a_scale_mx;
  const void* b_scale_mx;
  const float* scale_a;
  const float* scale_b;
  void* out;
  void* q_mx;
  void* s_mx;
  void* workspace;
  int64_t workspace_bytes;
  int32_t m, n, k;
  /* fused epilogue, warpy_kernels/gemm/base.py:436-497; all zero = plain product */
  int32_t scale_a_rows; /* 1: scale_a holds M entries (one per output row) instead of one */
  int32_t scale_b_cols; /* 1: scale_b holds N entries (one per output column), 16-byte aligned */
  int32_t accum;        /* 1: add the scaled product to the values out already holds */
  int32_t act;          /* 0 none, 1 exact-erf GELU, 2 multiply by GELU'(pre_in) */
  int32_t out_f16;      /* 0: out / pre buffers are bf16, 1: fp16 */
  void* pre_out;        /* optional [M,N]: the value before the activation (act = 1) */
  const void* pre_in;   /* [M,N] pre-activation values, required for act = 2 */
  int32_t cta_pair;     /* kernel choice as in wk_gemm16_args: 0 the library's, 1 CTA pairs (tcgen05 cta_group::2, one
                           256 x 256 tile per two SMs), 2 single CTAs; bit-identical results.  wk_gemm_mxfp8_noalloc
                           always runs single CTAs. */
  int32_t a_scale_tiled; /* 1: a_scale_mx is not the row-major [M, K/32] tensor but the output of wk_tile_mx_scales
                            for it (16-byte aligned): the layout the kernels read, made once for scales that do not
                            change from call to call (weights).  0: row-major, re-tiled into the workspace per call. */
  int32_t b_scale_tiled; /* the same for b_scale_mx.  With both set the workspace may be NULL. */
  int32_t group_m;       /* as in wk_gemm16_args; 0 = 8 */
} wk_gemm_mx_args;

int64_t wk_gemm_mxfp8_workspace_bytes(int m, int n, int k);
int wk_gemm_mxfp8(const wk_gemm_mx_args* args, void* stream);

/* Re-tiles MX scale bytes for wk_gemm_mxfp8: s [rows, k/32] ue8m0 row-major (NULL: unit scales) ->
 * dst, wk_mx_scales_tiled_bytes(rows, k) bytes, 16-byte aligned: one 512-byte atom per 128 rows and 128 K
 * elements (byte (row % 32) * 16 + (row / 32 % 4) * 4 + kblock % 4), atoms ordered [row block][K block], which is
 * how tcgen05.mma reads block scales from tensor memory.  rows % 128 == 0, k % 128 == 0.  No counterpart in the
 * reference, whose mma.sync kernels read the row-major tensor (warpy_kernels/gemm/sm120.py:121-146). */
int64_t wk_mx_scales_tiled_bytes(int rows, int k);
int wk_tile_mx_scales(const void* s, int rows, int k, void* dst, void* stream);

/* MXFP8 GEMM for callers that cannot allocate device memory.  No counterpart in the
 * reference (its host API allocates its workspaces with torch on every make_gemm).
 *
 * Who needs it: code that runs inside a process whose GPU memory has already been
 * handed out in full -- an inference server that reserves the whole card for its own
 * pool at start-up, a plugin that is only given pre-made buffers -- or on a latency
 * path where a cudaMalloc (which may synchronise the device, and may simply fail) is
 * not acceptable.  Such a caller still passes a, b, the scale tensors and the outputs,
 * but no workspace: `workspace` and `workspace_bytes` of the argument block are
 * ignored, and the re-tiled scale factors go into an array of WK_NOALLOC_SCRATCH_BYTES
 * bytes that is part of the library image on every GPU that loads it.  This entry
 * point calls no cudaMalloc, cudaFree or other allocating routine, not even for the
 * status word: wk_gemm_mxfp8_noalloc_status() reads its own.
 *
 * Limits and rules
 *  - (M + N) * K / 32 + 32 must not exceed WK_NOALLOC_SCRATCH_BYTES (see
 *    wk_gemm_mxfp8_noalloc_max_bytes()); larger problems return WK_E_TOO_LARGE and
 *    launch nothing.
 *  - The first call on a device looks up the array's device address; make that first
 *    call on each device before starting any stream capture.
 *  - All calls on a device share the one array.  Each call rewrites every byte it
 *    later reads, so earlier contents never leak into a result, but two calls that
 *    can run at the same time on the GPU (different streams) race on it: keep calls
 *    to this entry point on one stream, or order them with events.
 * Otherwise identical to wk_gemm_mxfp8 (same kernels, bit-identical results). */
int wk_gemm_mxfp8_noalloc(const wk_gemm_mx_args* args, void* stream);
int64_t wk_gemm_mxfp8_noalloc_max_bytes(void);
/* wk_status() for the no-allocation entry point: synchronises, returns and clears the
 * status word its kernels report to. */
int wk_gemm_mxfp8_noalloc_status(void);

/* FP8 attention forward.  Replaces the launch built in
 * warpy_kernels/attn/fwd_api.py:344-390 (kernel: warpy_kernels/attn/fwd_base.py:670-758 with the
 * e4m3 overrides of warpy_kernels/attn/fwd_sm120.py:81-136).
 *   q [B,Hq,Nq,d], k,v [B,Hkv,Nk,d]  e4m3 bytes; *_strides = element (= byte) strides of
 *       dims (B, H, N), the last dimension is contiguous; every stride and base address
 *       a multiple of 16; d == 128; Hq % Hkv == 0
 *   out [B,Hq,Nq,d] bf16, out_strides in elements (multiples of 8), base 16-byte aligned
 *   lse, pmax  fp32, element strides lse_strides = (B, H) with rows contiguous; may be
 *       NULL when write_lse == 0
 *   q/k/v_descale  fp32 [B,Hkv] contiguous
 *   causal: bottom-right aligned mask (key j visible to query i iff j <= i + Nk - Nq,
 *       with Nk replaced by seqused_k[b] when that is given)
 *   softmax_scale > 0
 * Outputs: out = softmax(scale . q k^T) v on the dequantised inputs; lse = base-2
 * log-sum-exp of the scaled logits (+inf for rows without a visible key, which get
 * out = 0 and pmax = 0); pmax = largest probability of the row. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* pmax;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  int64_t q_strides[3];
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t out_strides[3];
  int64_t lse_strides[2];
  int32_t B, Hq, Hkv, Nq, Nk, d;
  int32_t causal;
  int32_t write_lse;
  int32_t lse_natural;      /* 1: lse is written in natural log units instead of base 2 */
  const int32_t* seqused_k; /* optional [B] int32: keys each batch item attends to (<= Nk) */
  float softmax_scale;
  int32_t ctas_per_sm; /* fp8 forward: 2 = two CTAs per SM with 64-key tiles, 1 = one CTA per SM with 128-key
                          rounds and four softmax groups (long sequences), 0 = pick by Nk.  The reference's
                          tuning option of the same name (warpy_kernels/attn/fwd_api.py:196-208) */
  void* workspace;     /* optional scratch of wk_attn_fwd_workspace_bytes(B, Hq, Nq) bytes, 4-byte aligned: one
                          flag per block of 128 queries.  It must hold zeros when the call is made and holds zeros
                          again when the call's work has completed, so one buffer can serve every call on a stream.
                          The tensor-core kernels keep one reference exponent per query row, taken from the row's
                          first 64 keys; a query block in which some later key lies more than 2^100 (69 nats) above
                          it is flagged there and recomputed by a plain two-pass fp32 kernel (exact row maximum
                          first), which is what the reference's moving tile maximum
                          (warpy_kernels/attn/fwd_base.py:337-360) achieves.  NULL: no recomputation; such an
                          input then leaves WK_ERR_RANGE (110) in the status word and a wrong result. */
  int64_t workspace_bytes;
} wk_attn_fwd_args;

int64_t wk_attn_fwd_workspace_bytes(int B, int Hq, int Nq);
int wk_attn_fwd_fp8(const wk_attn_fwd_args* args, void* stream);

/* BF16 attention forward: q, k, v bf16 (element strides multiples of 8), the three descale
 * pointers NULL, everything else as for wk_attn_fwd_fp8.  Replaces the same launch for 16-bit
 * inputs (warpy_kernels/attn/fwd_api.py:383-390, kernel warpy_kernels/attn/fwd_base.py:374-416). */
int wk_attn_fwd_bf16(const wk_attn_fwd_args* args, void* stream);

/* FP8 attention backward.  Replaces the launches of warpy_kernels/attn/bwd_api.py:381-398
 * (BwdPrep warpy_kernels/attn/bwd_common.py:23-266, AttnBwdSm120 warpy_kernels/attn/bwd_sm120.py:38-1202,
 * BwdDqPost warpy_kernels/attn/bwd_common.py:307-403).
 *   q [B,Hq,Nq,d], k,v [B,Hkv,Nk,d]  e4m3, strides as in wk_attn_fwd_args
 *   out, dout [B,Hq,Nq,d] bf16, element strides of (B, H, N) multiples of 4, last dim contiguous,
 *       base 8-byte aligned
 *   lse   fp32 base-2 log-sum-exp of the forward (+inf for rows without a visible key),
 *       element strides lse_strides = (B, H)
 *   dq [B,Hq,Nq,d], dk, dv [B,Hkv,Nk,d]  bf16 contiguous, 16-byte aligned: gradients with
 *       respect to the dequantised q, k, v
 *   workspace: scratch of wk_attn_bwd_fp8_workspace_bytes(B, Hq, Nq) bytes, 16-byte aligned
 *       (the e4m3 copy of dout and one 16-byte record per query row)
 * d == 128, Hq % Hkv == 0, softmax_scale > 0. */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* out;
  const void* dout;
  const float* lse;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  void* dq;
  void* dk;
  void* dv;
  void* workspace;
  int64_t workspace_bytes;
  int64_t q_strides[3];
  int64_t k_strides[3];
  int64_t v_strides[3];
  int64_t out_strides[3];
  int64_t dout_strides[3];
  int64_t lse_strides[2];
  int32_t B, Hq, Hkv, Nq, Nk, d;
  int32_t causal;
  float softmax_scale;
} wk_attn_bwd_args;

int64_t wk_attn_bwd_fp8_workspace_bytes(int B, int Hq, int Nq);
int wk_attn_bwd_fp8(const wk_attn_bwd_args* args, void* stream);

/* BF16 attention backward: q, k, v and dout bf16 read through TMA (16-byte aligned, element strides
 * multiples of 8), the three descale pointers NULL, workspace of wk_attn_bwd_bf16_workspace_bytes
 * (one 16-byte record per query row); everything else as for wk_attn_bwd_fp8.  Replaces the same
 * launches for 16-bit inputs (warpy_kernels/attn/bwd_api.py:381-398, bwd_sm120.py:436-464). */
int64_t wk_attn_bwd_bf16_workspace_bytes(int B, int Hq, int Nq);
int wk_attn_bwd_bf16(const wk_attn_bwd_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WARPY_B200_H */
