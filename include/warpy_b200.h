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

/* dtype codes */
#define WK_BF16 0
#define WK_F32 1

/* Replaces warpy_kernels/arch.py:69-94 (supports): 1 if `feature` ("gemm",
 * "gemm_fp8", "gemm_mx", "gemm_mx_out", "attn_fwd_fp8", "attn_bwd_fp8", ...) has a
 * kernel in this library, 0 if not, WK_E_ARG for an unknown name.  Host only. */
int wk_query(const char* feature);

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

#ifdef __cplusplus
}
#endif
#endif /* WARPY_B200_H */
