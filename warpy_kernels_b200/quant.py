"""Standalone MXFP8 quantiser: the arithmetic of the reference's ``out_mx`` GEMM epilogue as its own pass.

Reference arithmetic: ``warpy_kernels/gemm/sm89.py:65-93`` (``_store_mx``), ``warpy_kernels/ptx/common.py:539-565``
(``abs_bits``, ``mx_scale``), ``warpy_kernels/ptx/sm89.py:85-93`` (``pack_e4m3x2``).
"""

import torch

from . import _lib
from .arch import require


def quantize_mx(x, q=None, s=None):
    """Quantise ``x`` to MXFP8 along its last dimension.

    Args:
        x: ``[M, K]`` bf16 or float32 CUDA tensor with last stride 1, ``K`` a multiple of 32, rows 16-byte aligned.
        q: Optional contiguous ``[M, K]`` ``torch.float8_e4m3fn`` output.
        s: Optional contiguous ``[M, K / 32]`` uint8 output.

    Returns:
        ``(q, s)``: e4m3 codes and one ue8m0 scale byte per row and block of 32 consecutive elements, each block
        scaled by the smallest power of two that keeps it within 448. ``q.float() * 2 ** (s - 127)`` dequantises.

    Raises:
        ValueError: If the dtype, shape, strides or alignment are unsupported.
        NotImplementedError: If the GPU is not supported.
    """
    if x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("x must be a [M, K] bf16 or float32 tensor")
    require("gemm_mx_out", x)
    m, k = x.shape
    if k % 32:
        raise ValueError(f"K must be a multiple of 32, got {k}")
    if m > 1 and (x.stride(1) != 1 or x.stride(0) % 8) or (m <= 1 and k and x.stride(1) != 1):
        raise ValueError("x needs last stride 1 and a row stride that is a multiple of 8 elements")
    if q is None:
        q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    elif q.shape != x.shape or q.dtype != torch.float8_e4m3fn or not q.is_contiguous() or q.device != x.device:
        raise ValueError("q must be a contiguous float8_e4m3fn tensor shaped like x")
    if s is None:
        s = torch.empty(m, k // 32, dtype=torch.uint8, device=x.device)
    elif s.shape != (m, k // 32) or s.dtype != torch.uint8 or not s.is_contiguous() or s.device != x.device:
        raise ValueError(f"s must be a contiguous [{m}, {k // 32}] uint8 tensor")
    ld = x.stride(0) if m > 1 else max(k, 8)
    with torch.cuda.device(x.device):
        code = _lib.lib().wk_quantize_mx(
            x.data_ptr(),
            _lib.WK_BF16 if x.dtype == torch.bfloat16 else _lib.WK_F32,
            m,
            k,
            ld,
            q.data_ptr(),
            s.data_ptr(),
            _lib.stream_ptr(x.device),
        )
    _lib.check(code, "quantize_mx")
    return q, s
