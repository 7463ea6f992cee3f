"""B200 (sm_100a) implementation of the warpy-kernels hot path behind the reference's Python surface."""

from .arch import device_arch, supports
from .interface import attn_bwd, attn_fwd, autotune_gemm, gemm, make_gemm
from .quant import quantize_mx

__all__ = [
    "attn_bwd",
    "attn_fwd",
    "autotune_gemm",
    "device_arch",
    "gemm",
    "make_gemm",
    "quantize_mx",
    "supports",
]
