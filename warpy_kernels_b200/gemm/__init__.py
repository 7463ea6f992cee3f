from .api import autotune_gemm, gemm, make_gemm

__all__ = ["autotune_gemm", "gemm", "make_gemm"]
