"""ctypes binding of ``libwarpy_b200.so`` (declared in ``include/warpy_b200.h``).

This plays the role of the reference's TVM-FFI call (``warpy_kernels/utils/__init__.py:44-52``): the
single place where Python hands raw device pointers to compiled kernels.  There is no fallback: if the
library is missing the import of any kernel wrapper fails with an explicit error.
"""

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# the library built next to this file; WARPY_KERNELS_B200_LIB points at another build of it (e.g. one with a probe)
LIB_PATH = os.environ.get("WARPY_KERNELS_B200_LIB") or os.path.join(_HERE, "libwarpy_b200.so")

_i32, _i64, _ptr, _str = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p

WK_BF16, WK_F32 = 0, 1

# name -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "wk_query": (_i32, [_str]),
    "wk_device_arch": (_i32, [_i32]),
    "wk_status": (_i32, []),
    "wk_error_string": (_str, [_i32]),
    "wk_quantize_mx": (_i32, [_ptr, _i32, _i64, _i64, _i64, _ptr, _ptr, _ptr]),
    "wk_gemm_bf16": (_i32, [_ptr, _ptr, _ptr, _i32, _i32, _i32, _ptr]),
    "wk_gemm_16bit": (_i32, [_ptr, _ptr]),
    "wk_attn_fwd_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "wk_attn_fwd_fp8": (_i32, [_ptr, _ptr]),
    "wk_attn_fwd_bf16": (_i32, [_ptr, _ptr]),
    "wk_attn_bwd_fp8_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "wk_attn_bwd_fp8": (_i32, [_ptr, _ptr]),
    "wk_attn_bwd_bf16_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "wk_attn_bwd_bf16": (_i32, [_ptr, _ptr]),
    "wk_gemm_mxfp8_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "wk_gemm_mxfp8": (_i32, [_ptr, _ptr]),
    "wk_mx_scales_tiled_bytes": (_i64, [_i32, _i32]),
    "wk_tile_mx_scales": (_i32, [_ptr, _i32, _i32, _ptr, _ptr]),
    "wk_gemm_mxfp8_noalloc": (_i32, [_ptr, _ptr]),
    "wk_gemm_mxfp8_noalloc_max_bytes": (_i64, []),
    "wk_gemm_mxfp8_noalloc_status": (_i32, []),
}

_lib = None


def lib():
    """Return the loaded library, loading it on first use.

    Raises:
        RuntimeError: If ``libwarpy_b200.so`` has not been built (run ``python -c "import __graft_entry__ as g;
            g.build()"`` or ``make -C warpy_kernels_b200/csrc``). There is deliberately no CPU or PyTorch fallback.
    """
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}`; "
                "warpy_kernels has no fallback path"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def stream_ptr(device=None):
    """``cudaStream_t`` of torch's current stream on ``device`` as an integer."""
    return torch.cuda.current_stream(device).cuda_stream


def check(code, what):
    """Turn a negative return code of the C ABI into a Python exception."""
    if code == 0:
        return
    text = lib().wk_error_string(code).decode()
    if code == -1:
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: {text} (code {code})")


def device_status():
    """Synchronise the current device and raise if a kernel gave up on a bounded wait."""
    code = lib().wk_status()
    if code != 0:
        raise RuntimeError(f"warpy_kernels device status {code}: {lib().wk_error_string(code).decode()}")
