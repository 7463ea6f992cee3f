"""GEMM host API with the reference's call surface (``warpy_kernels/gemm/api.py:45-391``).

``out = a @ b.T * scale_a * scale_b`` for bf16 inputs (tcgen05 ``kind::f16``) and e4m3 inputs (tcgen05
``kind::mxf8f6f4`` with ue8m0 scales per 32 elements along K; unit scales when none are given).  The reference's
SM80-SM120 tuning knobs (``bk, stages, group_m, min_blocks, bn, frag_pipe, tma, warp_spec, persistent,
setmaxnreg``) are accepted so existing call sites keep working; the sm_100a kernels have one fixed tiling and
ignore them, except that ``bn`` and ``bk`` still define the divisibility the reference enforces.
"""

import ctypes

import torch

from .. import _lib
from ..arch import require
from ..utils import time_candidates

_TYPES = {torch.bfloat16: "bf16", torch.float16: "f16"}
BM = 128


class _MxArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("a_scale_mx", ctypes.c_void_p),
        ("b_scale_mx", ctypes.c_void_p), ("scale_a", ctypes.c_void_p), ("scale_b", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("q_mx", ctypes.c_void_p), ("s_mx", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
    ]


def _gemm_arch(a, fp8, act, accum, mx_in, mx_out):
    arch = require("gemm", a)
    for on, feature in (
        (fp8, "gemm_fp8"),
        (act == "gelu", "gemm_gelu"),
        (act == "dgelu", "gemm_dgelu"),
        (accum, "gemm_accum"),
        (mx_in, "gemm_mx"),
        (mx_out, "gemm_mx_out"),
    ):
        if on:
            require(feature, a)
    return arch


def _check_mx(name, s, rows, k, fp8):
    if s is not None and (
        not fp8 or s.dtype != torch.uint8 or s.shape != (rows, k // 32) or not s.is_contiguous()
    ):
        raise ValueError(f"{name} must be a contiguous [{rows}, {k // 32}] uint8 tensor with fp8 inputs")


def make_gemm(
    a,
    b,
    out=None,
    bk=None,
    stages=3,
    group_m=8,
    min_blocks=1,
    bn=128,
    frag_pipe=False,
    tma=False,
    warp_spec=False,
    persistent=False,
    setmaxnreg=False,
    scale_a=None,
    scale_b=None,
    out_dtype=torch.bfloat16,
    act="",
    store_pre=False,
    pre=None,
    a_trans=False,
    b_trans=False,
    accum=False,
    a_scale_mx=None,
    out_mx=False,
    b_scale_mx=None,
):
    """Prepare ``out = a @ b.T * scale_a * scale_b``.

    Args:
        a: ``[M, K]`` bf16 or ``torch.float8_e4m3fn``, contiguous.
        b: ``[N, K]`` with the dtype of ``a``, contiguous.
        out: Optional contiguous ``[M, N]`` bf16 output, 16-byte aligned. Allocated if ``None``.
        bk: K elements per pipeline stage in the reference; here only the divisibility rule ``K % bk == 0`` is
            kept. Defaults to 64 for bf16 and 128 for fp8.
        stages, group_m, min_blocks, frag_pipe, tma, warp_spec, persistent, setmaxnreg: Accepted for
            compatibility and ignored: the sm_100a kernels are always TMA-fed, warp-specialised and persistent.
        bn: Output columns per CTA in the reference, 128 or 256; ``N`` must be a multiple of it.
        scale_a: Float32 CUDA tensor with one element that scales ``a`` (fp8 inputs only).
        scale_b: As ``scale_a``, for ``b``.
        out_dtype: Output dtype when ``out`` is ``None`` and the inputs are fp8; must be bf16.
        act, store_pre, pre, a_trans, b_trans, accum: The reference's epilogue fusions and transposed operands.
            Not implemented by this build; anything but the defaults raises ``NotImplementedError``.
        a_scale_mx: ``[M, K / 32]`` uint8 ue8m0 scales of ``a``, one per row and block of 32 along K, as
            ``out_mx`` writes them. Needs fp8 inputs.
        out_mx: Whether to also write the result as MXFP8: e4m3 values ``[M, N]`` and ``[M, N / 32]`` uint8 ue8m0
            scales computed from the fp32 values before they are rounded to bf16.
        b_scale_mx: ``[N, K / 32]`` uint8 ue8m0 scales of ``b``. Not in the reference (which scales only ``a``);
            ``None`` gives the reference's behaviour.

    Returns:
        ``(launch, out)``; with ``out_mx``, the e4m3 values and their scales follow. ``launch()`` runs the kernel
        on the current stream and fills the outputs.

    Raises:
        ValueError: If the dtype is unsupported, the shapes do not match, an input is not contiguous, or ``M`` is
            not a multiple of 128, ``N`` is not a multiple of ``bn`` or ``K`` is not a multiple of ``bk``.
        NotImplementedError: If the GPU does not support the dtype or a requested option.
    """
    fp8 = a.dtype == torch.float8_e4m3fn
    if (a.dtype not in _TYPES and not fp8) or b.dtype != a.dtype:
        raise ValueError("a and b must share a bf16, fp16 or float8_e4m3fn dtype")
    _gemm_arch(a, fp8, act, accum, a_scale_mx is not None or b_scale_mx is not None, out_mx)
    if a.dtype == torch.float16:
        raise NotImplementedError("warpy_kernels has no fp16 gemm for SM100 yet; supported: bfloat16 and float8_e4m3fn")
    if act or store_pre or pre is not None or a_trans or b_trans or accum:
        raise NotImplementedError(
            "warpy_kernels for SM100 has no act/store_pre/pre/a_trans/b_trans/accum gemm epilogue yet"
        )
    odt = out_dtype if fp8 and out is None else out.dtype if out is not None else a.dtype
    if odt not in _TYPES:
        raise ValueError("the output must be bf16 or fp16")
    if not fp8 and odt != a.dtype:
        raise ValueError(f"out must have the dtype of a and b for 16-bit inputs, got {odt} and {a.dtype}")
    if odt != torch.bfloat16:
        raise NotImplementedError("warpy_kernels for SM100 writes bf16 outputs only")
    bk = bk or (128 if fp8 else 64)
    if bn not in (128, 256):
        raise ValueError("bn must be 128 or 256")
    m, k = a.shape
    n, kb = b.shape
    if kb != k:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if not (a.is_contiguous() and b.is_contiguous()):
        raise ValueError("a and b must be contiguous")
    if m % BM or n % bn or k % bk or k % (128 if fp8 else 64):
        raise ValueError(f"M must be a multiple of 128, N of {bn} and K of {bk}, got {m}, {n}, {k}")
    if out is None:
        out = torch.empty(m, n, dtype=odt, device=a.device)
    elif out.shape != (m, n) or not out.is_contiguous() or out.data_ptr() % 16:
        raise ValueError("out must be a contiguous [M, N] tensor aligned to 16 bytes")
    alpha = 1.0
    for name, s, size in (("scale_a", scale_a, m), ("scale_b", scale_b, n)):
        if s is None:
            continue
        if s.dtype != torch.float32 or not s.is_cuda or s.numel() not in (1, size):
            raise ValueError(
                f"{name} must be a float32 CUDA tensor of 1 or {size} elements, contiguous and 8-byte aligned"
            )
        if s.numel() > 1 and size != 1:
            raise NotImplementedError("warpy_kernels for SM100 has no per-row / per-column gemm scales yet")
    _check_mx("a_scale_mx", a_scale_mx, m, k, fp8)
    _check_mx("b_scale_mx", b_scale_mx, n, k, fp8)
    q_mx = torch.empty(m, n, dtype=torch.float8_e4m3fn, device=a.device) if out_mx else None
    s_mx = torch.empty(m, n // 32, dtype=torch.uint8, device=a.device) if out_mx else None
    lib = _lib.lib()
    dev = a.device

    if not fp8:
        if out_mx:
            raise NotImplementedError("warpy_kernels for SM100 writes MXFP8 outputs from the fp8 gemm only")

        def launch():
            with torch.cuda.device(dev):
                code = lib.wk_gemm_bf16(
                    a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, _lib.stream_ptr(dev)
                )
            _lib.check(code, "gemm (bf16)")

    else:
        ws_bytes = lib.wk_gemm_mxfp8_workspace_bytes(m, n, k)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)  # re-tiled scale factors
        args = _MxArgs()
        args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
        args.a_scale_mx = a_scale_mx.data_ptr() if a_scale_mx is not None else None
        args.b_scale_mx = b_scale_mx.data_ptr() if b_scale_mx is not None else None
        args.scale_a = scale_a.data_ptr() if scale_a is not None else None
        args.scale_b = scale_b.data_ptr() if scale_b is not None else None
        args.q_mx = q_mx.data_ptr() if out_mx else None
        args.s_mx = s_mx.data_ptr() if out_mx else None
        args.workspace, args.workspace_bytes = workspace.data_ptr(), ws_bytes
        args.m, args.n, args.k = m, n, k
        keep = (a, b, a_scale_mx, b_scale_mx, scale_a, scale_b, workspace)

        def launch():
            with torch.cuda.device(dev):
                code = lib.wk_gemm_mxfp8(ctypes.byref(args), _lib.stream_ptr(dev))
            _lib.check(code, "gemm (fp8)")
            return keep

    mx = (q_mx, s_mx) if out_mx else ()
    return (launch, out, *mx)


def gemm(a, b, out=None, **kwargs):
    """Compute ``(a @ b.T) * scale_a * scale_b``; arguments as in ``make_gemm``.

    Returns:
        ``[M, N]`` in the output dtype. With ``out_mx``, a tuple that ends with the e4m3 values and their scales.
    """
    launch, out, *rest = make_gemm(a, b, out, **kwargs)
    launch()
    return (out, *rest) if rest else out


def autotune_gemm(a, b, candidates=None, iters=20, verbose=True, **kwargs):
    """Time candidate configs for these shapes.

    The sm_100a kernels have a single tiling, so the default candidate list has one entry; the function exists so
    that callers of the reference's ``autotune_gemm`` keep working.

    Returns:
        ``(best_config, results)``, where ``results`` is a list of ``(config, milliseconds or error string)``.
    """
    require("gemm", a)
    candidates = candidates or [{}]
    return time_candidates(candidates, lambda cfg: make_gemm(a, b, **cfg, **kwargs)[0], iters, verbose, "gemm")
