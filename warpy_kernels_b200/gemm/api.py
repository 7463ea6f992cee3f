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
from ..utils import gemm_tune_key, time_candidates, tune_lookup, tune_store

_TYPES = {torch.bfloat16: "bf16", torch.float16: "f16"}
BM = 128


_EPILOGUE_FIELDS = [
    ("scale_a_rows", ctypes.c_int32), ("scale_b_cols", ctypes.c_int32), ("accum", ctypes.c_int32),
    ("act", ctypes.c_int32),
]


class _MxArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("a_scale_mx", ctypes.c_void_p),
        ("b_scale_mx", ctypes.c_void_p), ("scale_a", ctypes.c_void_p), ("scale_b", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("q_mx", ctypes.c_void_p), ("s_mx", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
        *_EPILOGUE_FIELDS, ("out_f16", ctypes.c_int32),
        ("pre_out", ctypes.c_void_p), ("pre_in", ctypes.c_void_p), ("cta_pair", ctypes.c_int32),
        ("a_scale_tiled", ctypes.c_int32), ("b_scale_tiled", ctypes.c_int32), ("group_m", ctypes.c_int32),
    ]


class _Gemm16Args(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("f16", ctypes.c_int32),
        ("scale_a", ctypes.c_void_p), ("scale_b", ctypes.c_void_p),
        *_EPILOGUE_FIELDS,
        ("pre_out", ctypes.c_void_p), ("pre_in", ctypes.c_void_p),
        ("q_mx", ctypes.c_void_p), ("s_mx", ctypes.c_void_p),
        ("a_trans", ctypes.c_int32), ("b_trans", ctypes.c_int32), ("cta_pair", ctypes.c_int32),
        ("group_m", ctypes.c_int32),
    ]


_ACT = {"": 0, "gelu": 1, "dgelu": 2}


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
    group_m=None,
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
    cta_pair=None,
):
    """Prepare ``out = a @ b.T * scale_a * scale_b``.

    Args:
        a: ``[M, K]`` bf16, fp16 or ``torch.float8_e4m3fn``, contiguous. ``[K, M]`` if ``a_trans``.
        b: ``[N, K]`` with the dtype of ``a``, contiguous. ``[K, N]`` if ``b_trans``, so the product is ``a @ b``.
        out: Optional contiguous ``[M, N]`` bf16 output, 16-byte aligned. Allocated if ``None``.
        bk: K elements per pipeline stage in the reference; here only the divisibility rule ``K % bk == 0`` is
            kept. Defaults to 64 for bf16 and 128 for fp8.
        group_m: Output tiles are visited in groups of ``group_m`` tile rows that sweep all tile columns, as in the
            reference; it decides which operand rows the CTAs that run together share in L2. ``None`` takes the tuned
            value for the shape (``autotune_gemm``), else 8. The result does not depend on it.
        stages, min_blocks, frag_pipe, tma, warp_spec, persistent, setmaxnreg: Accepted for
            compatibility and ignored: the sm_100a kernels are always TMA-fed, warp-specialised and persistent.
        bn: Output columns per CTA in the reference, 128 or 256; ``N`` must be a multiple of it.
        scale_a: Float32 CUDA tensor that scales ``a``: one element (used for fp8 inputs only), or ``M`` elements
            to scale each output row (any input dtype), applied before ``accum`` and ``act``.
        scale_b: As ``scale_a``, for ``b``, with ``N`` elements to scale each output column.
        out_dtype: Output dtype when ``out`` is ``None`` and the inputs are fp8: bf16 or fp16.
        act: ``"gelu"`` to apply the exact erf GELU to the scaled product before storing it in ``out``, or
            ``"dgelu"`` to multiply the scaled product by the GELU derivative at ``pre``.
        store_pre: Whether to also store the product before the activation. Needs ``act="gelu"``.
        pre: The pre-activation values the forward stored, ``[M, N]`` with the dtype of ``out``. Needed for
            ``act="dgelu"``.
        a_trans: Whether ``a`` is stored ``[K, M]``. Needs bf16 or fp16 inputs.
        b_trans: Whether ``b`` is stored ``[K, N]``. Same limits as ``a_trans``.
        accum: Whether to add the scaled product to the values ``out`` already holds, before the activation.
        a_scale_mx: ``[M, K / 32]`` uint8 ue8m0 scales of ``a``, one per row and block of 32 along K, as
            ``out_mx`` writes them. Needs fp8 inputs.
        out_mx: Whether to also write the result as MXFP8: e4m3 values ``[M, N]`` and ``[M, N / 32]`` uint8 ue8m0
            scales computed from the fp32 values before they are rounded to bf16.
        cta_pair: Not in the reference. ``True`` runs the CTA-pair kernel (``tcgen05`` ``cta_group::2``: two SMs
            share a 256 x 256 tile). ``False`` never uses pairs. ``None`` leaves the choice to the library: for 16-bit inputs pairs when the
            256 x 256 tiles fill the GPU about as well as 128 x 256 ones, for fp8 inputs single CTAs. The results
            are bit-identical either way.
        b_scale_mx: ``[N, K / 32]`` uint8 ue8m0 scales of ``b``. Not in the reference (which scales only ``a``);
            ``None`` gives the reference's behaviour. ``b`` plays the weights: its scales are re-tiled into the
            kernels' layout once, when the launch is prepared, so ``launch()`` does not see later in-place changes
            to this tensor (those of ``a_scale_mx`` are re-read at every launch).

    Returns:
        ``(launch, out)``, or ``(launch, out, pre)`` if ``act="gelu"``, where ``pre`` is ``None`` unless
        ``store_pre`` is set. With ``out_mx``, the e4m3 values and their scales follow. ``launch()`` runs the kernel
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
    if act not in _ACT:
        raise ValueError(f"act must be '', 'gelu' or 'dgelu', got {act!r}")
    if (a_trans or b_trans) and fp8:
        raise ValueError("transposed operands need bf16 or fp16 inputs")
    if store_pre and act != "gelu":
        raise ValueError("store_pre needs act='gelu'")
    odt = out_dtype if fp8 and out is None else out.dtype if out is not None else a.dtype
    if odt not in _TYPES:
        raise ValueError("the output must be bf16 or fp16")
    if not fp8 and odt != a.dtype:
        raise ValueError(f"out must have the dtype of a and b for 16-bit inputs, got {odt} and {a.dtype}")
    bk = bk or (128 if fp8 else 64)
    if bn not in (128, 256):
        raise ValueError("bn must be 128 or 256")
    m, k = a.shape[::-1] if a_trans else a.shape
    n, kb = b.shape[::-1] if b_trans else b.shape
    if kb != k:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if not (a.is_contiguous() and b.is_contiguous()):
        raise ValueError("a and b must be contiguous")
    if m % BM or n % bn or k % bk or k % (128 if fp8 else 64):
        raise ValueError(f"M must be a multiple of 128, N of {bn} and K of {bk}, got {m}, {n}, {k}")
    if accum and out is None:
        raise ValueError("accum needs an out tensor holding the addend")
    if out is None:
        out = torch.empty(m, n, dtype=odt, device=a.device)
    elif out.shape != (m, n) or not out.is_contiguous() or out.data_ptr() % 16:
        raise ValueError("out must be a contiguous [M, N] tensor aligned to 16 bytes")
    if act == "dgelu" and (
        pre is None or pre.shape != out.shape or pre.dtype != out.dtype or not pre.is_contiguous()
    ):
        raise ValueError("act='dgelu' needs a contiguous pre shaped and typed like out")
    pre_out = torch.empty_like(out) if store_pre else None
    pre_in = pre if act == "dgelu" else None
    for name, s, size in (("scale_a", scale_a, m), ("scale_b", scale_b, n)):
        if s is None:
            continue
        if (
            s.dtype != torch.float32
            or not s.is_cuda
            or s.numel() not in (1, size)
            or (s.numel() > 1 and (not s.is_contiguous() or s.data_ptr() % 8))
        ):
            raise ValueError(
                f"{name} must be a float32 CUDA tensor of 1 or {size} elements, contiguous and 8-byte aligned"
            )
    # a one-element scale is only used for fp8 inputs (as in the reference); vectors apply to every dtype
    row_scale = scale_a is not None and scale_a.numel() > 1 and m > 1
    col_scale = scale_b is not None and scale_b.numel() > 1 and n > 1
    if not fp8:
        scale_a = scale_a if row_scale else None
        scale_b = scale_b if col_scale else None
    if col_scale and scale_b.data_ptr() % 16:
        scale_b = scale_b.clone()  # the kernel reads column scales as 16-byte vectors
    if cta_pair is None or group_m is None:
        # what autotune_gemm found fastest for this shape, if it was run; else the library's own choice
        tuned = tune_lookup(gemm_tune_key("gemm_fp8" if fp8 else "gemm", m, n, k)) or {}
        cta_pair = tuned.get("cta_pair") if cta_pair is None else cta_pair
        group_m = tuned.get("group_m") if group_m is None else group_m
    if group_m is not None and (not isinstance(group_m, int) or group_m < 1):
        raise ValueError("group_m must be a positive integer")
    _check_mx("a_scale_mx", a_scale_mx, m, k, fp8)
    _check_mx("b_scale_mx", b_scale_mx, n, k, fp8)
    q_mx = torch.empty(m, n, dtype=torch.float8_e4m3fn, device=a.device) if out_mx else None
    s_mx = torch.empty(m, n // 32, dtype=torch.uint8, device=a.device) if out_mx else None
    lib = _lib.lib()
    dev = a.device
    ptr = lambda t: t.data_ptr() if t is not None else None

    def fill_epilogue(args):
        args.scale_a, args.scale_b = ptr(scale_a), ptr(scale_b)
        args.scale_a_rows, args.scale_b_cols = int(row_scale), int(col_scale)
        args.accum, args.act = int(bool(accum)), _ACT[act]
        args.pre_out, args.pre_in = ptr(pre_out), ptr(pre_in)

    if not fp8:
        args = _Gemm16Args()
        args.q_mx, args.s_mx = ptr(q_mx), ptr(s_mx)
        args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
        args.m, args.n, args.k = m, n, k
        args.f16 = int(a.dtype == torch.float16)
        args.a_trans, args.b_trans = int(bool(a_trans)), int(bool(b_trans))
        args.cta_pair = 0 if cta_pair is None else 1 if cta_pair else 2
        args.group_m = int(group_m or 0)
        fill_epilogue(args)
        keep = (a, b, out, scale_a, scale_b, pre_out, pre_in, q_mx, s_mx)  # inputs and outputs stay alive

        def launch():
            with torch.cuda.device(dev):
                code = lib.wk_gemm_16bit(ctypes.byref(args), _lib.stream_ptr(dev))
            _lib.check(code, "gemm (16-bit)")
            return keep

    else:
        ws_bytes = lib.wk_gemm_mxfp8_workspace_bytes(m, n, k)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)  # the scales of a, re-tiled at every launch
        # b plays the weights: its scales (unit scales if none are given) are re-tiled once, here, into the layout the
        # kernels read; like every make_* closure, launch() then does not see later in-place changes to b_scale_mx
        b_tiled = torch.empty(lib.wk_mx_scales_tiled_bytes(n, k), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.wk_tile_mx_scales(ptr(b_scale_mx), n, k, b_tiled.data_ptr(), _lib.stream_ptr(dev)),
                       "gemm (fp8 scales)")
        args = _MxArgs()
        args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
        args.a_scale_mx, args.b_scale_mx = ptr(a_scale_mx), b_tiled.data_ptr()
        args.a_scale_tiled, args.b_scale_tiled = 0, 1
        args.q_mx, args.s_mx = ptr(q_mx), ptr(s_mx)
        args.workspace, args.workspace_bytes = workspace.data_ptr(), ws_bytes
        args.m, args.n, args.k = m, n, k
        args.out_f16 = int(odt == torch.float16)
        args.cta_pair = 0 if cta_pair is None else 1 if cta_pair else 2
        args.group_m = int(group_m or 0)
        fill_epilogue(args)
        keep = (a, b, out, a_scale_mx, b_tiled, scale_a, scale_b, workspace, pre_out, pre_in, q_mx, s_mx)

        def launch():
            with torch.cuda.device(dev):
                code = lib.wk_gemm_mxfp8(ctypes.byref(args), _lib.stream_ptr(dev))
            _lib.check(code, "gemm (fp8)")
            return keep

    mx = (q_mx, s_mx) if out_mx else ()
    return (launch, out, pre_out, *mx) if act == "gelu" else (launch, out, *mx)


def gemm(a, b, out=None, **kwargs):
    """Compute ``(a @ b.T) * scale_a * scale_b``; arguments as in ``make_gemm``.

    Returns:
        ``[M, N]`` in the output dtype, or ``(out, pre)`` if ``act="gelu"``. With ``out_mx``, a tuple that ends with
        the e4m3 values and their scales.
    """
    launch, out, *rest = make_gemm(a, b, out, **kwargs)
    launch()
    return (out, *rest) if kwargs.get("act") == "gelu" or kwargs.get("out_mx") else out


def candidates_for(fp8):
    """The variants ``autotune_gemm`` times: single CTAs (128 x 256 tiles) or CTA pairs (``tcgen05``
    ``cta_group::2``, 256 x 256 tiles over two SMs), each with tile groups of 8 and of 32 rows (``group_m``: few
    rows suit a narrow output, many a wide one), for 16-bit and for fp8 inputs alike.  The counterpart of the
    reference's ``candidates_for`` (``warpy_kernels/gemm/configs.py``), whose knobs tune its SM80-SM120 kernels."""
    del fp8  # the same kernels exist for both input types
    return [{"cta_pair": pair, "group_m": g} for pair in (False, True) for g in (8, 32)]


def autotune_gemm(a, b, candidates=None, iters=20, verbose=True, **kwargs):
    """Time candidate configs for these shapes and remember the fastest.

    ``make_gemm`` and ``gemm`` look the winner up (tune cache, keyed by input type and ``M, N, K``) whenever
    ``cta_pair`` is not given; without an entry the library chooses by a size rule.

    Args:
        a: As in ``make_gemm``.
        b: As in ``make_gemm``.
        candidates: Config dicts with keyword arguments of ``make_gemm``. Defaults to ``candidates_for`` the input type.
        iters: Timed launches per candidate.
        verbose: Whether to print one line per candidate.
        **kwargs: Extra keyword arguments for ``make_gemm``, such as ``scale_a``.

    Returns:
        ``(best_config, results)``, where ``results`` is a list of ``(config, milliseconds or error string)``.

    Raises:
        RuntimeError: If no candidate runs.
        NotImplementedError: If the GPU does not support the dtype of ``a``.
    """
    require("gemm", a)
    fp8 = a.dtype == torch.float8_e4m3fn
    best, results = time_candidates(
        candidates or candidates_for(fp8), lambda cfg: make_gemm(a, b, **cfg, **kwargs)[0], iters, verbose, "gemm"
    )
    m, k = a.shape[::-1] if kwargs.get("a_trans") else a.shape
    n = b.shape[1] if kwargs.get("b_trans") else b.shape[0]
    tune_store(gemm_tune_key("gemm_fp8" if fp8 else "gemm", m, n, k), best)
    return best, results
