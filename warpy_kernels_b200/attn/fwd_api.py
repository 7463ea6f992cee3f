"""Attention forward host API with the reference's call surface (``warpy_kernels/attn/fwd_api.py:141-548``).

Validation, defaults, output layout and return values follow the reference; the SM80-SM120 tuning knobs are
accepted and ignored because the sm_100a kernel has one fixed configuration (128 queries per CTA, 128-key tiles,
TMA loads, dedicated load / MMA / softmax warps).
"""

import ctypes
import math

import torch

from .. import _lib
from ..arch import require
from ..utils import autotune, cached_tensor, check_descale, round_up, tune_key, tune_lookup

BM = 128


class _FwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p), ("pmax", ctypes.c_void_p),
        ("q_descale", ctypes.c_void_p), ("k_descale", ctypes.c_void_p), ("v_descale", ctypes.c_void_p),
        ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3), ("v_strides", ctypes.c_int64 * 3),
        ("out_strides", ctypes.c_int64 * 3), ("lse_strides", ctypes.c_int64 * 2),
        ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32), ("Nq", ctypes.c_int32),
        ("Nk", ctypes.c_int32), ("d", ctypes.c_int32),
        ("causal", ctypes.c_int32), ("write_lse", ctypes.c_int32), ("lse_natural", ctypes.c_int32),
        ("seqused_k", ctypes.c_void_p), ("softmax_scale", ctypes.c_float), ("ctas_per_sm", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
    ]


_flag_buffers = {}


def _block_flags(dev, nbytes):
    """Zeroed flag scratch of the forward for the current stream of ``dev``, at least ``nbytes`` long.

    The kernels mark query blocks whose scores outgrow the range of their fixed row reference; the library
    recomputes those and hands the buffer back all zero, so calls that follow one another on a stream can share it.
    """
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    buf = _flag_buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _flag_buffers[key] = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=dev)
    return buf


def _kernel_view(x):
    """Zero-copy when TMA can address ``x`` (last stride 1, 16-byte aligned base and strides); else a compact copy.

    The reference makes the same decision in ``_kernel_view`` (``attn/fwd_api.py:129-138``); rows need no padding here
    because TMA zero-fills past the end of the sequence.
    """
    direct = x.stride(3) == 1 and x.data_ptr() % 16 == 0 and all(st % 16 == 0 for st in x.stride()[:3])
    return x if direct else x.contiguous()


def _check_qkv(q, k, v):
    if not (q.dtype == k.dtype == v.dtype and q.dtype in (torch.float8_e4m3fn, torch.bfloat16)):
        raise ValueError("q, k and v must all be torch.float8_e4m3fn or all torch.bfloat16")


def _check_shapes(q, k, v):
    B, Hq, Nq, d = q.shape
    Hkv = k.shape[1]
    if k.dim() != 4 or v.shape != k.shape or k.shape[0] != B or k.shape[3] != d or d not in (64, 128) or Hq % Hkv:
        raise ValueError(
            "need q [B, Hq, Nq, d] and k, v [B, Hkv, Nk, d] with d 64 or 128 and Hq a multiple of Hkv, "
            f"got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}"
        )


def make_attn_fwd(
    q,
    k,
    v,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    causal=False,
    softmax_scale=None,
    num_stages=None,
    pipelined=None,
    block_n=None,
    block_m=None,
    warp_rows=None,
    ctas_per_sm=None,
    tile_local=True,
    lpt=None,
    tma=None,
    out=None,
    return_lse=True,
    seqused_k=None,
    lse_natural=False,
    warp_spec=None,
    split_kv=None,
):
    """Prepare an attention forward launch.

    ``launch()`` may not see later in-place changes to the inputs. Call ``make_attn_fwd`` again for new values.

    Args:
        q: ``[B, Hq, Nq, d]`` ``torch.float8_e4m3fn`` or bf16, ``d`` 64 or 128. Any strides work if the last one is 1, such as a
            transposed ``[B, N, H, d]`` tensor. Inputs are copied if a stride or the base address is not a multiple
            of 16 bytes.
        k: ``[B, Hkv, Nk, d]``, same dtype and stride rules. ``Hq`` must be a multiple of ``Hkv``.
        v: Same shape and dtype as ``k``.
        q_descale: ``[B, Hkv]`` float32 dequantization scale, or ``None`` for 1.
        k_descale: Same as ``q_descale``, for ``k``.
        v_descale: Same as ``q_descale``, for ``v``.
        causal: Whether to apply a bottom-right aligned causal mask.
        softmax_scale: Scale on the logits, positive. Defaults to ``1 / sqrt(d)``.
        ctas_per_sm: FP8 inputs: 2 runs the kernel with two CTAs per SM and 64-key tiles, 1 the one with a single
            CTA per SM, 128-key rounds and four softmax groups, which is the faster one on long sequences. ``None``
            takes the tuned value for the shape (``autotune_attn_fwd``), else 1 from 2048 keys on and 2 below.
        num_stages, pipelined, block_n, block_m, warp_rows, tile_local, lpt, tma, warp_spec, split_kv:
            Other tuning options of the reference's SM80-SM120 kernels; accepted and ignored.
        out: Output buffer, ``[B, Hq, Nq, d]`` bf16 with last stride 1 and even other strides. ``None`` allocates one
            with the memory layout of ``q``.
        return_lse: Whether to compute ``lse`` and ``pmax``. The backward pass needs them.
        seqused_k: ``[B]`` int32 number of keys each batch item attends to, at most ``Nk``. Causal masking is aligned
            to this length.
        lse_natural: Whether ``lse`` is the natural-log log-sum-exp instead of base 2.

    Returns:
        ``(launch, out, lse, pmax)``. ``out`` is ``[B, Hq, Nq, d]`` bf16, ``lse`` is the ``[B, Hq, Nq]`` base-2
        log-sum-exp of the scaled logits (``+inf`` for rows with no visible key), ``pmax`` the largest probability
        per row. ``lse`` and ``pmax`` are ``None`` if ``return_lse`` is false.

    Raises:
        ValueError: If ``q``, ``k`` or ``v`` has the wrong dtype or shape, a descale is not ``[B, Hkv]`` or is given
            for bf16 inputs, ``out`` has the wrong shape, dtype or strides, or ``seqused_k`` is not an int32 CUDA
            tensor of shape ``[B]``.
        NotImplementedError: If the GPU does not support the dtype of ``q``.
    """
    _check_qkv(q, k, v)
    bf16 = q.dtype == torch.bfloat16
    require("attn_fwd" if bf16 else "attn_fwd_fp8", q)
    if bf16 and not (q_descale is None and k_descale is None and v_descale is None):
        raise ValueError("descales apply to float8_e4m3fn inputs only")
    _check_shapes(q, k, v)
    B, Hq, Nq, d = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    for x, name in ((q_descale, "q_descale"), (k_descale, "k_descale"), (v_descale, "v_descale")):
        check_descale(x, B, Hkv, name)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    if not softmax_scale > 0:
        raise ValueError("softmax_scale must be positive")
    dev = q.device
    if bf16:
        dq_ = dk_ = dv_ = None
    else:
        ones = cached_tensor(("ones", dev, B, Hkv), lambda: torch.ones(B, Hkv, dtype=torch.float32, device=dev))
        dq_, dk_, dv_ = [(x if x is not None else ones).float().contiguous() for x in (q_descale, k_descale, v_descale)]

    qv, kv, vv = (_kernel_view(x) for x in (q, k, v))  # head dimension 64 and 128 both run natively
    if out is None:
        out = torch.empty_like(q, dtype=torch.bfloat16)
    elif (
        out.shape != q.shape
        or out.dtype != torch.bfloat16
        or out.device != dev
        or out.stride(3) != 1
        or any(st % 2 for st in out.stride()[:3])
        or out.data_ptr() % 4
    ):
        raise ValueError("out must be a bf16 tensor shaped like q, with last stride 1 and even other strides")
    # the kernel stores 16-byte vectors; an output it cannot address that way is filled through a staging copy
    out_direct = out.stride(3) == 1 and out.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in out.stride()[:3])
    out_k = out if out_direct else torch.empty(B, Hq, Nq, d, dtype=torch.bfloat16, device=dev)
    if seqused_k is not None and (
        seqused_k.shape != (B,) or seqused_k.dtype != torch.int32 or seqused_k.device != dev
    ):
        raise ValueError("seqused_k must be an int32 CUDA tensor of shape [B]")
    seq = seqused_k.contiguous() if seqused_k is not None else None
    nq_pad = round_up(Nq, BM)
    if return_lse:
        lse = torch.empty(B, Hq, nq_pad, dtype=torch.float32, device=dev)
        pmax = torch.empty(B, Hq, nq_pad, dtype=torch.float32, device=dev)
    else:
        lse = pmax = None

    args = _FwdArgs()
    args.q, args.k, args.v, args.out = qv.data_ptr(), kv.data_ptr(), vv.data_ptr(), out_k.data_ptr()
    args.lse = lse.data_ptr() if return_lse else None
    args.pmax = pmax.data_ptr() if return_lse else None
    if not bf16:
        args.q_descale, args.k_descale, args.v_descale = dq_.data_ptr(), dk_.data_ptr(), dv_.data_ptr()
    args.q_strides = (ctypes.c_int64 * 3)(*qv.stride()[:3])
    args.k_strides = (ctypes.c_int64 * 3)(*kv.stride()[:3])
    args.v_strides = (ctypes.c_int64 * 3)(*vv.stride()[:3])
    args.out_strides = (ctypes.c_int64 * 3)(*out_k.stride()[:3])
    args.lse_strides = (ctypes.c_int64 * 2)(Hq * nq_pad, nq_pad)
    args.B, args.Hq, args.Hkv, args.Nq, args.Nk, args.d = B, Hq, Hkv, Nq, Nk, d
    args.causal, args.write_lse, args.lse_natural = int(bool(causal)), int(bool(return_lse)), int(bool(lse_natural))
    args.seqused_k = seq.data_ptr() if seq is not None else None
    args.softmax_scale = float(softmax_scale)
    if ctas_per_sm is None and not bf16:
        tuned = tune_lookup(tune_key("fwd", d, causal, Nq, Nk, Hq // Hkv))
        ctas_per_sm = (tuned or {}).get("ctas_per_sm")
    if ctas_per_sm not in (None, 1, 2):
        raise ValueError("ctas_per_sm must be 1 or 2")
    args.ctas_per_sm = int(ctas_per_sm or 0)
    # the launch closure owns everything the argument block points at, outputs included: a caller may keep the
    # closure and drop the tensors it was handed
    keep = (qv, kv, vv, dq_, dk_, dv_, seq, out_k, out, lse, pmax)
    lib = _lib.lib()
    entry = lib.wk_attn_fwd_bf16 if bf16 else lib.wk_attn_fwd_fp8
    args.workspace_bytes = lib.wk_attn_fwd_workspace_bytes(B, Hq, Nq)

    def launch():
        with torch.cuda.device(dev):
            args.workspace = _block_flags(dev, args.workspace_bytes).data_ptr()
            code = entry(ctypes.byref(args), _lib.stream_ptr(dev))
        _lib.check(code, "attn_fwd")
        if not out_direct:
            out.copy_(out_k)
        return keep

    if return_lse:
        return launch, out, lse[:, :, :Nq], pmax[:, :, :Nq]
    return launch, out, None, None


def attn_fwd(q, k, v, q_descale=None, k_descale=None, v_descale=None, causal=False, softmax_scale=None, **config):
    """Run the attention forward kernel; arguments as in ``make_attn_fwd``.

    Returns:
        ``(out, lse, pmax)``.
    """
    launch, out, lse, pmax = make_attn_fwd(q, k, v, q_descale, k_descale, v_descale, causal, softmax_scale, **config)
    launch()
    return out, lse, pmax


def autotune_attn_fwd(q, k, v, candidates=None, iters=20, verbose=True, **kwargs):
    """Time candidate configs and store the fastest in the tune cache, as the reference's tuner does.

    The FP8 forward has two kernels to choose from (``ctas_per_sm`` 1 and 2, the default candidates); ``make_attn_fwd``
    looks the winner up when ``ctas_per_sm`` is not given. The cache entry keeps the reference's key format (``fwd`` /
    ``fwd_bf16``, head dimension, mask, length buckets, GQA ratio, ``sm100``).

    Returns:
        ``(best_config, results)``.
    """
    _check_qkv(q, k, v)
    bf16 = q.dtype == torch.bfloat16
    require("attn_fwd" if bf16 else "attn_fwd_fp8", q)
    _check_shapes(q, k, v)
    return autotune(
        "fwd_bf16" if bf16 else "fwd", q.shape[3], bool(kwargs.get("causal", False)), q.shape[2], k.shape[2],
        q.shape[1] // k.shape[1], candidates or ([{}] if bf16 else [{"ctas_per_sm": 2}, {"ctas_per_sm": 1}]),
        lambda cfg: make_attn_fwd(q, k, v, **cfg, **kwargs)[0], iters, verbose,
    )
