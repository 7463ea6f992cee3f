"""Attention backward host API with the reference's call surface (``warpy_kernels/attn/bwd_api.py:26-476``).

Validation and return values follow the reference.  Its tuning options (``num_stages, dq_bulk, dq_interleave,
block_m, kb_major, one_barrier``) are accepted and ignored; ``deterministic`` is always satisfied (this backward has
no atomics, so two runs are bit-identical whatever the flag says).
"""

import ctypes
import math

import torch

from .. import _lib
from ..arch import require
from ..utils import autotune, cached_tensor, check_descale
from .fwd_api import _check_qkv, _check_shapes, _kernel_view


class _BwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("dout", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("q_descale", ctypes.c_void_p), ("k_descale", ctypes.c_void_p), ("v_descale", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
        ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3), ("v_strides", ctypes.c_int64 * 3),
        ("out_strides", ctypes.c_int64 * 3), ("dout_strides", ctypes.c_int64 * 3), ("lse_strides", ctypes.c_int64 * 2),
        ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32), ("Nq", ctypes.c_int32),
        ("Nk", ctypes.c_int32), ("d", ctypes.c_int32), ("causal", ctypes.c_int32), ("softmax_scale", ctypes.c_float),
    ]


def _bf16_view(x):
    """bf16 tensor the prep kernel can address: last stride 1, other strides multiples of 4 elements, 8-byte base."""
    x = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    ok = x.stride(3) == 1 and x.data_ptr() % 8 == 0 and all(st % 4 == 0 for st in x.stride()[:3])
    return x if ok else x.contiguous()


def make_attn_bwd(
    q,
    k,
    v,
    out,
    lse,
    pmax,
    dout,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    causal=False,
    softmax_scale=None,
    num_stages=None,
    dq_bulk=None,
    dq_interleave=None,
    deterministic=False,
    block_m=None,
    kb_major=None,
    seqused_k=None,
    one_barrier=None,
):
    """Prepare the attention backward.

    ``launch()`` may not see later in-place changes to the inputs. Call ``make_attn_bwd`` again for new values.

    Args:
        q: The forward's ``q``, ``[B, Hq, Nq, d]`` ``torch.float8_e4m3fn``.
        k: The forward's ``k``, ``[B, Hkv, Nk, d]``, same dtype as ``q``.
        v: The forward's ``v``, ``[B, Hkv, Nk, d]``, same dtype as ``q``.
        out: The forward's ``out`` (bf16).
        lse: The forward's base-2 ``lse``.
        pmax: The forward's largest probability per row. Accepted for compatibility; this backward scales its e4m3
            operands from the values themselves and does not need it.
        dout: Gradient of ``out``, ``[B, Hq, Nq, d]``. Read as bf16; other dtypes are converted first.
        q_descale: ``[B, Hkv]`` float32 dequantization scale, or ``None`` for 1.
        k_descale: Same as ``q_descale``, for ``k``.
        v_descale: Same as ``q_descale``, for ``v``.
        causal: The ``causal`` given to the forward.
        softmax_scale: The ``softmax_scale`` given to the forward. Defaults to ``1 / sqrt(d)``.
        num_stages, dq_bulk, dq_interleave, deterministic, block_m, kb_major, one_barrier: Options of the reference's
            kernels; accepted and ignored.
        seqused_k: Must be ``None``, as in the reference.

    Returns:
        ``(launch, finish)``. ``launch()`` runs the kernels; ``finish()`` returns ``(dq, dk, dv)`` in bf16, shaped like
        ``q``, ``k`` and ``v``: gradients with respect to the dequantized ``q``, ``k`` and ``v``.

    Raises:
        NotImplementedError: If ``seqused_k`` is given, or the GPU or head dimension is unsupported.
        ValueError: If a tensor has the wrong dtype or shape, or a descale is not ``[B, Hkv]``.
    """
    if seqused_k is not None:
        raise NotImplementedError(
            "the backward does not support seqused_k; it would compute gradients over all Nk keys"
        )
    _check_qkv(q, k, v)
    bf16 = q.dtype == torch.bfloat16
    require("attn_bwd" if bf16 else "attn_bwd_fp8", q)
    if bf16 and not (q_descale is None and k_descale is None and v_descale is None):
        raise ValueError("descales apply to float8_e4m3fn inputs only")
    _check_shapes(q, k, v)
    B, Hq, Nq, d = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    if out.shape != q.shape or dout.shape != q.shape:
        raise ValueError(
            f"out and dout must be shaped like q {tuple(q.shape)}, got {tuple(out.shape)} and {tuple(dout.shape)}"
        )
    if lse.shape != (B, Hq, Nq) or pmax.shape != (B, Hq, Nq):
        raise ValueError(
            f"lse and pmax must be [B, Hq, Nq] = [{B}, {Hq}, {Nq}], got {tuple(lse.shape)} and {tuple(pmax.shape)}"
        )
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
    qv, kv, vv = _kernel_view(q), _kernel_view(k), _kernel_view(v)  # head dimension 64 and 128 both run natively
    ov = _bf16_view(out)
    # the bf16 kernels read dout through TMA like q: 16-byte aligned base and strides
    dov = _kernel_view(dout if dout.dtype == torch.bfloat16 else dout.to(torch.bfloat16)) if bf16 else _bf16_view(dout)
    lsev = lse.float()
    if lsev.stride(2) != 1:
        lsev = lsev.contiguous()
    dq = torch.empty(B, Hq, Nq, d, dtype=torch.bfloat16, device=dev)
    dk = torch.empty(B, Hkv, Nk, d, dtype=torch.bfloat16, device=dev)
    dv = torch.empty(B, Hkv, Nk, d, dtype=torch.bfloat16, device=dev)
    lib = _lib.lib()
    ws_bytes = (lib.wk_attn_bwd_bf16_workspace_bytes if bf16 else lib.wk_attn_bwd_fp8_workspace_bytes)(B, Hq, Nq)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)

    args = _BwdArgs()
    args.q, args.k, args.v = qv.data_ptr(), kv.data_ptr(), vv.data_ptr()
    args.out, args.dout, args.lse = ov.data_ptr(), dov.data_ptr(), lsev.data_ptr()
    if not bf16:
        args.q_descale, args.k_descale, args.v_descale = dq_.data_ptr(), dk_.data_ptr(), dv_.data_ptr()
    args.dq, args.dk, args.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    args.workspace, args.workspace_bytes = workspace.data_ptr(), ws_bytes
    args.q_strides = (ctypes.c_int64 * 3)(*qv.stride()[:3])
    args.k_strides = (ctypes.c_int64 * 3)(*kv.stride()[:3])
    args.v_strides = (ctypes.c_int64 * 3)(*vv.stride()[:3])
    args.out_strides = (ctypes.c_int64 * 3)(*ov.stride()[:3])
    args.dout_strides = (ctypes.c_int64 * 3)(*dov.stride()[:3])
    args.lse_strides = (ctypes.c_int64 * 2)(*lsev.stride()[:2])
    args.B, args.Hq, args.Hkv, args.Nq, args.Nk, args.d = B, Hq, Hkv, Nq, Nk, d
    args.causal, args.softmax_scale = int(bool(causal)), float(softmax_scale)
    keep = (qv, kv, vv, ov, dov, lsev, dq_, dk_, dv_, workspace, dq, dk, dv)  # inputs, scratch and outputs

    entry = lib.wk_attn_bwd_bf16 if bf16 else lib.wk_attn_bwd_fp8

    def launch():
        with torch.cuda.device(dev):
            code = entry(ctypes.byref(args), _lib.stream_ptr(dev))
        _lib.check(code, "attn_bwd")
        return keep

    def finish():
        return dq, dk, dv

    return launch, finish


def attn_bwd(
    q, k, v, out, lse, pmax, dout, q_descale=None, k_descale=None, v_descale=None, causal=False,
    softmax_scale=None, **config,
):
    """Run the attention backward; arguments as in ``make_attn_bwd``.

    Returns:
        ``(dq, dk, dv)`` in bf16.
    """
    launch, finish = make_attn_bwd(
        q, k, v, out, lse, pmax, dout, q_descale, k_descale, v_descale, causal, softmax_scale, **config
    )
    launch()
    return finish()


def autotune_attn_bwd(q, k, v, out, lse, pmax, dout, candidates=None, iters=20, verbose=True, **kwargs):
    """Time candidate configs and store the fastest in the tune cache, as the reference's tuner does.

    The SM100 kernels have a single configuration, so the default candidate list is ``[{}]``.

    Returns:
        ``(best_config, results)``.
    """
    _check_qkv(q, k, v)
    bf16 = q.dtype == torch.bfloat16
    require("attn_bwd" if bf16 else "attn_bwd_fp8", q)
    _check_shapes(q, k, v)
    return autotune(
        "bwd_bf16" if bf16 else "bwd", q.shape[3], bool(kwargs.get("causal", False)), q.shape[2], k.shape[2],
        q.shape[1] // k.shape[1], candidates or [{}],
        lambda cfg: make_attn_bwd(q, k, v, out, lse, pmax, dout, **cfg, **kwargs)[0], iters, verbose,
    )
