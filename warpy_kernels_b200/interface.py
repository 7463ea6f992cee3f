"""Public entry points, same names and signatures as ``warpy_kernels/interface.py:20-111`` of the reference."""

import torch

from .arch import require
from .gemm.api import autotune_gemm, gemm, make_gemm

__all__ = ["attn_bwd", "attn_fwd", "autotune_gemm", "gemm", "make_gemm"]


_ATTN_DTYPES = {torch.float8_e4m3fn: "_fp8", torch.bfloat16: ""}


def _check(q, what, feature):
    """Gate an attention entry point on the dtype of ``q`` and on the GPU it lives on."""
    suffix = _ATTN_DTYPES.get(q.dtype)
    if suffix is None:
        accepted = ", ".join(str(t).split(".")[-1] for t in _ATTN_DTYPES)
        raise NotImplementedError(f"the attention {what} takes {accepted} inputs, not {q.dtype}")
    require(feature + suffix, q)


def attn_fwd(q, k, v, q_descale=None, k_descale=None, v_descale=None, causal=False, softmax_scale=None, **config):
    """Run the FP8 attention forward kernel.

    Args:
        q: ``[B, Hq, Nq, d]`` ``torch.float8_e4m3fn``.
        k: ``[B, Hkv, Nk, d]``, same dtype.
        v: ``[B, Hkv, Nk, d]``, same dtype.
        q_descale: ``[B, Hkv]`` float32 dequantization scale, or ``None`` for 1.
        k_descale: Same, for ``k``.
        v_descale: Same, for ``v``.
        causal: Whether to apply a bottom-right aligned causal mask.
        softmax_scale: Scale on the logits. Defaults to ``1 / sqrt(d)``.
        **config: See ``warpy_kernels.attn.make_attn_fwd``.

    Returns:
        ``(out, lse, pmax)``: ``out`` ``[B, Hq, Nq, d]`` bf16, ``lse`` the ``[B, Hq, Nq]`` base-2 log-sum-exp, ``pmax``
        the largest probability per row. Pass all three to ``attn_bwd``.

    Raises:
        NotImplementedError: If there is no kernel for the dtype or the GPU.
    """
    from .attn import attn_fwd as _attn_fwd

    _check(q, "forward", "attn_fwd")
    return _attn_fwd(q, k, v, q_descale, k_descale, v_descale, causal, softmax_scale, **config)


def attn_bwd(
    q, k, v, out, lse, pmax, dout, q_descale=None, k_descale=None, v_descale=None, causal=False,
    softmax_scale=None, **config,
):
    """Run the FP8 attention backward kernel for the outputs of ``attn_fwd``.

    Returns:
        ``(dq, dk, dv)`` in bf16: gradients with respect to the dequantized ``q``, ``k`` and ``v``.

    Raises:
        NotImplementedError: If there is no kernel for the dtype or the GPU.
    """
    from .attn import attn_bwd as _attn_bwd

    _check(q, "backward", "attn_bwd")
    return _attn_bwd(
        q, k, v, out, lse, pmax, dout, q_descale, k_descale, v_descale, causal, softmax_scale, **config
    )
