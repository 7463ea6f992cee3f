"""Capability table of the B200 build.

Mirrors ``warpy_kernels/arch.py:3-116`` of the reference (``device_arch``, ``supports``, ``require``) with one
architecture: compute capability 10.0 -> 100.  The feature names are the reference's.
"""

import torch

ARCHS = {(10, 0): 100, (10, 3): 100}
NAMES = {100: "SM100"}
SUPPORTED = "compute capability 10.0 (SM100, B200)"

# usable shared memory bytes per CTA
_SMEM_LIMIT = {100: 232448}

_FEATURES = {
    "gemm": (100,),
    "gemm_gelu": (100,),
    "gemm_dgelu": (100,),
    "gemm_accum": (100,),
    "gemm_fp8": (100,),
    "gemm_mx": (100,),
    "gemm_mx_out": (100,),
    "attn_fwd": (100,),
    "attn_bwd": (100,),
    "attn_fwd_fp8": (100,),
    "attn_bwd_fp8": (100,),
}

_device_arch = {}


def device_arch(device=None):
    """Return the architecture of a CUDA device as a number (100 for B200).

    Args:
        device: CUDA device, index or tensor. Defaults to the current device.

    Raises:
        NotImplementedError: If there is no usable CUDA device or it is not compute capability 10.x.
    """
    if not torch.cuda.is_available():
        raise NotImplementedError(f"warpy_kernels needs a usable CUDA device; supported: {SUPPORTED}")
    if isinstance(device, torch.Tensor):
        device = device.device
    if device is None:
        idx = torch.cuda.current_device()
    elif isinstance(device, int):
        idx = device
    else:
        device = torch.device(device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
    arch = _device_arch.get(idx)
    if arch is None:
        cap = torch.cuda.get_device_capability(idx)
        if cap not in ARCHS:
            raise NotImplementedError(
                f"warpy_kernels has no kernels for compute capability {cap}; supported: {SUPPORTED}"
            )
        arch = _device_arch[idx] = ARCHS[cap]
    return arch


def smem_limit(arch):
    return _SMEM_LIMIT[arch]


def supports(feature, device=None):
    """Return whether a feature runs on a GPU.

    Args:
        feature: One of the reference's feature names: ``"gemm"``, ``"gemm_gelu"``, ``"gemm_dgelu"``,
            ``"gemm_accum"``, ``"gemm_fp8"``, ``"gemm_mx"``, ``"gemm_mx_out"``, ``"attn_fwd"``, ``"attn_bwd"``,
            ``"attn_fwd_fp8"``, ``"attn_bwd_fp8"``.
        device: CUDA device, index or tensor, or the architecture number 100.

    Raises:
        ValueError: If ``feature`` is not one of the names above.
    """
    if feature not in _FEATURES:
        raise ValueError(f"unknown feature {feature!r}; known: {', '.join(_FEATURES)}")
    if isinstance(device, int) and device in NAMES:
        arch = device
    else:
        try:
            arch = device_arch(device)
        except NotImplementedError:
            return False
    return arch in _FEATURES[feature]


def require(feature, device):
    """Raise ``NotImplementedError`` unless ``feature`` runs on ``device``; return the architecture number."""
    arch = device_arch(device)
    if arch not in _FEATURES[feature]:
        archs = ", ".join(NAMES[a] for a in _FEATURES[feature]) or "no architecture of this build"
        raise NotImplementedError(f"warpy_kernels has no {feature} for {NAMES[arch]}; supported on: {archs}")
    return arch
