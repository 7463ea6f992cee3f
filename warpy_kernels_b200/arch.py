"""Which GPU this build runs on and which features it has.

Same three functions and error types as the reference's ``warpy_kernels/arch.py`` (``device_arch`` ``:29-60``,
``supports`` ``:69-94``, ``require`` ``:97-116``), but the answers are not a Python table: the compiled library
says which device it accepts (``wk_device_arch``: compute capability 10.x is architecture 100) and which of the
reference's feature names it has a kernel for (``wk_query``), so the Python layer cannot drift from the kernels.
"""

import torch

from . import _lib

ARCH = 100
ARCH_NAME = "SM100"
SUPPORTED = "compute capability 10.x (SM100, B200)"

# the reference's feature vocabulary; wk_query() knows the same names
FEATURES = (
    "gemm", "gemm_gelu", "gemm_dgelu", "gemm_accum", "gemm_fp8", "gemm_mx", "gemm_mx_out",
    "attn_fwd", "attn_bwd", "attn_fwd_fp8", "attn_bwd_fp8",
)

_arch_of_index = {}


def _device_index(device):
    """CUDA device ordinal of a tensor, ``torch.device``, string, integer or ``None`` (= the current device)."""
    if isinstance(device, torch.Tensor):
        device = device.device
    if isinstance(device, int):
        return device
    if device is not None:
        index = torch.device(device).index
        if index is not None:
            return index
    return torch.cuda.current_device()


def device_arch(device=None):
    """Architecture number of a CUDA device: 100 for B200.

    Args:
        device: CUDA device, index or tensor. Defaults to the current device.

    Raises:
        NotImplementedError: If there is no usable CUDA device or the library has no kernels for it.
    """
    if not torch.cuda.is_available():
        raise NotImplementedError(f"warpy_kernels found no usable CUDA device; it runs on {SUPPORTED}")
    index = _device_index(device)
    if index not in _arch_of_index:
        answer = _lib.lib().wk_device_arch(index)
        if answer != ARCH:
            capability = torch.cuda.get_device_capability(index)
            raise NotImplementedError(
                f"this build of warpy_kernels runs on {SUPPORTED}; device {index} is compute capability "
                f"{capability[0]}.{capability[1]} ({_lib.lib().wk_error_string(answer).decode()})"
            )
        _arch_of_index[index] = answer
    return _arch_of_index[index]


def _has_kernel(feature):
    answer = _lib.lib().wk_query(feature.encode())
    if answer < 0:
        raise ValueError(f"unknown feature {feature!r}; the feature names are: {', '.join(FEATURES)}")
    return answer == 1


def supports(feature, device=None):
    """Whether ``feature`` runs on a GPU.

    Args:
        feature: One of the reference's feature names (``FEATURES``).
        device: CUDA device, index or tensor, or the architecture number 100. Other architecture numbers (the
            reference's 80, 86, 89, 120) are answered with ``False``: this build has kernels for 100 only.

    Raises:
        ValueError: If ``feature`` is not a feature name.
    """
    built = _has_kernel(feature)
    if isinstance(device, int) and device >= 50:  # an architecture number, not a device ordinal
        return built and device == ARCH
    try:
        device_arch(device)
    except NotImplementedError:
        return False
    return built


def require(feature, device):
    """Return the architecture number of ``device``; raise ``NotImplementedError`` unless ``feature`` runs there."""
    arch = device_arch(device)
    if not _has_kernel(feature):
        raise NotImplementedError(f"this build of warpy_kernels has no {feature} kernel for {ARCH_NAME}")
    return arch
