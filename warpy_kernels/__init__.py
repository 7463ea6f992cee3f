"""Drop-in alias: ``from warpy_kernels import attn_fwd, attn_bwd, gemm`` resolves to the B200 build.

Sub-modules ``warpy_kernels.attn``, ``warpy_kernels.gemm``, ``warpy_kernels.utils`` and ``warpy_kernels.arch`` are
the same module objects as their ``warpy_kernels_b200`` counterparts.
"""

import sys

import warpy_kernels_b200 as _impl
import warpy_kernels_b200.gemm.api  # noqa: F401  (registers the sub-package in sys.modules)
from warpy_kernels_b200 import arch, attn, interface, quant, utils
from warpy_kernels_b200 import (
    attn_bwd,
    attn_fwd,
    autotune_gemm,
    device_arch,
    gemm,
    make_gemm,
    quantize_mx,
    supports,
)

# ``gemm`` the attribute is the function (as in the reference); the sub-package is reached through sys.modules
for _name in ("arch", "attn", "gemm", "gemm.api", "interface", "quant", "utils"):
    sys.modules[f"{__name__}.{_name}"] = sys.modules[f"warpy_kernels_b200.{_name}"]

__all__ = list(_impl.__all__)
