from .bwd_api import attn_bwd, autotune_attn_bwd, make_attn_bwd
from .fwd_api import attn_fwd, autotune_attn_fwd, make_attn_fwd

__all__ = [
    "attn_bwd",
    "attn_fwd",
    "autotune_attn_bwd",
    "autotune_attn_fwd",
    "make_attn_bwd",
    "make_attn_fwd",
]
