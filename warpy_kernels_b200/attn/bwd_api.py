"""Attention backward host API (reference: ``warpy_kernels/attn/bwd_api.py:26-476``)."""


def make_attn_bwd(*args, **kwargs):
    raise NotImplementedError("warpy_kernels for SM100: the attention backward is being built")


def attn_bwd(*args, **kwargs):
    raise NotImplementedError("warpy_kernels for SM100: the attention backward is being built")


def autotune_attn_bwd(*args, **kwargs):
    raise NotImplementedError("warpy_kernels for SM100: the attention backward is being built")
