"""GPU: attention forward on rows whose late keys lie far above the first ones.

The tensor-core kernels fix one reference exponent per query row from the row's first 64 keys and can represent
scores up to 2^100 (69 nats) above it; the reference has no such limit because its reference moves with every key
tile (``warpy_kernels/attn/fwd_base.py:337-360``).  Query blocks that leave the range are recomputed by the
library (two-pass fp32 kernel) when the call is given its flag workspace, as the Python wrappers always do.  These
tests put peaks of 120 to 400 nats behind the first tile and apply the usual gates against the oracle, then check
the raw C-ABI behaviour without a workspace: the status word says ``WK_ERR_RANGE`` (nothing faults).
"""

import ctypes
import math

import pytest
import torch

from oracle import reference_math as R
from tests.helpers import fwd_errors

pytestmark = pytest.mark.gpu

WK_ERR_RANGE = 110


def late_peak_qkv(B, Hq, Hkv, Nq, Nk, d, peaks, seed=0, device="cuda"):
    """Near-uniform logits except for keys ``peaks = [(index, gap_nats), ...]`` that rise ``gap_nats`` above the rest
    (the recipe of the reference's long-tail case, ``tests/fixtures.py:81-88``, with the peak moved off key 0)."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = 1.0 + 0.1 * torch.randn(B, Hq, Nq, d, device=device, generator=g)
    k = 0.01 * torch.randn(B, Hkv, Nk, d, device=device, generator=g)
    for index, gap in peaks:
        k[:, :, index, :] = gap / math.sqrt(d)
    v = torch.randn(B, Hkv, Nk, d, device=device, generator=g)
    return q, k, v


def gates(errs):
    assert errs["out"] <= 6e-2 and errs["cos"] >= 0.999 and errs["max_abs"] <= 2e-2, errs
    assert errs["lse"] <= 5e-2, errs


CASES = [
    # (B, Hq, Hkv, Nq, Nk, peaks, causal, ctas_per_sm)
    (1, 2, 1, 384, 640, [(300, 120.0)], False, 2),
    (1, 2, 1, 384, 640, [(300, 120.0)], True, 2),
    (2, 4, 2, 300, 777, [(100, 90.0), (500, 250.0)], True, 2),      # two rising peaks, ragged, GQA
    (1, 2, 2, 256, 2304, [(1500, 400.0)], False, None),             # persistent kernel (from 2048 keys on)
    (1, 4, 1, 640, 2176, [(70, 80.0), (2100, 160.0)], True, 1),     # persistent kernel, causal
]


@pytest.mark.parametrize("case", CASES)
def test_fp8_late_peaks_match_oracle(cuda, case):
    from warpy_kernels import attn_fwd
    from warpy_kernels_b200.attn import fwd_api

    B, Hq, Hkv, Nq, Nk, peaks, causal, ctas = case
    q, k, v = late_peak_qkv(B, Hq, Hkv, Nq, Nk, 128, peaks, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, ctas_per_sm=ctas)
    qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
    out_ref, lse_ref = R.attention_reference(qd, kd, vd, causal)
    gates(fwd_errors(out, lse, out_ref, lse_ref, Nq, Nk, causal))
    # rows that see a peak put nearly all their weight on it
    assert pmax.max().item() > 0.99
    # the flag scratch is handed back all zero, so the next call on the stream starts clean
    assert int(fwd_api._block_flags(cuda, 16).count_nonzero()) == 0
    again = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, ctas_per_sm=ctas)
    assert torch.equal(again[0], out) and torch.equal(again[1], lse)


@pytest.mark.parametrize("causal", [False, True])
def test_bf16_late_peaks_match_oracle(cuda, causal):
    from warpy_kernels import attn_fwd

    q, k, v = late_peak_qkv(1, 4, 2, 300, 700, 128, [(200, 100.0), (650, 300.0)], seed=2, device=cuda)
    qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out, lse, _ = attn_fwd(qb, kb, vb, causal=causal)
    out_ref, lse_ref = R.attention_reference(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(), causal)
    errs = fwd_errors(out, lse, out_ref, lse_ref, 300, 700, causal)
    assert errs["out"] <= 1e-2 and errs["lse"] <= 1e-2, errs  # the reference's bf16 gates (tests/attn/test_fwd.py)


def test_rows_inside_the_range_are_not_recomputed(cuda):
    """A 60-nat peak stays inside the range: the tensor-core result is kept and passes the gates."""
    from warpy_kernels import attn_fwd

    q, k, v = late_peak_qkv(1, 2, 1, 256, 512, 128, [(300, 60.0)], device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, lse, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=False)
    qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
    out_ref, lse_ref = R.attention_reference(qd, kd, vd, False)
    gates(fwd_errors(out, lse, out_ref, lse_ref, 256, 512, False))


def test_without_workspace_the_status_word_reports_the_range(cuda):
    """Raw C ABI, ``workspace = NULL``: no recomputation, ``wk_status()`` returns ``WK_ERR_RANGE`` once and clears it."""
    from warpy_kernels_b200 import _lib
    from warpy_kernels_b200.attn.fwd_api import _FwdArgs

    lib = _lib.lib()
    B, H, Nq, Nk, d = 1, 1, 128, 256, 128
    q, k, v = late_peak_qkv(B, H, H, Nq, Nk, d, [(200, 150.0)], device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out = torch.empty(B, H, Nq, d, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(B, H, Nq, dtype=torch.float32, device=cuda)
    pmax = torch.empty_like(lse)
    a = _FwdArgs()
    a.q, a.k, a.v, a.out, a.lse, a.pmax = (t.data_ptr() for t in (q8, k8, v8, out, lse, pmax))
    a.q_descale, a.k_descale, a.v_descale = sq.data_ptr(), sk.data_ptr(), sv.data_ptr()
    a.q_strides = (ctypes.c_int64 * 3)(*q8.stride()[:3])
    a.k_strides = (ctypes.c_int64 * 3)(*k8.stride()[:3])
    a.v_strides = (ctypes.c_int64 * 3)(*v8.stride()[:3])
    a.out_strides = (ctypes.c_int64 * 3)(*out.stride()[:3])
    a.lse_strides = (ctypes.c_int64 * 2)(H * Nq, Nq)
    a.B, a.Hq, a.Hkv, a.Nq, a.Nk, a.d = B, H, H, Nq, Nk, d
    a.causal, a.write_lse, a.lse_natural, a.seqused_k = 0, 1, 0, None
    a.softmax_scale, a.ctas_per_sm = 1.0 / math.sqrt(d), 0
    a.workspace, a.workspace_bytes = None, 0
    assert lib.wk_attn_fwd_fp8(ctypes.byref(a), _lib.stream_ptr(cuda)) == 0
    assert lib.wk_status() == WK_ERR_RANGE
    assert lib.wk_status() == 0
    # the same call with the workspace: recomputed, clean status, right answer
    ws = torch.zeros(lib.wk_attn_fwd_workspace_bytes(B, H, Nq), dtype=torch.uint8, device=cuda)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.wk_attn_fwd_fp8(ctypes.byref(a), _lib.stream_ptr(cuda)) == 0
    assert lib.wk_status() == 0 and int(ws.count_nonzero()) == 0
    qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
    out_ref, lse_ref = R.attention_reference(qd, kd, vd, False)
    gates(fwd_errors(out, lse, out_ref, lse_ref, Nq, Nk, False))
    # a workspace that is too small is rejected before anything is launched
    a.workspace_bytes = 0
    assert lib.wk_attn_fwd_fp8(ctypes.byref(a), _lib.stream_ptr(cuda)) == -1


@pytest.mark.parametrize("bf16", [False, True])
def test_head_dim_64_late_peaks_match_oracle(cuda, bf16):
    """Head dimension 64 takes the same path: flagged blocks are recomputed with half the head-dim lanes idle."""
    from warpy_kernels import attn_fwd

    q, k, v = late_peak_qkv(1, 4, 2, 300, 700, 64, [(200, 100.0), (650, 300.0)], seed=3, device=cuda)
    if bf16:
        qx, kx, vx = q.bfloat16(), k.bfloat16(), v.bfloat16()
        out, lse, _ = attn_fwd(qx, kx, vx, causal=True)
        out_ref, lse_ref = R.attention_reference(qx.float().cpu(), kx.float().cpu(), vx.float().cpu(), True)
        errs = fwd_errors(out, lse, out_ref, lse_ref, 300, 700, True)
        assert errs["out"] <= 1e-2 and errs["lse"] <= 1e-2, errs
    else:
        q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
        out, lse, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
        qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
        out_ref, lse_ref = R.attention_reference(qd, kd, vd, True)
        gates(fwd_errors(out, lse, out_ref, lse_ref, 300, 700, True))
    assert out.shape == q.shape
