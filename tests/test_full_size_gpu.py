"""GPU: parity at the benchmark configurations' full sizes.

The oracle cannot evaluate these shapes whole in seconds, so each test runs the kernel on the full problem and
checks (a) a slice of the result against the oracle evaluated on that slice only, and (b) a size-independent
property of the whole result.
"""

import math

import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn


def _per_tensor(x):
    scale = x.abs().amax().clamp_min(1e-12) / 448.0
    return (x / scale).to(FP8), scale


def _attn_inputs(cuda, B, Hq, Hkv, N, d, seed):
    g = torch.Generator(device=cuda).manual_seed(seed)
    mk = lambda h: torch.randn(B, h, N, d, device=cuda, generator=g).bfloat16().float()
    q8, sq = _per_tensor(mk(Hq))
    k8, sk = _per_tensor(mk(Hkv))
    v8, sv = _per_tensor(mk(Hkv))
    full = lambda s: torch.full((B, Hkv), float(s), device=cuda)
    return q8, k8, v8, full(sq), full(sk), full(sv)


def _oracle_head(q8, k8, v8, sq, sk, sv, b, hq, rows, dout=None):
    """Oracle for query rows ``rows`` (a slice) of head ``hq`` of batch ``b``; causal, bottom-right aligned."""
    group = q8.shape[1] // k8.shape[1]
    hk = hq // group
    qd = (q8[b, hq, rows].float() * sq[b, hk])[None, None]
    kd = (k8[b, hk].float() * sk[b, hk])[None, None]
    vd = (v8[b, hk].float() * sv[b, hk])[None, None]
    offset = rows.start + k8.shape[2] - q8.shape[2]
    return R._attn_offset(qd, kd, vd, offset, None) if dout is None else None


def test_config1_attention_forward_b4_h32_n4096(cuda):
    """The forward benchmark shape (B4 H32 N4096 d128, causal): slices of two heads against the oracle (cosine >= 0.999, max-abs <= 2e-2), and rows of
    the probability simplex: every lse finite, pmax in (0, 1], out bounded by the largest |v|."""
    from warpy_kernels import attn_fwd

    B, H, N, d = 4, 32, 4096, 128
    q8, k8, v8, sq, sk, sv = _attn_inputs(cuda, B, H, H, N, d, 0)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    for b, h, rows in ((0, 0, slice(0, 512)), (3, 31, slice(3584, 4096)), (1, 17, slice(1900, 2200))):
        ref, lse_ref = _oracle_head(q8, k8, v8, sq, sk, sv, b, h, rows)
        got = out[b, h, rows].float()
        assert R.cosine(got, ref[0, 0]) >= 0.999
        assert R.max_abs(got, ref[0, 0]) <= 2e-2
        assert (lse[b, h, rows] - lse_ref[0, 0]).abs().max().item() <= 5e-2
    assert torch.isfinite(lse).all() and bool((pmax > 0).all()) and bool((pmax <= 1.0001).all())
    vmax = (v8.float().abs().amax() * sv[0, 0]).item()
    assert out.float().abs().max().item() <= vmax * 1.01


def test_config2_attention_backward_b4_h32_n4096(cuda):
    """The backward benchmark shape (B4 H32 N4096 d128, causal): gradients of one head against autograd through the oracle (cosine >= 0.995)."""
    from warpy_kernels import attn_bwd, attn_fwd

    B, H, N, d = 4, 32, 4096, 128
    q8, k8, v8, sq, sk, sv = _attn_inputs(cuda, B, H, H, N, d, 0)
    dout = torch.randn(B, H, N, d, device=cuda, generator=torch.Generator(device=cuda).manual_seed(7)).bfloat16()
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    dq, dk, dv = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=True)
    b, h = 2, 5
    qd = (q8[b, h].float() * sq[b, h])[None, None].requires_grad_()
    kd = (k8[b, h].float() * sk[b, h])[None, None].requires_grad_()
    vd = (v8[b, h].float() * sv[b, h])[None, None].requires_grad_()
    ref, _ = R.attention_reference(qd, kd, vd, True)
    ref.backward(dout[b, h].float()[None, None])
    for got, want in ((dq[b, h], qd.grad), (dk[b, h], kd.grad), (dv[b, h], vd.grad)):
        assert R.cosine(got.float(), want[0, 0]) >= 0.995
        assert R.rel_l2(got.float(), want[0, 0]) <= 8e-2
    assert not torch.isnan(dq).any() and not torch.isnan(dk).any() and not torch.isnan(dv).any()


def test_config4_gqa_long_context_one_kv_group(cuda):
    """The GQA benchmark shape (B1 Hq64 Hkv8 N32768 d128) restricted to one KV head (8 query heads, N = 32768): the shard one GPU of eight runs.
    The last 256 queries of two heads against the oracle."""
    from warpy_kernels import attn_fwd

    q8, k8, v8, sq, sk, sv = _attn_inputs(cuda, 1, 8, 1, 32768, 128, 4)
    out, lse, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    for h in (0, 7):
        rows = slice(32768 - 256, 32768)
        ref, lse_ref = _oracle_head(q8, k8, v8, sq, sk, sv, 0, h, rows)
        assert R.cosine(out[0, h, rows].float(), ref[0, 0]) >= 0.999
        assert R.max_abs(out[0, h, rows].float(), ref[0, 0]) <= 2e-2
        assert (lse[0, h, rows] - lse_ref[0, 0]).abs().max().item() <= 5e-2


def test_config4_gqa_long_context_whole_shape(cuda):
    """The GQA benchmark shape whole, as one GPU runs it (B1 Hq64 Hkv8 N32768 d128, causal: 16384 query blocks through the persistent kernel's
    hand-over): slices at the start, in the middle and at the end of heads from different KV groups against the oracle,
    plus the properties of a probability row for every row."""
    from warpy_kernels import attn_fwd

    N = 32768
    q8, k8, v8, sq, sk, sv = _attn_inputs(cuda, 1, 64, 8, N, 128, 4)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    for h, rows in ((0, slice(0, 384)), (13, slice(16000, 16256)), (42, slice(N - 4224, N - 3968)), (63, slice(N - 256, N))):
        ref, lse_ref = _oracle_head(q8, k8, v8, sq, sk, sv, 0, h, rows)
        assert R.cosine(out[0, h, rows].float(), ref[0, 0]) >= 0.999, h
        assert R.max_abs(out[0, h, rows].float(), ref[0, 0]) <= 2e-2, h
        assert (lse[0, h, rows] - lse_ref[0, 0]).abs().max().item() <= 5e-2, h
    assert torch.isfinite(lse).all() and bool((pmax > 0).all()) and bool((pmax <= 1.0001).all())
    vmax = (v8.float().abs().amax() * sv[0, 0]).item()
    assert out.float().abs().max().item() <= vmax * 1.01


def test_config2_sized_gqa_backward(cuda):
    """A backward of the benchmark's size with grouped heads (B2 Hq32 Hkv8 N4096 d128, causal): all gradients of one
    KV group (its four query heads' dQ, its dK and dV) against autograd through the oracle."""
    from warpy_kernels import attn_bwd, attn_fwd

    B, Hq, Hkv, N, d = 2, 32, 8, 4096, 128
    q8, k8, v8, sq, sk, sv = _attn_inputs(cuda, B, Hq, Hkv, N, d, 1)
    dout = torch.randn(B, Hq, N, d, device=cuda, generator=torch.Generator(device=cuda).manual_seed(7)).bfloat16()
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    dq, dk, dv = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=True)
    b, hk = 1, 5
    heads = slice(4 * hk, 4 * hk + 4)
    qd = (q8[b, heads].float() * sq[b, hk])[None].requires_grad_()
    kd = (k8[b, hk].float() * sk[b, hk])[None, None].requires_grad_()
    vd = (v8[b, hk].float() * sv[b, hk])[None, None].requires_grad_()
    ref, _ = R.attention_reference(qd, kd, vd, True)
    ref.backward(dout[b, heads].float()[None])
    for got, want in ((dq[b, heads], qd.grad[0]), (dk[b, hk], kd.grad[0, 0]), (dv[b, hk], vd.grad[0, 0])):
        assert R.cosine(got.float(), want) >= 0.995
        assert R.rel_l2(got.float(), want) <= 8e-2
    for g in (dq, dk, dv):
        assert not torch.isnan(g).any()


@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
def test_config3_mxfp8_gemm_m8192(cuda, n, k):
    """The MXFP8 GEMM benchmark shape (M8192 N14336 K4096): a band of rows against the oracle, and linearity in the scale bytes: raising every scale
    byte of A by one doubles the product exactly."""
    from warpy_kernels import gemm, quantize_mx

    m = 8192
    g = torch.Generator(device=cuda).manual_seed(0)
    a8, sa = quantize_mx(torch.randn(m, k, device=cuda, generator=g).bfloat16())
    b8, sb = quantize_mx(torch.randn(n, k, device=cuda, generator=g).bfloat16())
    out = gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb)
    rows = slice(4096 - 128, 4096 + 128)
    want = R.mx_dequant(a8[rows], sa[rows]) @ R.mx_dequant(b8, sb).T
    assert R.rel_l2(out[rows].float(), want) <= 1e-2
    assert R.rel_l2(out[rows].float(), want.bfloat16().float()) <= 1e-3
    out2 = gemm(a8, b8, a_scale_mx=sa + 1, b_scale_mx=sb)
    assert torch.equal(out2.float(), out.float() * 2)


def test_config0_bf16_gemm_2048(cuda):
    """The BF16 GEMM benchmark shape (M = N = K = 2048) whole: relative Frobenius error <= 1e-2 against fp32 accumulation."""
    from warpy_kernels import gemm

    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(2048, 2048, device=cuda, generator=g).bfloat16()
    b = torch.randn(2048, 2048, device=cuda, generator=g).bfloat16()
    out = gemm(a, b)
    want = a.float() @ b.float().T
    assert R.rel_l2(out, want) <= 1e-2
