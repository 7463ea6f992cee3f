"""GPU: FP8 attention backward against the fp32 oracle (autograd through the reference's attention).

Tolerances: this library's target (cosine >= 0.995 for dq, dk, dv) and the reference's gate (rel-L2 <= 8e-2,
``tests/attn/test_grad.py:19``).
"""

import os

import pytest
import torch

from oracle import reference_math as R
from tests.helpers import hard_inputs, load_golden, randn_qkv

pytestmark = pytest.mark.gpu

GOLDEN = ["attn_mha_causal", "attn_gqa_ragged_causal", "attn_gqa_noncausal", "attn_short_q_causal"]
# shapes of the reference's gradient test (tests/attn/test_grad.py) plus ragged / GQA / Nq != Nk cases
SHAPES = [
    (1, 1, 1, 128, 128, 128),
    (2, 4, 2, 1000, 1000, 128),
    (1, 2, 1, 300, 777, 64),
    (1, 2, 2, 512, 1024, 128),
    (1, 4, 4, 2048, 2048, 64),
    (1, 2, 1, 512, 128, 128),
    (1, 2, 1, 512, 128, 64),
    (1, 8, 2, 384, 640, 128),
    # more key blocks than SMs: the dK/dV CTAs that start take over the blocks of those that have not
    (3, 8, 8, 1024, 1024, 128),
    (5, 8, 4, 1024, 1024, 64),
]


def check_grads(got, want):
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        g, w = g.float().cpu(), w.float().cpu()
        assert not torch.isnan(g).any().item(), f"{name} contains NaN"
        assert R.cosine(g, w) >= 0.995, (name, R.cosine(g, w))
        assert R.rel_l2(g, w) <= 8e-2, (name, R.rel_l2(g, w))


@pytest.mark.parametrize("name", GOLDEN)
def test_against_reference_fixture(cuda, golden_dir, name):
    from warpy_kernels import attn_bwd, attn_fwd

    t = load_golden(os.path.join(golden_dir, f"{name}.npz"), cuda)
    args = (t["q8"], t["k8"], t["v8"])
    scales = (t["sq"], t["sk"], t["sv"])
    out, lse, pmax = attn_fwd(*args, *scales, causal=t["causal"])
    dq, dk, dv = attn_bwd(*args, out, lse, pmax, t["dout"], *scales, causal=t["causal"])
    assert dq.shape == t["q8"].shape and dk.shape == t["k8"].shape and dv.dtype == torch.bfloat16
    check_grads((dq, dk, dv), (t["dq"], t["dk"], t["dv"]))


def _oracle_grads(q8, k8, v8, sq, sk, sv, dout, causal):
    qd, kd, vd = [x.requires_grad_() for x in R.dequantize_qkv(q8, k8, v8, sq, sk, sv)]
    out, _ = R.attention_reference(qd, kd, vd, causal)
    out.backward(dout.float())
    return qd.grad, kd.grad, vd.grad


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_reference_shapes(cuda, shape, causal):
    from warpy_kernels import attn_bwd, attn_fwd

    q, k, v = randn_qkv(*shape, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    dout = torch.randn(q.shape, device=cuda, generator=torch.Generator(device=cuda).manual_seed(7)).bfloat16()
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal)
    got = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=causal)
    check_grads(got, _oracle_grads(q8, k8, v8, sq, sk, sv, dout, causal))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 4, 2, 640, 640, 128), (2, 4, 2, 1000, 1000, 128), (1, 4, 4, 2048, 2048, 64)])
def test_repeat_is_bit_identical(cuda, shape, causal):
    """Four runs: dK and dV bit-identical ("else a race", the reference's ``repeat`` shapes,
    ``tests/attn/test_grad.py:108-135``); dQ too, since this backward has no atomics."""
    from warpy_kernels import attn_bwd, attn_fwd

    q, k, v = randn_qkv(*shape, seed=3, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    dout = torch.randn(q.shape, device=cuda).bfloat16()
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal)
    first = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=causal)
    for _ in range(3):
        again = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=causal, deterministic=True)
        for a, b in zip(first, again):
            assert torch.equal(a, b)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 4, 2, 512, 512, 128), (1, 4, 2, 1024, 1024, 128), (1, 4, 4, 1024, 1024, 64)])
def test_hard_inputs_mean_over_seeds(cuda, shape, causal):
    """Peaky softmax, log-normal dO row norms (``grad_hard`` with the reference's ``HARD_SHAPES``,
    ``tests/attn/test_grad.py:87-105``): mean error over 3 seeds."""
    from warpy_kernels import attn_bwd, attn_fwd

    errs = {"dq": 0.0, "dk": 0.0, "dv": 0.0}
    for seed in range(3):
        q, k, v, dout = hard_inputs(*shape, seed=seed, device=cuda)
        dout = dout.bfloat16()
        q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
        out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal)
        got = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=causal)
        want = _oracle_grads(q8, k8, v8, sq, sk, sv, dout, causal)
        for name, g, w in zip(errs, got, want):
            errs[name] += R.rel_l2(g, w) / 3
    assert max(errs.values()) <= 8e-2, errs


def test_strided_inputs_and_float_dout(cuda):
    from warpy_kernels import attn_bwd, attn_fwd

    B, H, N, d = 2, 4, 300, 128
    q, k, v = randn_qkv(B, H, H, N, N, d, seed=5, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    dout = torch.randn(q.shape, device=cuda)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    base = attn_bwd(q8, k8, v8, out, lse, pmax, dout.bfloat16(), sq, sk, sv, causal=True)
    tq, tk, tv = [x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q8, k8, v8)]
    tout = out.transpose(1, 2).contiguous().transpose(1, 2)
    got = attn_bwd(tq, tk, tv, tout, lse, pmax, dout, sq, sk, sv, causal=True)  # float32 dout is converted
    for a, b in zip(base, got):
        assert torch.equal(a, b)


def test_rows_on_8_byte_boundaries(cuda):
    """``dout`` / ``out`` rows that start on 8-byte but not 16-byte boundaries take the one-row-per-warp prep kernel
    instead of the 16-byte-load one; the two differ only in the order of the sum over the head dimension."""
    from warpy_kernels import attn_bwd, attn_fwd

    B, H, N, d = 1, 2, 333, 128
    q, k, v = randn_qkv(B, H, H, N, N, d, seed=11, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    dout = torch.randn(q.shape, device=cuda).bfloat16()
    base = attn_bwd(q8, k8, v8, out, lse, pmax, dout, sq, sk, sv, causal=True)
    wide = torch.zeros(B, H, N, d + 4, device=cuda, dtype=torch.bfloat16)
    wide[..., :d] = dout
    wide_out = torch.zeros(B, H, N, d + 4, device=cuda, dtype=torch.bfloat16)
    wide_out[..., :d] = out
    got = attn_bwd(q8, k8, v8, wide_out[..., :d], lse, pmax, wide[..., :d], sq, sk, sv, causal=True)
    for a, b in zip(base, got):
        assert R.cosine(a.float().cpu(), b.float().cpu()) >= 0.9999
        assert R.rel_l2(a.float().cpu(), b.float().cpu()) <= 1e-2


def test_validation_errors(cuda):
    from warpy_kernels import attn_bwd

    q = torch.zeros(1, 2, 128, 128, device=cuda).to(torch.float8_e4m3fn)
    kv = torch.zeros(1, 1, 128, 128, device=cuda).to(torch.float8_e4m3fn)
    o = torch.zeros(1, 2, 128, 128, device=cuda, dtype=torch.bfloat16)
    l = torch.zeros(1, 2, 128, device=cuda)
    with pytest.raises(NotImplementedError):
        attn_bwd(q, kv, kv, o, l, l, o, seqused_k=torch.ones(1, device=cuda, dtype=torch.int32))
    with pytest.raises(ValueError):
        attn_bwd(q, kv, kv, o[:, :1], l, l, o)
    with pytest.raises(ValueError):
        attn_bwd(q, kv, kv, o, l[:, :, :64], l, o)
    with pytest.raises(ValueError):
        attn_bwd(q, kv.bfloat16(), kv, o, l, l, o)


# ---- bf16 inputs ---------------------------------------------------------------------------------------------
def _bf16_case(cuda, q, k, v, dout, causal):
    """The reference's ``_bf16_grad`` (``tests/attn/test_grad.py:139-183``): rel-L2 <= 2e-2 for dq, dk, dv."""
    from warpy_kernels import attn_bwd, attn_fwd

    q, k, v, dout = [x.bfloat16() for x in (q, k, v, dout)]
    out, lse, pmax = attn_fwd(q, k, v, causal=causal)
    got = attn_bwd(q, k, v, out, lse, pmax, dout, causal=causal)
    qf, kf, vf = [x.float().cpu().requires_grad_() for x in (q, k, v)]
    out_ref, _ = R.attention_reference(qf, kf, vf, causal)
    out_ref.backward(dout.float().cpu())
    for name, g, w in zip(("dq", "dk", "dv"), got, (qf.grad, kf.grad, vf.grad)):
        g = g.float().cpu()
        assert g.shape == w.shape and not torch.isnan(g).any().item(), name
        assert R.rel_l2(g, w) <= 2e-2, (name, R.rel_l2(g, w))
        assert R.cosine(g, w) >= 0.995, (name, R.cosine(g, w))
    return got


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bf16_reference_shapes(cuda, shape, causal):
    q, k, v = randn_qkv(*shape, device=cuda)
    dout = torch.randn(q.shape, device=cuda, generator=torch.Generator(device=cuda).manual_seed(7))
    _bf16_case(cuda, q, k, v, dout, causal)


@pytest.mark.parametrize("causal", [False, True])
def test_bf16_hard_inputs_and_repeat(cuda, causal):
    """Peaky softmax and log-normal dO row norms (``grad_bf16_hard``); a second run gives the same bits."""
    from warpy_kernels import attn_bwd, attn_fwd

    q, k, v, dout = hard_inputs(1, 4, 2, 640, 640, 128, device=cuda)
    first = _bf16_case(cuda, q, k, v, dout, causal)
    qb, kb, vb, db = [x.bfloat16() for x in (q, k, v, dout)]
    out, lse, pmax = attn_fwd(qb, kb, vb, causal=causal)
    again = attn_bwd(qb, kb, vb, out, lse, pmax, db, causal=causal)
    for a, b in zip(first, again):
        assert torch.equal(a, b)


def test_bf16_strided_views(cuda):
    """``[B, N, H, d]`` storage for q, k, v and dout."""
    B, Hq, Hkv, Nq, Nk, d = 2, 4, 2, 200, 333, 128
    g = torch.Generator(device=cuda).manual_seed(11)
    mk = lambda n, h: torch.randn(B, n, h, d, device=cuda, generator=g).transpose(1, 2)
    _bf16_case(cuda, mk(Nq, Hq), mk(Nk, Hkv), mk(Nk, Hkv), mk(Nq, Hq), True)
