"""GPU: FP8 attention forward against the fp32 oracle.

Tolerances: this library's target gates (cosine >= 0.999, max-abs <= 2e-2) and the reference's own
(``tests/attn/test_fwd.py:21``: out rel-L2 <= 6e-2, lse max-abs <= 5e-2).
"""

import os

import pytest
import torch

from oracle import reference_math as R
from tests.helpers import fwd_errors, load_golden, randn_qkv, sink_qkv

pytestmark = pytest.mark.gpu

GOLDEN = ["attn_mha_causal", "attn_gqa_ragged_causal", "attn_gqa_noncausal", "attn_short_q_causal"]
# the shapes of the reference's forward test (tests/attn/test_fwd.py:23-31) plus one more: (B, Hq, Hkv, Nq, Nk, d)
SHAPES = [
    (1, 1, 1, 128, 64, 128),
    (2, 4, 2, 1000, 1000, 128),
    (1, 2, 1, 300, 777, 64),
    (1, 2, 2, 512, 1024, 128),
    (1, 4, 4, 2048, 2048, 64),
    (1, 2, 1, 512, 128, 128),
    (1, 2, 1, 512, 128, 64),
    (1, 8, 2, 384, 640, 128),
]


def check(errs):
    assert errs["out"] <= 6e-2, errs
    assert errs["lse"] <= 5e-2, errs
    assert errs["cos"] >= 0.999, errs
    assert errs["max_abs"] <= 2e-2, errs


@pytest.mark.parametrize("name", GOLDEN)
def test_against_reference_fixture(cuda, golden_dir, name):
    from warpy_kernels import attn_fwd

    t = load_golden(os.path.join(golden_dir, f"{name}.npz"), cuda)
    out, lse, pmax = attn_fwd(t["q8"], t["k8"], t["v8"], t["sq"], t["sk"], t["sv"], causal=t["causal"])
    assert out.dtype == torch.bfloat16 and out.shape == t["q8"].shape
    Nq, Nk = t["q8"].shape[2], t["k8"].shape[2]
    check(fwd_errors(out, lse, t["out"], t["lse"], Nq, Nk, t["causal"]))
    # pmax = largest probability of the row
    qd, kd, vd = R.dequantize_qkv(t["q8"].cpu(), t["k8"].cpu(), t["v8"].cpu(), t["sq"].cpu(), t["sk"].cpu(), t["sv"].cpu())
    rep = qd.shape[1] // kd.shape[1]
    s = (qd @ kd.repeat_interleave(rep, 1).transpose(-1, -2)) / (128**0.5)
    if t["causal"]:
        row = torch.arange(Nq)[:, None]
        col = torch.arange(Nk)[None, :]
        s = s.masked_fill(col > row + Nk - Nq, float("-inf"))
    want = torch.softmax(s, -1).amax(-1)
    vis = torch.isfinite(t["lse"])
    assert (pmax.cpu()[vis] - want[vis]).abs().max().item() <= 0.05 * want[vis].max().item() + 1e-3


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_reference_shapes(cuda, shape, causal):
    from warpy_kernels import attn_fwd

    q, k, v = randn_qkv(*shape, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, lse, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal)
    qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
    out_ref, lse_ref = R.attention_reference(qd, kd, vd, causal)
    check(fwd_errors(out, lse, out_ref, lse_ref, shape[3], shape[4], causal))


def test_repeat_is_bit_identical(cuda):
    from warpy_kernels import attn_fwd

    q, k, v = randn_qkv(1, 4, 2, 640, 640, 128, seed=3, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    a = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    b = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_layouts_bit_equal(cuda):
    """``[B, N, H, d]``-strided views, ``out=`` reuse and ``return_lse=False`` (``tests/attn/test_layout.py:24-80``)."""
    from warpy_kernels import attn_fwd

    B, H, N, d = 2, 4, 300, 128
    q, k, v = randn_qkv(B, H, H, N, N, d, seed=5, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    base = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    tq, tk, tv = [x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q8, k8, v8)]  # [B, N, H, d] storage
    out, lse, pmax = attn_fwd(tq, tk, tv, sq, sk, sv, causal=True)
    assert out.stride() == tq.stride()  # out keeps q's memory layout
    assert torch.equal(out, base[0]) and torch.equal(lse, base[1]) and torch.equal(pmax, base[2])
    qkv = torch.stack([q8.view(torch.uint8), k8.view(torch.uint8), v8.view(torch.uint8)], dim=3).view(torch.float8_e4m3fn)
    out2, _, _ = attn_fwd(qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2], sq, sk, sv, causal=True)  # fused QKV
    assert torch.equal(out2, base[0])
    buf = torch.empty_like(base[0])
    out3, l3, p3 = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True, out=buf, return_lse=False)
    assert out3 is buf and l3 is None and p3 is None and torch.equal(buf, base[0])


def test_seqused_and_natural_lse(cuda):
    """``seqused_k`` equals truncating K/V; ``lse_natural`` is ``lse * ln 2`` (``tests/attn/test_seqused.py:13-88``)."""
    from warpy_kernels import attn_fwd

    q, k, v = randn_qkv(2, 2, 1, 256, 512, 128, seed=9, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    used = torch.tensor([200, 512], dtype=torch.int32, device=cuda)
    for causal in (False, True):
        out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, seqused_k=used)
        for b, n in enumerate(used.tolist()):
            o1, l1, p1 = attn_fwd(q8[b : b + 1], k8[b : b + 1, :, :n], v8[b : b + 1, :, :n], sq[b : b + 1],
                                  sk[b : b + 1], sv[b : b + 1], causal=causal)
            assert torch.equal(out[b : b + 1], o1) and torch.equal(lse[b : b + 1], l1)
    _, lse2, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    _, lsen, _ = attn_fwd(q8, k8, v8, sq, sk, sv, causal=True, lse_natural=True)
    assert torch.allclose(lsen, lse2 * 0.6931471805599453, rtol=1e-6, atol=1e-6)


def test_seqused_persistent_kernel(cuda):
    """``seqused_k`` through the persistent kernel (picked from 2048 keys on): a batch item with few keys belongs
    wholly to the two-term launch, so the persistent CTAs skip its query blocks; one with a ragged length mixes
    both.  Each item equals the call on its truncated K/V."""
    from warpy_kernels import attn_fwd

    q, k, v = randn_qkv(3, 4, 2, 640, 2560, 128, seed=13, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    used = torch.tensor([2560, 700, 300], dtype=torch.int32, device=cuda)
    for causal in (False, True):
        out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, seqused_k=used)
        for b, n in enumerate(used.tolist()):
            o1, l1, p1 = attn_fwd(q8[b : b + 1], k8[b : b + 1, :, :n], v8[b : b + 1, :, :n], sq[b : b + 1],
                                  sk[b : b + 1], sv[b : b + 1], causal=causal, ctas_per_sm=1)
            assert torch.equal(out[b : b + 1], o1) and torch.equal(lse[b : b + 1], l1), (causal, b)
        qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
        out_ref, lse_ref = R.attention_reference(qd[:1], kd[:1], vd[:1], causal)
        check(fwd_errors(out[:1], lse[:1], out_ref, lse_ref, 640, 2560, causal))


@pytest.mark.parametrize("gap", [8])
def test_sink_long_tail(cuda, gap):
    """One dominant key over a 32768-key tail (``tests/attn/test_fwd.py:104-114``, gate 2e-2)."""
    from warpy_kernels import attn_fwd

    q, k, v = sink_qkv(256, 32768, 128, gap, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, _, _ = attn_fwd(q8, k8, v8, sq, sk, sv)
    ref, _ = R.attention_reference(*R.dequantize_qkv(q8, k8, v8, sq, sk, sv), False)
    assert R.rel_l2(out, ref) <= 2e-2


def test_validation_errors(cuda):
    from warpy_kernels import attn_fwd

    q = torch.zeros(1, 2, 128, 128, device=cuda).to(torch.float8_e4m3fn)
    kv = torch.zeros(1, 1, 128, 128, device=cuda).to(torch.float8_e4m3fn)
    with pytest.raises(ValueError):
        attn_fwd(q, kv.bfloat16(), kv)
    with pytest.raises(ValueError):
        attn_fwd(q, kv[:, :, :, :64], kv)
    with pytest.raises(ValueError):
        attn_fwd(q, kv, kv, q_descale=torch.ones(1, 2, device=cuda))
    with pytest.raises(ValueError):
        attn_fwd(q, kv, kv, seqused_k=torch.ones(1, device=cuda))
    with pytest.raises(ValueError):
        attn_fwd(q.bfloat16(), kv.bfloat16(), kv.bfloat16(), q_descale=torch.ones(1, 1, device=cuda))  # bf16 has no descales
    with pytest.raises(ValueError):
        attn_fwd(q, kv, kv, out=torch.empty(1, 2, 128, 128, device=cuda))


# ---- bf16 inputs ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_bf16_reference_shapes(cuda, shape, causal):
    """The reference's ``fwd_bf16`` case (``tests/attn/test_fwd.py:117-144``): out rel-L2 and lse max-abs <= 1e-2."""
    from warpy_kernels import attn_fwd

    q, k, v = [x.bfloat16() for x in randn_qkv(*shape, device=cuda)]
    out, lse, pmax = attn_fwd(q, k, v, causal=causal)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    out_ref, lse_ref = R.attention_reference(q.float().cpu(), k.float().cpu(), v.float().cpu(), causal)
    errs = fwd_errors(out, lse, out_ref, lse_ref, shape[3], shape[4], causal)
    assert errs["out"] <= 1e-2 and errs["lse"] <= 1e-2 and errs["cos"] >= 0.999, errs
    assert torch.equal(attn_fwd(q, k, v, causal=causal)[0], out), "repeated launches differ"


def test_bf16_sink_and_late_peaks(cuda):
    """A row reference fixed by the first tile must survive much larger scores later in the row, and a huge first
    score (attention sink) with small ones after it."""
    from warpy_kernels import attn_fwd

    B, H, N, d = 1, 2, 1024, 128
    g = torch.Generator(device=cuda).manual_seed(5)
    q = torch.randn(B, H, N, d, device=cuda, generator=g)
    k = torch.randn(B, H, N, d, device=cuda, generator=g)
    v = torch.randn(B, H, N, d, device=cuda, generator=g)
    for mode in ("late_peak", "sink"):
        kk = k.clone()
        if mode == "late_peak":
            kk[:, :, 700:] *= 6.0  # logits grow by tens of bits after the first tile
        else:
            kk[:, :, 0] = q.mean(2) * 8.0  # key 0 dominates every row
        qb, kb, vb = q.bfloat16(), kk.bfloat16(), v.bfloat16()
        out, lse, _ = attn_fwd(qb, kb, vb, causal=False)
        out_ref, lse_ref = R.attention_reference(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(), False)
        errs = fwd_errors(out, lse, out_ref, lse_ref, N, N, False)
        assert errs["out"] <= 1e-2 and errs["lse"] <= 1e-2, (mode, errs)


def test_bf16_layouts_and_options(cuda):
    """``[B, N, H, d]`` views, GQA, ragged lengths, ``seqused_k``, natural-log lse, ``return_lse=False``, d = 64."""
    from warpy_kernels import attn_fwd

    B, Hq, Hkv, Nq, Nk, d = 2, 4, 2, 200, 333, 128
    g = torch.Generator(device=cuda).manual_seed(9)
    q = torch.randn(B, Nq, Hq, d, device=cuda, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(B, Nk, Hkv, d, device=cuda, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(B, Nk, Hkv, d, device=cuda, generator=g).bfloat16().transpose(1, 2)
    out, lse, _ = attn_fwd(q, k, v, causal=True, lse_natural=True)
    out_ref, lse_ref = R.attention_reference(q.float().cpu(), k.float().cpu(), v.float().cpu(), True)
    errs = fwd_errors(out, lse / 0.6931471805599453, out_ref, lse_ref, Nq, Nk, True)
    assert errs["out"] <= 1e-2 and errs["lse"] <= 1.5e-2, errs
    out2, lse2, pmax2 = attn_fwd(q, k, v, causal=True, return_lse=False)
    assert lse2 is None and pmax2 is None and torch.equal(out2, out)
    used = torch.tensor([333, 100], dtype=torch.int32, device=cuda)
    out3, lse3, _ = attn_fwd(q, k, v, causal=False, seqused_k=used)
    ref3, _ = R.attention_reference(q[1:].float().cpu(), k[1:, :, :100].float().cpu(), v[1:, :, :100].float().cpu(), False)
    assert R.rel_l2(out3[1:].float().cpu(), ref3) <= 1e-2
    q64, k64, v64 = [x[..., :64].contiguous() for x in (q, k, v)]
    out4, lse4, _ = attn_fwd(q64, k64, v64, causal=True)
    ref4, lse_ref4 = R.attention_reference(q64.float().cpu(), k64.float().cpu(), v64.float().cpu(), True)
    errs = fwd_errors(out4, lse4, ref4, lse_ref4, Nq, Nk, True)
    assert out4.shape == q64.shape and errs["out"] <= 1e-2 and errs["lse"] <= 1e-2, errs


def test_autotune_stores_the_winner(cuda, tmp_path, monkeypatch):
    """``autotune_attn_fwd`` times its candidates and writes the reference's cache entry for the shape."""
    import json

    from warpy_kernels.attn import autotune_attn_fwd
    from warpy_kernels_b200 import utils

    monkeypatch.setattr(utils, "TUNE_CACHE_PATH", str(tmp_path / "tune.json"))
    q, k, v = randn_qkv(1, 4, 2, 256, 384, 128, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    best, results = autotune_attn_fwd(q8, k8, v8, iters=2, verbose=False, q_descale=sq, k_descale=sk, v_descale=sv,
                                      causal=True)
    assert best in ({"ctas_per_sm": 1}, {"ctas_per_sm": 2}) and len(results) == 2
    assert all(isinstance(t, float) for _, t in results)
    assert json.load(open(tmp_path / "tune.json")) == {"fwd|d=128|causal=1|nq=1024|nk=1024|rep=2|sm100": best}


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 4, 2, 1000, 1000, 128), (1, 2, 2, 512, 1024, 128), (1, 8, 2, 384, 1300, 128),
                                   (1, 2, 1, 300, 777, 64)])
def test_wide_kernel(cuda, shape, causal):
    """``ctas_per_sm=1``: the one-CTA-per-SM kernel with 128-key rounds, on shapes with odd and even numbers of
    64-key tiles, ragged ends and GQA; same gates as the default kernel, and the two agree closely."""
    from warpy_kernels import attn_fwd

    q, k, v = randn_qkv(*shape, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    out, lse, pmax = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, ctas_per_sm=1)
    qd, kd, vd = R.dequantize_qkv(q8.cpu(), k8.cpu(), v8.cpu(), sq.cpu(), sk.cpu(), sv.cpu())
    out_ref, lse_ref = R.attention_reference(qd, kd, vd, causal)
    check(fwd_errors(out, lse, out_ref, lse_ref, shape[3], shape[4], causal))
    out2, lse2, pmax2 = attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, ctas_per_sm=2)
    vis = torch.isfinite(lse2)
    assert (lse[vis] - lse2[vis]).abs().max().item() <= 1e-3 and (pmax[vis] - pmax2[vis]).abs().max().item() <= 1e-3
    assert torch.equal(attn_fwd(q8, k8, v8, sq, sk, sv, causal=causal, ctas_per_sm=1)[0], out), "repeated launches differ"


def test_launch_closure_keeps_its_outputs_alive(cuda):
    """A caller may keep only ``launch`` and drop ``out``, ``lse`` and ``pmax``: the closure must own them, or the
    kernel writes into memory the allocator has already handed to someone else."""
    import gc

    from warpy_kernels.attn import make_attn_fwd

    q, k, v = randn_qkv(2, 4, 4, 256, 256, 128, device=cuda)
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
    launch, out, lse, pmax = make_attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
    sizes = [t.numel() * t.element_size() for t in (out, lse, pmax)]
    del out, lse, pmax
    gc.collect()
    canaries = [torch.zeros(n, dtype=torch.uint8, device=cuda) for n in sizes for _ in range(4)]
    launch()
    torch.cuda.synchronize()
    assert all(int(c.count_nonzero()) == 0 for c in canaries)
