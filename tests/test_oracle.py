"""CPU: the oracle restatements against fixtures produced by the reference's own test oracle, and the quantiser
restatements against known answers derived from the reference's PTX text (``warpy_kernels/ptx/common.py:546-565``)."""

import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import reference_math as R

ATTN = ["attn_mha_causal", "attn_gqa_ragged_causal", "attn_gqa_noncausal", "attn_short_q_causal"]


def load_attn(golden_dir, name):
    z = np.load(os.path.join(golden_dir, f"{name}.npz"))
    B, Hq, Hkv, Nq, Nk, d, causal, seed = [int(x) for x in z["shape"]]
    f8 = lambda a: torch.from_numpy(a).view(torch.float8_e4m3fn)
    return z, dict(
        q8=f8(z["q8"]), k8=f8(z["k8"]), v8=f8(z["v8"]),
        sq=torch.from_numpy(z["sq"]), sk=torch.from_numpy(z["sk"]), sv=torch.from_numpy(z["sv"]),
        dout=torch.from_numpy(z["dout_bf16"]).view(torch.bfloat16), causal=bool(causal),
    )


def _same_to_ulps(got, want, rtol, atol):
    finite = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), finite)
    assert np.array_equal(got[~finite], want[~finite], equal_nan=True)
    assert np.allclose(got[finite], want[finite], rtol=rtol, atol=atol)


@pytest.mark.parametrize("name", ATTN)
def test_attention_oracle_matches_reference_fixture(golden_dir, name):
    z, t = load_attn(golden_dir, name)
    qd, kd, vd = [x.requires_grad_() for x in R.dequantize_qkv(t["q8"], t["k8"], t["v8"], t["sq"], t["sk"], t["sv"])]
    out, lse = R.attention_reference(qd, kd, vd, t["causal"])
    out.backward(t["dout"].float())
    # fp32 reductions on the CPU depend on how torch splits them over threads (one thread under torchrun, all
    # cores otherwise), so the pin is to a few ulp, not to the bit; the pattern of non-finite entries is exact
    _same_to_ulps(out.detach().numpy(), z["out"].astype(np.float32), rtol=2.0**-10, atol=2.0**-14)  # stored as fp16
    _same_to_ulps(lse.detach().numpy(), z["lse"], rtol=2e-6, atol=2e-6)  # includes -inf rows
    for got, key in ((qd.grad, "dq"), (kd.grad, "dk"), (vd.grad, "dv")):
        _same_to_ulps(got.numpy(), z[key], rtol=2e-5, atol=2e-6 * float(np.abs(z[key]).max()))


@pytest.mark.parametrize("name", ATTN)
def test_chunked_oracle_equals_plain(golden_dir, name):
    z, t = load_attn(golden_dir, name)
    qd, kd, vd = R.dequantize_qkv(t["q8"], t["k8"], t["v8"], t["sq"], t["sk"], t["sv"])
    out, lse, dq, dk, dv = R.attention_reference_chunked(qd, kd, vd, t["causal"], dout=t["dout"], q_chunk=96)
    assert np.abs(out.numpy() - z["out"].astype(np.float32)).max() < 2e-3
    fin = np.isfinite(z["lse"])
    assert np.array_equal(np.isfinite(lse.numpy()), fin)
    assert np.abs(lse.numpy()[fin] - z["lse"][fin]).max() < 1e-4
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert np.abs(got.numpy() - z[key]).max() < 1e-3


def test_quantize_qkv_roundtrip_matches_fixture(golden_dir):
    z, t = load_attn(golden_dir, "attn_gqa_ragged_causal")
    # the fixture stores the first rows of the float inputs: re-quantising the dequantised tensors is a fixed point
    qd, kd, vd = R.dequantize_qkv(t["q8"], t["k8"], t["v8"], t["sq"], t["sk"], t["sv"])
    q8, k8, v8, sq, sk, sv = R.quantize_qkv(qd, kd, vd)
    assert torch.equal(q8.view(torch.uint8), t["q8"].view(torch.uint8))
    assert torch.equal(k8.view(torch.uint8), t["k8"].view(torch.uint8))
    assert torch.allclose(sq, t["sq"], rtol=1e-6) and torch.allclose(sv, t["sv"], rtol=1e-6)


def test_metrics_match_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "metrics.npz"))
    a, b = torch.from_numpy(z["a"]), torch.from_numpy(z["b"])
    assert R.rel_l2(a, b) == pytest.approx(float(z["rel_l2"]), rel=1e-6)
    assert R.row_p99(a, b) == pytest.approx(float(z["row_p99"]), rel=1e-6)


def test_mx_dequant_and_gemm_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "gemm_mx.npz"))
    f8 = lambda a: torch.from_numpy(a).view(torch.float8_e4m3fn)
    a, b, sa, sb = f8(z["a8"]), f8(z["b8"]), torch.from_numpy(z["sa"]), torch.from_numpy(z["sb"])
    assert np.array_equal(R.mx_dequant(a, sa).numpy(), z["deq_a"])
    assert np.array_equal(R.gemm_reference(a, b, a_scale_mx=sa).numpy(), z["want_a"])
    assert np.array_equal(R.gemm_reference(a, b, a_scale_mx=sa, b_scale_mx=sb).numpy(), z["want_ab"])


# ---- quantiser: known answers worked out by hand from the PTX of mx_scale --------------------------------------
# e = clamp(((A + 0x1fffff) >> 23) - 8, 0, 254): a block whose amax has mantissa <= 1.75 gets e = exp(A) - 8 + 127,
# otherwise one more; the scaled peak then lies in (224, 448].
KNOWN = [
    # (block amax, expected scale byte, expected peak code)
    (448.0, 127, 0x7E),        # 1.75 * 2^8 -> scale 1, code 448
    (1.0, 119, 0x78),          # 1.0 * 2^0 -> scale 2^-8, 256 = 0x78
    (1.75, 119, 0x7E),         # threshold mantissa maps to 448
    (1.7500001, 120, 0x76),    # just above: next power of two, 224.00002 -> 224 = 0x76
    (3.0, 120, 0x7C),          # 1.5 * 2^1 -> scale 2^-7, 384 = 0x7c
    (2.0**-126, 0, 0x40),      # smallest normal: e clamps at 0, inv = 2^127 -> 2.0 = 0x40
    (0.0, 0, 0x00),
]


@pytest.mark.parametrize("amax,scale,code", KNOWN)
@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_quantizer_known_answers(amax, scale, code, impl):
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 5] = -np.float32(amax)
    x[0, 6] = np.float32(amax) / 4
    q, s = R.quantize_mx(x) if impl == "numpy" else c_oracle.quantize_mx(x)
    assert int(s[0, 0]) == scale
    assert int(q[0, 5]) == (code | 0x80 if amax else 0x80)
    if amax and scale:
        assert R.e4m3_decode(q)[0, 6] == pytest.approx(-R.e4m3_decode(q)[0, 5] / 4, rel=0.07)


def test_quantizer_smallest_normal_arithmetic():
    # 2^-126 with e = 0: inv = 2^127, scaled = 2.0 -> e4m3 2.0 = 0x40
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 0] = 2.0**-126
    q, s = R.quantize_mx(x)
    assert int(s[0, 0]) == 0 and int(q[0, 0]) == 0x40


def test_quantizer_reference_properties_and_cross_check():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((256, 512)) * np.exp2(rng.integers(-30, 30, (256, 1)))).astype(np.float32)
    q, s = R.quantize_mx(x)
    qc, sc = c_oracle.quantize_mx(x, threads=3)
    assert np.array_equal(q, qc) and np.array_equal(s, sc)
    deq = R.mx_dequant(torch.from_numpy(q).view(torch.float8_e4m3fn), torch.from_numpy(s))
    assert R.rel_l2(deq, torch.from_numpy(x)) <= 4e-2  # tests/gemm/test_gemm.py:171
    peak = np.abs(R.e4m3_decode(q)).reshape(256, 16, 32).max(-1)
    assert ((peak >= 224) & (peak <= 448)).all()  # tests/gemm/test_gemm.py:172-175
    # bf16 inputs: identical to quantising their exact fp32 values
    xb = torch.from_numpy(x).bfloat16()
    qb, sb = c_oracle.quantize_mx(xb.view(torch.int16).numpy().view(np.uint16), threads=2)
    q2, s2 = R.quantize_mx(xb.float().numpy())
    assert np.array_equal(qb, q2) and np.array_equal(sb, s2)


def test_e4m3_codec_matches_torch_cast():
    codes = np.arange(256, dtype=np.uint8)
    vals = R.e4m3_decode(codes)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(vals, nan=1e9), np.nan_to_num(want, nan=1e9))
    rng = np.random.default_rng(3)
    x = np.clip(rng.standard_normal(200000) * np.exp2(rng.uniform(-12, 9, 200000)), -448, 448).astype(np.float32)
    assert np.array_equal(R.e4m3_encode_rne_sat(x), torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    ties = np.array([0.5 * (vals[i] + vals[i + 1]) for i in range(126)], dtype=np.float32)
    assert np.array_equal(R.e4m3_encode_rne_sat(ties), torch.from_numpy(ties).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    # saturation (the PTX conversion saturates where torch's cast gives NaN)
    assert list(R.e4m3_encode_rne_sat(np.array([1e9, -1e9, 465.0], dtype=np.float32))) == [0x7E, 0xFE, 0x7E]
