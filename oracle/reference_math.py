"""CPU restatement of the reference's torch fp32 oracle and of its MXFP8 quantiser.  TEST INFRASTRUCTURE ONLY.

Pinning
  * ``attention_reference``, ``quantize_qkv``, ``dequantize_qkv``, ``mx_dequant``, ``rel_l2`` and ``row_p99`` restate
    plain-torch functions of the reference's test suite and are pinned against them: ``tests/golden/make_golden.py``
    imports the reference's own ``tests/fixtures.py`` / ``tests/gemm/test_gemm.py`` on CPU, runs them on seeded
    inputs and stores inputs and outputs under ``tests/golden/``; ``tests/test_oracle.py`` replays them.
  * ``quantize_mx`` (numpy) restates arithmetic that exists in the reference only as PTX strings inside GPU kernels
    (no CPU code, no golden vectors, and the package cannot be imported or run here).  PARITY UNPINNED against
    reference outputs; it is pinned instead by (a) known answers derived by hand from the PTX text, (b) the two
    properties the reference's own test asserts (dequantised error <= 4e-2, every block peak in [224, 448];
    ``tests/gemm/test_gemm.py:171-175``) and (c) agreement of its e4m3 rounding with ``torch.Tensor.to(float8_e4m3fn)``
    on all representable inputs.
"""

import math

import numpy as np
import torch

LN2 = math.log(2.0)


# ----------------------------------------------------------------------------------------------------------------
# metrics (reference: tests/fixtures.py:42-55)
# ----------------------------------------------------------------------------------------------------------------
def rel_l2(a, b):
    """Relative Frobenius error of ``a`` against ``b`` (``tests/fixtures.py:42-43``)."""
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def row_p99(a, b):
    """99th percentile over rows of the per-row relative L2 error (``tests/fixtures.py:46-55``)."""
    a, b = a.float().flatten(0, -2), b.float().flatten(0, -2)
    ref = b.norm(dim=1)
    floor = 0.1 * ref.median().clamp_min(1e-30)
    return ((a - b).norm(dim=1) / torch.maximum(ref, floor)).quantile(0.99).item()


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return (a @ b / (a.norm() * b.norm()).clamp_min(1e-300)).item()


def max_abs(a, b):
    return (a.float() - b.float()).abs().max().item()


# ----------------------------------------------------------------------------------------------------------------
# per-(batch, kv head) e4m3 quantisation of q, k, v (reference: tests/fixtures.py:91-120)
# ----------------------------------------------------------------------------------------------------------------
def _quantize(x, group_dims):
    scale = x.abs().amax(dim=group_dims, keepdim=True).clamp_min(1e-12) / 448.0
    return (x / scale).to(torch.float8_e4m3fn), scale


def quantize_qkv(q, k, v):
    """E4M3 ``q, k, v`` with one scale per (batch, kv head); queries share the scale of their kv group.

    Follows ``tests/fixtures.py:91-114``.  Returns ``(q8, k8, v8, q_descale, k_descale, v_descale)``.
    """
    B, Hq, Nq, d = q.shape
    Hkv = k.shape[1]
    q8, sq = _quantize(q.view(B, Hkv, Hq // Hkv, Nq, d), (2, 3, 4))
    k8, sk = _quantize(k, (2, 3))
    v8, sv = _quantize(v, (2, 3))
    return q8.view(B, Hq, Nq, d), k8, v8, sq.view(B, Hkv), sk.view(B, Hkv), sv.view(B, Hkv)


def quantize_per_tensor(x):
    """Per-tensor e4m3 quantisation with ``scale = amax / 448`` (the benchmark configs' input recipe)."""
    scale = x.abs().amax().clamp_min(1e-12) / 448.0
    return (x / scale).to(torch.float8_e4m3fn), scale


def dequantize_qkv(q8, k8, v8, sq, sk, sv):
    """Inverse of ``quantize_qkv`` (``tests/fixtures.py:117-120``)."""
    rep = q8.shape[1] // k8.shape[1]
    q = q8.float() * sq.repeat_interleave(rep, 1)[:, :, None, None]
    return q, k8.float() * sk[:, :, None, None], v8.float() * sv[:, :, None, None]


# ----------------------------------------------------------------------------------------------------------------
# attention (reference: tests/fixtures.py:166-185)
# ----------------------------------------------------------------------------------------------------------------
def attention_reference(q, k, v, causal, softmax_scale=None):
    """fp32 attention with a bottom-right aligned causal mask; differentiable.

    Rows that see no key give ``O = 0`` and ``lse = -inf``.  Follows ``tests/fixtures.py:166-185``; the optional
    ``softmax_scale`` (default ``1 / sqrt(d)``, the only value the reference's oracle has) is an extension.

    Returns:
        ``(out, lse)`` with ``lse`` in base 2.
    """
    _, Hq, Nq, d = q.shape
    Nk = k.shape[2]
    rep = Hq // k.shape[1]
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    s = (q @ k.transpose(-1, -2)) * scale if softmax_scale is not None else (q @ k.transpose(-1, -2)) / math.sqrt(d)
    visible = torch.ones(Nq, dtype=torch.bool, device=q.device)
    if causal:
        row = torch.arange(Nq, device=q.device)[:, None]
        col = torch.arange(Nk, device=q.device)[None, :]
        s = s.masked_fill(col > row + Nk - Nq, -1e30)
        visible = (torch.arange(Nq, device=q.device) + Nk - Nq) >= 0
    out = (torch.softmax(s, dim=-1) @ v) * visible[:, None]
    lse = torch.where(visible, torch.logsumexp(s, dim=-1) / LN2, -math.inf)
    return out, lse


def attention_reference_chunked(q, k, v, causal, softmax_scale=None, dout=None, q_chunk=1024):
    """``attention_reference`` evaluated one (batch, query head, query chunk) at a time.

    Same arithmetic per row; bounded memory so the benchmark shapes fit in host RAM.  With ``dout`` also returns the
    gradients with respect to ``q, k, v`` (autograd through the same function, ``tests/fixtures.py:197-200``).

    Returns:
        ``(out, lse)`` or ``(out, lse, dq, dk, dv)``.
    """
    B, Hq, Nq, d = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    out = torch.empty(B, Hq, Nq, d)
    lse = torch.empty(B, Hq, Nq)
    if dout is not None:
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            g = h // rep
            for r0 in range(0, Nq, q_chunk):
                r1 = min(Nq, r0 + q_chunk)
                # queries r0..r1 with the causal offset preserved: give the chunk the keys it can see plus alignment
                qc = q[b : b + 1, h : h + 1, r0:r1].detach().clone().requires_grad_(dout is not None)
                kc = k[b : b + 1, g : g + 1].detach().clone().requires_grad_(dout is not None)
                vc = v[b : b + 1, g : g + 1].detach().clone().requires_grad_(dout is not None)
                if causal:
                    # row i of the chunk sees keys j <= i + offset; keys past the last row's horizon are dropped
                    offset = r0 + Nk - Nq
                    nk_c = max(0, min(Nk, r1 - 1 + Nk - Nq + 1))
                    if nk_c == 0:
                        out[b, h, r0:r1] = 0
                        lse[b, h, r0:r1] = -math.inf
                        continue
                    o, l = _attn_offset(qc, kc[:, :, :nk_c], vc[:, :, :nk_c], offset, softmax_scale)
                else:
                    o, l = attention_reference(qc, kc, vc, False, softmax_scale)
                out[b, h, r0:r1] = o[0, 0].detach()
                lse[b, h, r0:r1] = l[0, 0].detach()
                if dout is not None:
                    o.backward(dout[b : b + 1, h : h + 1, r0:r1].float())
                    dq[b, h, r0:r1] = qc.grad[0, 0]
                    if kc.grad is not None:
                        dk[b, g] += kc.grad[0, 0]
                        dv[b, g] += vc.grad[0, 0]
    if dout is not None:
        return out, lse, dq, dk, dv
    return out, lse


def _attn_offset(q, k, v, offset, softmax_scale):
    """Attention where query row ``i`` sees keys ``j <= i + offset`` (the general causal chunk)."""
    d = q.shape[-1]
    Nq, Nk = q.shape[2], k.shape[2]
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    s = (q @ k.transpose(-1, -2)) * scale
    row = torch.arange(Nq, device=q.device)[:, None]
    col = torch.arange(Nk, device=q.device)[None, :]
    s = s.masked_fill(col > row + offset, -1e30)
    visible = (torch.arange(Nq, device=q.device) + offset) >= 0
    out = (torch.softmax(s, dim=-1) @ v) * visible[:, None]
    lse = torch.where(visible, torch.logsumexp(s, dim=-1) / LN2, -math.inf)
    return out, lse


# ----------------------------------------------------------------------------------------------------------------
# GEMM (reference: tests/gemm/test_gemm.py:73,147-148,203,239)
# ----------------------------------------------------------------------------------------------------------------
def mx_dequant(q, s):
    """``code * 2^(scale - 127)`` with one scale per 32 columns (``tests/gemm/test_gemm.py:147-148``)."""
    return q.float() * torch.exp2(s.float() - 127).repeat_interleave(32, dim=1)


def gemm_reference(a, b, a_scale_mx=None, b_scale_mx=None, alpha=1.0):
    """fp32 product ``a @ b.T`` of bf16 or (MX-)e4m3 operands (``tests/gemm/test_gemm.py:73,203,239``)."""
    af = mx_dequant(a, a_scale_mx) if a_scale_mx is not None else a.float()
    bf = mx_dequant(b, b_scale_mx) if b_scale_mx is not None else b.float()
    return (af @ bf.T) * alpha


# ----------------------------------------------------------------------------------------------------------------
# MXFP8 quantiser, integer restatement (reference: ptx/common.py:539-565, ptx/sm89.py:85-93, gemm/sm89.py:65-93)
# ----------------------------------------------------------------------------------------------------------------
def e4m3_encode_rne_sat(x):
    """fp32 array -> e4m3 byte codes, round to nearest even, saturating to +-448 (``cvt.rn.satfinite.e4m3x2.f32``).

    Integer arithmetic on the fp32 bit patterns; NaN inputs give 0x7f like the PTX instruction.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    mag = bits & 0x7FFFFFFF
    exp = (mag >> 23).astype(np.int32) - 127
    man = (mag & 0x7FFFFF).astype(np.int64) | 0x800000  # 24-bit significand with the hidden one
    out = np.zeros(x.shape, dtype=np.uint8)
    # normal e4m3 range: exponent >= -6; keep 3 mantissa bits -> drop 20 bits
    # subnormal: value = m * 2^-9, m in 0..7 -> total shift grows as the exponent falls below -6
    shift = np.where(exp >= -6, 20, 20 + (-6 - exp)).astype(np.int64)
    shift = np.minimum(shift, 40)
    q = man >> shift
    rem = man & ((np.int64(1) << shift) - 1)
    half = np.int64(1) << (shift - 1)
    q = q + ((rem > half) | ((rem == half) & ((q & 1) == 1)))
    # q is the significand in units of 2^(max(exp,-6) - 3); rebuild the code
    e_field = np.where(exp >= -6, exp + 7, 0).astype(np.int64)
    code = np.where(exp >= -6, ((e_field - 1) << 3) + q, q)  # q carries the hidden bit (8..16) for normals
    # for normals: q in [8, 16]; ((e_field-1)<<3)+q == (e_field<<3) + (q-8), carrying into the exponent at 16
    code = np.where(mag == 0, 0, code)
    code = np.minimum(code, 0x7E)  # saturate: 0x7e = 448
    nan = mag > 0x7F800000
    code = np.where(nan, 0x7F, code)
    out[...] = code.astype(np.uint8)
    return out | sign


def e4m3_decode(codes):
    """e4m3 byte codes -> fp32 (exact)."""
    c = np.asarray(codes, dtype=np.uint8).astype(np.int32)
    s = np.where(c & 0x80, -1.0, 1.0).astype(np.float32)
    e = (c >> 3) & 0xF
    m = c & 7
    val = np.where(e == 0, m * 2.0**-9, (8 + m) * np.exp2((e - 10).astype(np.float32)))
    val = np.where((c & 0x7F) == 0x7F, np.nan, val)
    return (s * val).astype(np.float32)


def mx_scale_bits(amax_bits):
    """Scale byte ``e`` and multiplier bit pattern for an integer amax (``ptx/common.py:546-565``)."""
    a = amax_bits.astype(np.int64)
    e = np.clip(((a + 0x1FFFFF) >> 23) - 8, 0, 254)
    inv_bits = (np.maximum(254 - e, 1) << 23).astype(np.uint32)
    return e.astype(np.uint8), inv_bits


def quantize_mx(x):
    """MXFP8-quantise the rows of ``x`` (numpy fp32 ``[M, K]``, ``K % 32 == 0``).

    Per row and block of 32 consecutive elements (``gemm/sm89.py:65-93``): integer max of the sign-cleared bit
    patterns, ``mx_scale``, multiply by the power-of-two inverse in fp32, RNE-saturating e4m3 conversion.

    Returns:
        ``(codes uint8 [M, K], scales uint8 [M, K // 32])``.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    blocks = x.reshape(m, k // 32, 32)
    amax = (blocks.view(np.uint32) & 0x7FFFFFFF).max(axis=-1)
    e, inv_bits = mx_scale_bits(amax)
    inv = inv_bits.view(np.float32)[..., None]
    scaled = (blocks * inv).astype(np.float32)
    return e4m3_encode_rne_sat(scaled).reshape(m, k), e
