"""GPU: GEMM kernels against the fp32 oracle (``tests/gemm/test_gemm.py:73,203,239`` of the reference)."""

import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu

# the reference's shapes (tests/gemm/test_gemm.py:42) plus the benchmark shape and tiling edge cases
BF16_SHAPES = [(256, 512, 1024), (4096, 4096, 2048), (2048, 2048, 2048), (128, 128, 64), (384, 640, 192)]


@pytest.mark.parametrize("shape", BF16_SHAPES)
def test_bf16_matches_fp32_product(cuda, shape):
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(m, k, device=cuda, generator=g).bfloat16()
    b = torch.randn(n, k, device=cuda, generator=g).bfloat16()
    out = gemm(a, b)
    assert out.dtype == torch.bfloat16 and out.shape == (m, n)
    want = R.gemm_reference(a.cpu(), b.cpu())
    # target tolerance 1e-2 (relative Frobenius vs fp32 accumulation); reference's matches_cublas gate is 1e-3
    # against the bf16-rounded product
    assert R.rel_l2(out.cpu(), want) <= 1e-2
    assert R.rel_l2(out.cpu(), want.bfloat16()) <= 1e-3
    # repeated launches are bit-identical (tests/gemm/test_gemm.py:92-94)
    assert torch.equal(gemm(a, b), out)


def test_bf16_structured_operands(cuda):
    """Operands that expose tile / swizzle / K-step indexing mistakes: each row and column carries its own value."""
    from warpy_kernels import gemm

    m, n, k = 256, 512, 256
    a = torch.zeros(m, k, device=cuda)
    b = torch.zeros(n, k, device=cuda)
    a[torch.arange(m), torch.arange(m) % k] = (torch.arange(m, device=cuda) % 61 + 1).float()
    b[torch.arange(n), (torch.arange(n) * 7) % k] = (torch.arange(n, device=cuda) % 53 + 1).float()
    out = gemm(a.bfloat16(), b.bfloat16())
    want = a @ b.T
    assert torch.equal(out, want.bfloat16())  # single products: exact up to the bf16 rounding of the output


def test_bf16_out_buffer_and_errors(cuda):
    from warpy_kernels import gemm, make_gemm

    a = torch.randn(128, 64, device=cuda).bfloat16()
    b = torch.randn(128, 64, device=cuda).bfloat16()
    buf = torch.empty(128, 128, device=cuda, dtype=torch.bfloat16)
    assert gemm(a, b, out=buf) is buf
    launch, out = make_gemm(a, b)
    launch()
    assert torch.equal(out, buf)
    with pytest.raises(ValueError):
        gemm(a[:100], b)  # M not a multiple of 128
    with pytest.raises(ValueError):
        gemm(a, b[:, :32])  # inner dimensions differ
    with pytest.raises(ValueError):
        gemm(a.t(), b.t())  # not contiguous
    with pytest.raises(ValueError):
        gemm(a, b, out=torch.empty(128, 64, device=cuda, dtype=torch.bfloat16))


# ---- fp8 / MXFP8 --------------------------------------------------------------------------------------------
FP8 = torch.float8_e4m3fn
FP8_SHAPES = [(256, 512, 1024), (4096, 4096, 2048), (128, 128, 128), (384, 640, 384)]


@pytest.mark.parametrize("shape", FP8_SHAPES)
def test_fp8_unit_scales_match_fp32_product(cuda, shape):
    """Plain e4m3 inputs (no MX scales): the reference's ``matches_cublas`` for fp8 (``tests/gemm/test_gemm.py:214-241``)."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    b = torch.randn(n, k, device=cuda, generator=g).to(FP8)
    out = gemm(a, b)
    want = R.gemm_reference(a.cpu(), b.cpu())
    assert R.rel_l2(out.cpu(), want.bfloat16()) <= 1e-3
    assert torch.equal(gemm(a, b), out)


@pytest.mark.parametrize("shape", FP8_SHAPES)
def test_mx_input_random_scale_bytes(cuda, shape):
    """Random scale bytes 118..135 on A plus a scalar on B (``tests/gemm/test_gemm.py:192-205``), then on both."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    b = torch.randn(n, k, device=cuda, generator=g).to(FP8)
    sa = torch.randint(118, 136, (m, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    beta = torch.tensor([0.75], device=cuda)
    got = gemm(a, b, a_scale_mx=sa, scale_b=beta)
    want = R.gemm_reference(a.cpu(), b.cpu(), a_scale_mx=sa.cpu(), alpha=0.75)
    assert R.rel_l2(got.cpu(), want) <= 1e-2
    got2 = gemm(a, b, a_scale_mx=sa, b_scale_mx=sb)
    want2 = R.gemm_reference(a.cpu(), b.cpu(), a_scale_mx=sa.cpu(), b_scale_mx=sb.cpu())
    assert R.rel_l2(got2.cpu(), want2) <= 1e-2
    assert R.rel_l2(got2.cpu(), want2.bfloat16()) <= 1e-3


def test_mx_golden_fixture(cuda, golden_dir):
    import os

    import numpy as np

    from warpy_kernels import gemm

    z = np.load(os.path.join(golden_dir, "gemm_mx.npz"))
    f8 = lambda x: torch.from_numpy(x).to(cuda).view(FP8)
    a, b = f8(z["a8"]), f8(z["b8"])
    sa, sb = torch.from_numpy(z["sa"]).to(cuda), torch.from_numpy(z["sb"]).to(cuda)
    assert R.rel_l2(gemm(a, b, a_scale_mx=sa).cpu(), torch.from_numpy(z["want_a"]).bfloat16()) <= 1e-3
    assert R.rel_l2(gemm(a, b, a_scale_mx=sa, b_scale_mx=sb).cpu(), torch.from_numpy(z["want_ab"]).bfloat16()) <= 1e-3


def test_mx_scale_layout_is_exact(cuda):
    """Power-of-two data with one distinct scale byte per (row, K block): every output is exact, so any mistake in
    the scale-factor tiling shows up as a wrong integer."""
    from warpy_kernels import gemm

    m, n, k = 256, 384, 512
    a = torch.zeros(m, k, device=cuda)
    b = torch.zeros(n, k, device=cuda)
    kb = k // 32
    # row i of a has a single 1 in K block (i % kb); row j of b has a single 1 at the same position of block (j % kb)
    a[torch.arange(m), (torch.arange(m) % kb) * 32 + 3] = 1.0
    b[torch.arange(n), (torch.arange(n) % kb) * 32 + 3] = 1.0
    sa = (120 + (torch.arange(m, device=cuda)[:, None] * 3 + torch.arange(kb, device=cuda)[None, :] * 5) % 9).to(torch.uint8)
    sb = (124 + (torch.arange(n, device=cuda)[:, None] + torch.arange(kb, device=cuda)[None, :] * 2) % 7).to(torch.uint8)
    got = gemm(a.to(FP8), b.to(FP8), a_scale_mx=sa, b_scale_mx=sb).float()
    want = R.gemm_reference(a.to(FP8).cpu(), b.to(FP8).cpu(), a_scale_mx=sa.cpu(), b_scale_mx=sb.cpu())
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("shape", [(256, 512, 1024), (4096, 4096, 2048)])
def test_mx_output_and_chain(cuda, shape):
    """``out_mx`` (``tests/gemm/test_gemm.py:151-175``) and the MX-out -> MX-in chain (``:206-211``)."""
    import numpy as np

    from oracle import c_oracle
    from warpy_kernels import gemm, quantize_mx

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    b = torch.randn(n, k, device=cuda, generator=g).to(FP8)
    out, q, sc = gemm(a, b, out_mx=True)
    assert R.rel_l2(R.mx_dequant(q, sc), out.float()) <= 4e-2
    peak = q.float().abs().view(m, n // 32, 32).amax(-1)
    assert bool(((peak >= 224) & (peak <= 448)).all()), "block scales are not tight"
    # the epilogue quantiser and the standalone kernel share their arithmetic: on the exact fp32 product of a small
    # integer-valued problem both must give the same bytes as the CPU oracle
    ai = torch.randint(-3, 4, (128, 128), device=cuda, generator=g).float()
    bi = torch.randint(-3, 4, (256, 128), device=cuda, generator=g).float()
    o2, q2, s2 = gemm(ai.to(FP8), bi.to(FP8), out_mx=True)
    exact = ai @ bi.T
    wq, ws = c_oracle.quantize_mx(exact.cpu().numpy())
    assert np.array_equal(q2.view(torch.uint8).cpu().numpy(), wq) and np.array_equal(s2.cpu().numpy(), ws)
    q3, s3 = quantize_mx(exact)
    assert torch.equal(q3.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s3, s2)
    # chain: the MX output of one product is the A operand of the next
    x = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    w2 = torch.randn(n, n, device=cuda, generator=g).to(FP8)
    h, hq, hs = gemm(x, b, out_mx=True)
    y = gemm(hq, w2, a_scale_mx=hs).float()
    assert R.rel_l2(y, h.float() @ w2.float().T) <= 5e-2


def test_fp8_rejects_bad_arguments(cuda):
    from warpy_kernels import gemm

    a = torch.zeros(128, 256, device=cuda).to(FP8)
    b = torch.zeros(128, 256, device=cuda).to(FP8)
    with pytest.raises(ValueError):
        gemm(a, b, a_scale_mx=torch.zeros(128, 4, device=cuda, dtype=torch.uint8))  # wrong scale shape
    with pytest.raises(ValueError):
        gemm(a, b, a_scale_mx=torch.zeros(128, 8, device=cuda))  # wrong dtype
    with pytest.raises(ValueError):
        gemm(a[:, :64].contiguous(), b[:, :64].contiguous())  # K not a multiple of 128
    with pytest.raises(ValueError):
        gemm(a, b, act="relu")
    with pytest.raises(ValueError):
        gemm(a, b, act="dgelu")  # no pre
    with pytest.raises(ValueError):
        gemm(a, b, store_pre=True)  # store_pre without gelu
    with pytest.raises(ValueError):
        gemm(a, b, accum=True)  # no addend
    with pytest.raises(ValueError):
        gemm(a, b, scale_a=torch.ones(7, device=cuda))  # neither 1 nor M entries
    with pytest.raises(ValueError):
        gemm(a, b, b_trans=True)  # transposed operands are for 16-bit inputs


# ---- fused epilogue: scales, accum, GELU and its derivative, fp16 ----------------------------------------------
EPI_SHAPES = [(256, 512, 1024), (4096, 4096, 2048)]


def _dgelu(x):
    return 0.5 * (1 + torch.erf(x * 0.7071067811865476)) + x * torch.exp(-0.5 * x * x) * 0.3989422804014327


def _operands(cuda, kind, m, n, k, g):
    a = torch.randn(m, k, device=cuda, generator=g)
    b = torch.randn(n, k, device=cuda, generator=g)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": FP8}[kind]
    odt = torch.float16 if kind == "fp16" else torch.bfloat16
    return a.to(dt), b.to(dt), odt


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8"])
@pytest.mark.parametrize("shape", EPI_SHAPES)
def test_epilogue_accum_gelu_dgelu(cuda, kind, shape):
    """The reference's ``epilogue`` case (``tests/gemm/test_gemm.py:65-97``), for every input dtype."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b, odt = _operands(cuda, kind, m, n, k, g)
    c0 = torch.randn(m, n, device=cuda, generator=g).to(odt)
    prod = a.float() @ b.float().T
    x = prod + c0.float()
    tol = 1e-2  # the reference's tolerance; bf16 rounding is about 4e-3
    assert R.rel_l2(gemm(a, b).float(), prod) <= tol
    got = gemm(a, b, out=c0.clone(), accum=True)
    assert got.dtype == odt and R.rel_l2(got.float(), x) <= tol
    post, pre = gemm(a, b, out=c0.clone(), accum=True, act="gelu", store_pre=True)
    assert R.rel_l2(post.float(), torch.nn.functional.gelu(x)) <= tol
    assert R.rel_l2(pre.float(), x) <= tol
    assert torch.equal(pre, got)  # pre is the accum result before the activation, rounded the same way
    d = gemm(a, b, out=c0.clone(), act="dgelu", pre=pre, accum=True)
    assert R.rel_l2(d.float(), x * _dgelu(pre.float())) <= tol
    post_only, none = gemm(a, b, act="gelu")
    assert none is None and R.rel_l2(post_only.float(), torch.nn.functional.gelu(prod)) <= tol
    assert torch.equal(gemm(a, b, act="gelu")[0], post_only), "repeated launches differ"


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8"])
@pytest.mark.parametrize("shape", EPI_SHAPES)
def test_vector_scales(cuda, kind, shape):
    """The reference's ``vector_scales`` case (``tests/gemm/test_gemm.py:99-138``)."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b, odt = _operands(cuda, kind, m, n, k, g)
    rows = torch.rand(m, device=cuda, generator=g) * 4 + 0.05
    cols = torch.rand(n, device=cuda, generator=g) * 4 + 0.05
    if kind == "fp16":  # keep |x| well inside the fp16 range
        rows, cols = rows * 0.25, cols * 0.25
    c0 = torch.randn(m, n, device=cuda, generator=g).to(odt)
    prod = (a.float() @ b.float().T) * rows[:, None] * cols
    x = prod + c0.float()
    tol = 1e-2
    assert R.rel_l2(gemm(a, b, scale_a=rows, scale_b=cols).float(), prod) <= tol
    half = torch.full((1,), 0.5, device=cuda)
    got = gemm(a, b, scale_a=rows, scale_b=half).float()
    # a one-element scale on the other side applies to fp8 inputs only (warpy_kernels/gemm/api.py:93-95)
    assert R.rel_l2(got, prod / cols * (0.5 if kind == "fp8" else 1.0)) <= tol
    got = gemm(a, b, scale_b=cols).float()
    assert R.rel_l2(got, prod / rows[:, None]) <= tol
    got = gemm(a, b, out=c0.clone(), accum=True, scale_a=rows, scale_b=cols).float()
    assert R.rel_l2(got, x) <= tol
    post, pre = gemm(a, b, out=c0.clone(), accum=True, scale_a=rows, scale_b=cols, act="gelu", store_pre=True)
    assert R.rel_l2(post.float(), torch.nn.functional.gelu(x)) <= tol
    assert R.rel_l2(pre.float(), x) <= tol


def test_vector_scales_are_exact_per_row_and_column(cuda):
    """Power-of-two scales on an integer product: a scale read from the wrong row or column changes an integer."""
    from warpy_kernels import gemm

    m, n, k = 256, 512, 128
    g = torch.Generator(device=cuda).manual_seed(1)
    ai = torch.randint(-2, 3, (m, k), device=cuda, generator=g).float()
    bi = torch.randint(-2, 3, (n, k), device=cuda, generator=g).float()
    rows = torch.exp2((torch.arange(m, device=cuda) % 5).float() - 2)
    cols = torch.exp2((torch.arange(n, device=cuda) % 7).float() - 3)
    want = ((ai @ bi.T) * rows[:, None] * cols).bfloat16()
    for dt in (torch.bfloat16, FP8):
        assert torch.equal(gemm(ai.to(dt), bi.to(dt), scale_a=rows, scale_b=cols), want)
    # a column-scale vector that is 8- but not 16-byte aligned
    buf = torch.zeros(n + 2, device=cuda)
    buf[2:] = cols
    assert torch.equal(gemm(ai.bfloat16(), bi.bfloat16(), scale_a=rows, scale_b=buf[2:]), want)


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
@pytest.mark.parametrize("shape", EPI_SHAPES)
def test_mx_output_after_gelu(cuda, kind, shape):
    """MXFP8 output of the activated value, for 16-bit inputs too (``tests/gemm/test_gemm.py:151-190``)."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b, odt = _operands(cuda, kind, m, n, k, g)
    c0 = torch.randn(m, n, device=cuda, generator=g).to(odt)
    out, q, sc = gemm(a, b, out_mx=True)
    assert R.rel_l2(R.mx_dequant(q, sc), out.float()) <= 4e-2
    peak = q.float().abs().view(m, n // 32, 32).amax(-1)
    assert bool(((peak >= 224) & (peak <= 448)).all()), "block scales are not tight"
    post, pre, q, sc = gemm(a, b, out=c0.clone(), accum=True, act="gelu", store_pre=True, out_mx=True)
    assert R.rel_l2(R.mx_dequant(q, sc), post.float()) <= 4e-2
    assert R.rel_l2(pre.float(), a.float() @ b.float().T + c0.float()) <= 1e-2


def test_fp16_matches_fp32_product(cuda):
    from warpy_kernels import gemm

    g = torch.Generator(device=cuda).manual_seed(0)
    a = torch.randn(384, 192, device=cuda, generator=g).half()
    b = torch.randn(640, 192, device=cuda, generator=g).half()
    out = gemm(a, b)
    assert out.dtype == torch.float16
    want = R.gemm_reference(a.cpu(), b.cpu())
    assert R.rel_l2(out.cpu(), want.half()) <= 1e-3
    with pytest.raises(ValueError):
        gemm(a, b, out=torch.empty(384, 640, device=cuda, dtype=torch.bfloat16))
    # fp8 inputs with an fp16 output
    a8, b8 = a.to(FP8), b.to(FP8)
    a8, b8 = a8[:, :128].contiguous(), b8[:, :128].contiguous()
    o16 = gemm(a8, b8, out_dtype=torch.float16)
    assert o16.dtype == torch.float16
    assert R.rel_l2(o16.cpu(), R.gemm_reference(a8.cpu(), b8.cpu()).half()) <= 1e-3


@pytest.mark.parametrize("kind", ["bf16", "fp16"])
@pytest.mark.parametrize("trans", [(True, False), (False, True), (True, True)])
def test_transposed_operands(cuda, kind, trans):
    """``a_trans`` / ``b_trans`` (``tests/gemm/test_gemm.py:83-91``): operands stored ``[K, M]`` / ``[K, N]``."""
    from warpy_kernels import gemm

    a_trans, b_trans = trans
    m, n, k = 384, 640, 192
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b, odt = _operands(cuda, kind, m, n, k, g)
    at = a.T.contiguous() if a_trans else a
    bt = b.T.contiguous() if b_trans else b
    got = gemm(at, bt, a_trans=a_trans, b_trans=b_trans)
    assert got.shape == (m, n) and got.dtype == odt
    # same products in the same order as the plain layout: bit-identical
    assert torch.equal(got, gemm(a, b))
    assert R.rel_l2(got.float(), a.float() @ b.float().T) <= 1e-2


def test_transposed_structured_operands(cuda):
    """One distinct value per row and column, transposed storage: exposes MN-major tile indexing mistakes."""
    from warpy_kernels import gemm

    m, n, k = 256, 512, 256
    a = torch.zeros(m, k, device=cuda)
    b = torch.zeros(n, k, device=cuda)
    a[torch.arange(m), torch.arange(m) % k] = (torch.arange(m, device=cuda) % 61 + 1).float()
    b[torch.arange(n), (torch.arange(n) * 7) % k] = (torch.arange(n, device=cuda) % 53 + 1).float()
    want = (a @ b.T).bfloat16()
    a16, b16 = a.bfloat16(), b.bfloat16()
    assert torch.equal(gemm(a16.T.contiguous(), b16, a_trans=True), want)
    assert torch.equal(gemm(a16, b16.T.contiguous(), b_trans=True), want)
    assert torch.equal(gemm(a16.T.contiguous(), b16.T.contiguous(), a_trans=True, b_trans=True), want)
    # the reference's backward use: dgelu with a transposed weight (tests/gemm/test_gemm.py:88-91)
    g = torch.Generator(device=cuda).manual_seed(2)
    x = torch.randn(256, 128, device=cuda, generator=g).bfloat16()
    w = torch.randn(512, 128, device=cuda, generator=g).bfloat16()
    c0 = torch.randn(256, 512, device=cuda, generator=g).bfloat16()
    post, pre = gemm(x, w, out=c0.clone(), accum=True, act="gelu", store_pre=True)
    d = gemm(x, w.T.contiguous(), out=c0.clone(), act="dgelu", pre=pre, accum=True, b_trans=True)
    assert torch.equal(d, gemm(x, w, out=c0.clone(), act="dgelu", pre=pre, accum=True))


@pytest.mark.parametrize("kind", ["bf16", "fp16"])
@pytest.mark.parametrize("shape", [(256, 256, 128), (128, 128, 64), (384, 640, 192), (512, 768, 384),
                                   (4096, 4096, 2048), (2176, 4224, 576)])
def test_cta_pair_kernel_matches_single_cta_kernel(cuda, kind, shape):
    """``cta_pair=True``: two SMs per 256 x 256 tile (tcgen05 ``cta_group::2``).  Same products in the same order as
    the single-CTA kernel, so the results are bit-identical; the fused epilogue goes through it as well.  Tiles that
    hang over the edge of M or N by 128 (one CTA of the pair, or half the columns of both) store nothing there."""
    from warpy_kernels import gemm

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b, odt = _operands(cuda, kind, m, n, k, g)
    guard = torch.full((m + 128, n), 7.0, device=cuda, dtype=odt)  # rows past M must stay untouched
    out = gemm(a, b, out=guard[:m], cta_pair=True)
    assert torch.equal(out, gemm(a, b, cta_pair=False))
    assert torch.equal(out, gemm(a, b))  # the library's own choice
    assert bool((guard[m:] == 7.0).all())
    assert R.rel_l2(out.float(), a.float() @ b.float().T) <= 1e-2
    rows = torch.rand(m, device=cuda, generator=g) + 0.5
    c0 = torch.randn(m, n, device=cuda, generator=g).to(odt)
    post, pre = gemm(a, b, out=c0.clone(), scale_a=rows, accum=True, act="gelu", store_pre=True, cta_pair=True)
    post1, pre1 = gemm(a, b, out=c0.clone(), scale_a=rows, accum=True, act="gelu", store_pre=True, cta_pair=False)
    assert torch.equal(post, post1) and torch.equal(pre, pre1)
    # transposed operands (MN-major tiles) through both kernels
    at, bt = a.T.contiguous(), b.T.contiguous()
    for kw in (dict(a_trans=True), dict(b_trans=True), dict(a_trans=True, b_trans=True)):
        x = at if kw.get("a_trans") else a
        y = bt if kw.get("b_trans") else b
        assert torch.equal(gemm(x, y, cta_pair=True, **kw), out), kw
        assert torch.equal(gemm(x, y, cta_pair=False, **kw), out), kw


@pytest.mark.parametrize("shape", [(256, 256, 128), (128, 128, 128), (384, 640, 384), (4096, 4096, 2048),
                                   (2176, 4224, 640)])
def test_mx_cta_pair_kernel_matches_single_cta_kernel(cuda, shape):
    """MXFP8 on CTA pairs (``cta_pair=True``): each CTA of a pair holds the scale factors of its own rows of ``a`` and
    of all 256 columns of the tile.  Bit-identical to the single-CTA kernel, fused epilogue and MX output included;
    tiles that hang over the edge of M or N by 128 store nothing there."""
    from warpy_kernels import gemm, quantize_mx

    m, n, k = shape
    g = torch.Generator(device=cuda).manual_seed(0)
    a8, sa = quantize_mx(torch.randn(m, k, device=cuda, generator=g).bfloat16() * 3)
    b8, sb = quantize_mx(torch.randn(n, k, device=cuda, generator=g).bfloat16() * 0.2)
    guard = torch.full((m + 128, n), 7.0, device=cuda, dtype=torch.bfloat16)
    out = gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb, out=guard[:m], cta_pair=True)
    assert torch.equal(out, gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb, cta_pair=False))
    assert torch.equal(out, gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb))
    assert bool((guard[m:] == 7.0).all())
    assert R.rel_l2(out.float(), R.mx_dequant(a8, sa) @ R.mx_dequant(b8, sb).T) <= 1e-2
    rows = torch.rand(m, device=cuda, generator=g) + 0.5
    c0 = torch.randn(m, n, device=cuda, generator=g).bfloat16()
    kw = dict(a_scale_mx=sa, scale_a=rows, accum=True, act="gelu", store_pre=True, out_mx=True)
    got = gemm(a8, b8, out=c0.clone(), cta_pair=True, **kw)
    want = gemm(a8, b8, out=c0.clone(), cta_pair=False, **kw)
    assert len(got) == len(want) and all(torch.equal(x.view(torch.uint8), y.view(torch.uint8)) for x, y in zip(got, want))


# ---- accumulator precision of the block-scaled MMA (tests/gemm/test_gemm.py:244-301 of the reference) -------------
def _wide(r, c, gen, device):
    """Magnitudes from e4m3 subnormals to near 448, random signs (``tests/gemm/test_gemm.py:244-249``)."""
    e = torch.rand(r, c, device=device, generator=gen) * 17.8 - 9.0
    s = torch.randint(0, 2, (r, c), device=device, generator=gen) * 2 - 1
    return s * torch.exp2(e)


def _fp8_inputs(kind, m, n, k, device):
    gen = torch.Generator(device=device).manual_seed(0)
    if kind == "normal":
        a, b = torch.randn(m, k, device=device, generator=gen), torch.randn(n, k, device=device, generator=gen)
    elif kind == "wide":
        a, b = _wide(m, k, gen, device), _wide(n, k, gen, device)
    else:  # "cancel": the exact results are 0
        a = torch.randn(m, k // 2, device=device, generator=gen) * 16
        b = torch.randn(n, k // 2, device=device, generator=gen) * 16
        a, b = torch.cat([a, -a], 1), torch.cat([b, b], 1)
    return a.to(FP8), b.to(FP8)


@pytest.mark.parametrize("cta_pair", [False, True])
@pytest.mark.parametrize("kind", ["normal", "wide", "cancel"])
def test_fp8_block_scaled_mma_accumulator(cuda, kind, cta_pair):
    """The reference's ``fp8_block_scaled_mma`` case for the tcgen05 ``kind::mxf8f6f4`` path of both MXFP8 kernels.

    Subtracting ``bf16(ref)`` through ``accum=True`` leaves the low accumulator bits in the bf16 output; the residual
    against a float64 product must stay within ``K / 32`` units of ``2^-21 . (|a| @ |b|^T)``, the reference's bound for
    a truncating 22-bit accumulator.  With MX scale bytes on both operands (powers of two: exact in float64) the same
    bound must hold.  The ``cancel`` inputs, whose exact result is 0, leave only the rounding of the partial sums,
    which the same bound covers (an fp32 accumulator does not return an exact 0 there).
    """
    from warpy_kernels import gemm

    m, n, k = 512, 512, 4096
    a, b = _fp8_inputs(kind, m, n, k, cuda)
    ad, bd = a.double(), b.double()
    ref = ad @ bd.T
    c0 = (-ref).to(torch.bfloat16)
    plain = gemm(a, b, cta_pair=cta_pair)
    resid = gemm(a, b, out=c0.clone(), accum=True, cta_pair=cta_pair)
    assert torch.equal(plain, gemm(a, b, cta_pair=not cta_pair)), "the two MXFP8 kernels differ"
    unit = ((ad.abs() @ bd.abs().T) * 2.0**-21).clamp_min(1e-300)
    err = ((resid.double() - c0.double() - ref).abs() / unit).max().item()
    assert err <= k / 32, f"accumulator error {err} units of 2^-21 (bound {k / 32})"
    if kind == "cancel":
        assert (plain.double().abs() / unit).max().item() <= k / 32, "cancelling product left more than the bound"
    # the same with block scales on both operands
    g = torch.Generator(device=cuda).manual_seed(1)
    sa = torch.randint(120, 134, (m, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    if kind == "cancel":  # keep the two halves of K on equal scales so that the product still cancels
        sa = torch.cat([sa[:, : k // 64], sa[:, : k // 64]], 1).contiguous()
        sb = torch.cat([sb[:, : k // 64], sb[:, : k // 64]], 1).contiguous()
    asd = ad * torch.exp2(sa.double() - 127).repeat_interleave(32, 1)
    bsd = bd * torch.exp2(sb.double() - 127).repeat_interleave(32, 1)
    ref_s = asd @ bsd.T
    c1 = (-ref_s).to(torch.bfloat16)
    resid_s = gemm(a, b, a_scale_mx=sa, b_scale_mx=sb, out=c1.clone(), accum=True, cta_pair=cta_pair)
    unit_s = ((asd.abs() @ bsd.abs().T) * 2.0**-21).clamp_min(1e-300)
    err_s = ((resid_s.double() - c1.double() - ref_s).abs() / unit_s).max().item()
    assert err_s <= k / 32, f"accumulator error {err_s} units with MX scales (bound {k / 32})"
    if kind == "cancel":
        left = gemm(a, b, a_scale_mx=sa, b_scale_mx=sb, cta_pair=cta_pair)
        assert (left.double().abs() / unit_s).max().item() <= k / 32


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_autotune_gemm_times_both_kernels_and_stores_the_winner(cuda, kind, tmp_path, monkeypatch):
    """``autotune_gemm`` times the single-CTA and the CTA-pair kernel, writes the winner into the tune cache and
    ``make_gemm`` picks it up (the reference's tuner: ``warpy_kernels/gemm/api.py:363-390``)."""
    import json

    from warpy_kernels import autotune_gemm, gemm
    from warpy_kernels_b200 import utils

    monkeypatch.setattr(utils, "TUNE_CACHE_PATH", str(tmp_path / "tune.json"))
    m, n, k = 512, 768, 512
    g = torch.Generator(device=cuda).manual_seed(0)
    a, b = torch.randn(m, k, device=cuda, generator=g), torch.randn(n, k, device=cuda, generator=g)
    a, b = (a.to(FP8), b.to(FP8)) if kind == "fp8" else (a.bfloat16(), b.bfloat16())
    best, results = autotune_gemm(a, b, iters=3, verbose=False)
    assert best["cta_pair"] in (False, True) and best["group_m"] in (8, 32) and len(results) == 4
    assert all(isinstance(t, float) for _, t in results)
    key = f"{'gemm_fp8' if kind == 'fp8' else 'gemm'}|m={m}|n={n}|k={k}|sm100"
    assert json.load(open(tmp_path / "tune.json")) == {key: best}
    assert torch.equal(gemm(a, b), gemm(a, b, **best))  # the cache entry is what runs by default
    assert torch.equal(gemm(a, b), gemm(a, b, cta_pair=False, group_m=3))  # any grouping gives the same bits


def test_mx_scales_tiled_once_through_the_c_abi(cuda):
    """``wk_tile_mx_scales`` + ``a_scale_tiled`` / ``b_scale_tiled``: scale tensors that do not change between calls
    (weights) are re-tiled once; with both tiled the GEMM needs no workspace and gives the same bits, on both kernels.
    ``make_gemm`` does this for ``b_scale_mx``: a prepared launch keeps the scales of ``b`` it was made with."""
    import ctypes

    from warpy_kernels import gemm, make_gemm
    from warpy_kernels_b200 import _lib
    from warpy_kernels_b200.gemm.api import _MxArgs

    lib = _lib.lib()
    m, n, k = 384, 640, 512
    g = torch.Generator(device=cuda).manual_seed(4)
    a = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    b = torch.randn(n, k, device=cuda, generator=g).to(FP8)
    sa = torch.randint(118, 136, (m, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    want = gemm(a, b, a_scale_mx=sa, b_scale_mx=sb)
    assert lib.wk_mx_scales_tiled_bytes(m, k) == m * k // 32
    ta = torch.empty(lib.wk_mx_scales_tiled_bytes(m, k), dtype=torch.uint8, device=cuda)
    tb = torch.empty(lib.wk_mx_scales_tiled_bytes(n, k), dtype=torch.uint8, device=cuda)
    stream = _lib.stream_ptr(cuda)
    assert lib.wk_tile_mx_scales(sa.data_ptr(), m, k, ta.data_ptr(), stream) == 0
    assert lib.wk_tile_mx_scales(sb.data_ptr(), n, k, tb.data_ptr(), stream) == 0
    for pair in (2, 1):
        got = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=cuda)
        x = _MxArgs()
        x.a, x.b, x.out = a.data_ptr(), b.data_ptr(), got.data_ptr()
        x.a_scale_mx, x.b_scale_mx, x.a_scale_tiled, x.b_scale_tiled = ta.data_ptr(), tb.data_ptr(), 1, 1
        x.workspace, x.workspace_bytes = None, 0
        x.m, x.n, x.k, x.cta_pair = m, n, k, pair
        assert lib.wk_gemm_mxfp8(ctypes.byref(x), stream) == 0
        assert torch.equal(got, want), pair
    x.a_scale_tiled = 0  # a row-major tensor again, but no workspace to re-tile it into
    assert lib.wk_gemm_mxfp8(ctypes.byref(x), stream) == -1
    # a prepared launch re-reads a's scales at every launch and keeps b's
    sa2, sb2 = sa.clone(), sb.clone()
    launch, out = make_gemm(a, b, a_scale_mx=sa2, b_scale_mx=sb2)
    sa2 += 1
    sb2 += 1
    launch()
    assert torch.equal(out.float(), want.float() * 2)
