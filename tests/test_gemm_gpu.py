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
    # north-star tolerance 1e-2 (relative Frobenius vs fp32 accumulation); reference's matches_cublas gate is 1e-3
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
