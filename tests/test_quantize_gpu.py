"""GPU: the MXFP8 quantiser kernel is bit-exact against the CPU oracle (codes and scales)."""

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import reference_math as R

pytestmark = pytest.mark.gpu


def _check(x_gpu):
    from warpy_kernels import quantize_mx

    q, s = quantize_mx(x_gpu)
    torch.cuda.synchronize()
    host = x_gpu.cpu()
    if host.dtype == torch.bfloat16:
        want_q, want_s = c_oracle.quantize_mx(host.contiguous().view(torch.int16).numpy().view(np.uint16), threads=4)
    else:
        want_q, want_s = c_oracle.quantize_mx(host.contiguous().numpy(), threads=4)
    assert np.array_equal(s.cpu().numpy(), want_s), "scale bytes differ"
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), want_q), "e4m3 codes differ"
    return q, s


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 32), (3, 96), (128, 4096), (1000, 224), (257, 14336)])
def test_bit_exact_random(cuda, dtype, shape):
    g = torch.Generator(device=cuda).manual_seed(0)
    x = torch.randn(*shape, device=cuda, generator=g)
    x = x * torch.exp2(torch.randint(-20, 20, (shape[0], 1), device=cuda, generator=g).float())
    _check(x.to(dtype))


def test_small_oracle_numpy_agrees(cuda):
    from warpy_kernels import quantize_mx

    g = torch.Generator(device=cuda).manual_seed(1)
    x = torch.randn(64, 256, device=cuda, generator=g)
    q, s = quantize_mx(x)
    wq, ws = R.quantize_mx(x.cpu().numpy())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq) and np.array_equal(s.cpu().numpy(), ws)


def test_edge_values(cuda):
    x = torch.zeros(8, 64, device=cuda)
    x[1, 0] = 448.0
    x[2, 3] = 1.75
    x[3, 3] = 1.7500001
    x[4, 40] = -3.0e38
    x[5, 1] = 2.0**-126
    x[6, :32] = 1e-30
    x[7, 33] = -0.0
    q, s = _check(x)
    assert int(s[0, 0]) == 0 and int(q.view(torch.uint8)[0].max()) == 0  # all-zero block


def test_strided_rows(cuda):
    from warpy_kernels import quantize_mx

    g = torch.Generator(device=cuda).manual_seed(2)
    full = torch.randn(64, 512, device=cuda, generator=g).bfloat16()
    view = full[:, 128:384]
    q, s = quantize_mx(view)
    q2, s2 = quantize_mx(view.contiguous())
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)


def test_reference_properties_at_full_size(cuda):
    """The reference test's two properties (``tests/gemm/test_gemm.py:171-175``) at a benchmark shape."""
    from warpy_kernels import quantize_mx

    g = torch.Generator(device=cuda).manual_seed(0)
    x = torch.randn(8192, 4096, device=cuda, generator=g).bfloat16()
    q, s = quantize_mx(x)
    deq = q.float() * torch.exp2(s.float() - 127).repeat_interleave(32, dim=1)
    assert R.rel_l2(deq, x.float()) <= 4e-2
    peak = q.float().abs().view(8192, 128, 32).amax(-1)
    assert bool(((peak >= 224) & (peak <= 448)).all())
    # fixed point: quantising the dequantised tensor reproduces the same values (a block whose peak code is
    # exactly 224 moves to the next smaller scale with doubled codes, so compare values, not bytes)
    q2, s2 = quantize_mx(deq)
    deq2 = q2.float() * torch.exp2(s2.float() - 127).repeat_interleave(32, dim=1)
    assert torch.equal(deq2, deq)


def test_rejects_bad_shapes(cuda):
    from warpy_kernels import quantize_mx

    with pytest.raises(ValueError):
        quantize_mx(torch.zeros(4, 48, device=cuda))
    with pytest.raises(ValueError):
        quantize_mx(torch.zeros(4, 64, device=cuda, dtype=torch.float16))
