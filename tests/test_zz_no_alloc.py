"""GPU: the no-allocation MXFP8 GEMM entry point against the regular one.

``wk_gemm_mxfp8_noalloc`` is for callers that may not allocate device memory (a process whose GPU memory is fully
reserved by its host framework, or a latency path where ``cudaMalloc`` is off limits): it keeps its scratch in an
array built into the library.  The test drives it through the C ABI exactly as such a caller would -- plain
pointers, no workspace -- twice in a row with different operands, so the second call runs on top of the first
call's leftovers in the shared array, and requires results bit-identical to ``wk_gemm_mxfp8``.

This file sorts last on purpose: a ``-x`` run reaches it only after every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn


def _args(a, b, sa, sb, out, q=None, s=None, workspace=None):
    from warpy_kernels_b200.gemm.api import _MxArgs

    x = _MxArgs()
    x.a, x.b, x.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    x.a_scale_mx = sa.data_ptr() if sa is not None else None
    x.b_scale_mx = sb.data_ptr() if sb is not None else None
    x.scale_a = x.scale_b = None
    x.q_mx = q.data_ptr() if q is not None else None
    x.s_mx = s.data_ptr() if s is not None else None
    if workspace is not None:
        x.workspace, x.workspace_bytes = workspace.data_ptr(), workspace.numel()
    else:
        x.workspace, x.workspace_bytes = None, 0
    x.m, x.n, x.k = a.shape[0], b.shape[0], a.shape[1]
    return x


def _problem(cuda, m, n, k, seed, with_b_scales):
    g = torch.Generator(device=cuda).manual_seed(seed)
    a = torch.randn(m, k, device=cuda, generator=g).to(FP8)
    b = torch.randn(n, k, device=cuda, generator=g).to(FP8)
    sa = torch.randint(118, 136, (m, k // 32), device=cuda, generator=g, dtype=torch.uint8)
    sb = torch.randint(120, 134, (n, k // 32), device=cuda, generator=g, dtype=torch.uint8) if with_b_scales else None
    return a, b, sa, sb


def test_noalloc_matches_regular_entry_point_twice(cuda):
    from warpy_kernels_b200 import _lib

    lib = _lib.lib()
    stream = _lib.stream_ptr(cuda)
    # two different problems back to back: the second one is smaller and has no B scales, so stale bytes of the
    # first call sit both inside and beyond the region it uses
    for m, n, k, seed, with_b in ((512, 768, 1024, 0, True), (256, 384, 512, 1, False)):
        a, b, sa, sb = _problem(cuda, m, n, k, seed, with_b)
        ws = torch.empty(lib.wk_gemm_mxfp8_workspace_bytes(m, n, k), dtype=torch.uint8, device=cuda)
        want, want_q = torch.empty(m, n, dtype=torch.bfloat16, device=cuda), torch.empty(m, n, dtype=torch.uint8, device=cuda)
        want_s = torch.empty(m, n // 32, dtype=torch.uint8, device=cuda)
        assert lib.wk_gemm_mxfp8(ctypes.byref(_args(a, b, sa, sb, want, want_q, want_s, ws)), stream) == 0
        # outputs pre-filled with a pattern so an entry point that silently did nothing cannot pass
        got = torch.full((m, n), -7.0, dtype=torch.bfloat16, device=cuda)
        got_q = torch.full((m, n), 0x55, dtype=torch.uint8, device=cuda)
        got_s = torch.full((m, n // 32), 0x55, dtype=torch.uint8, device=cuda)
        # Lazy module loading may take device memory the first time a kernel runs: warm the entry point up on
        # throw-away outputs, then watch the driver's own count of free device memory (it sees a cudaMalloc made
        # inside the library, which torch's allocator statistics cannot) around the call that is checked.
        tmp = [torch.empty_like(t) for t in (got, got_q, got_s)]
        assert lib.wk_gemm_mxfp8_noalloc(ctypes.byref(_args(a, b, sa, sb, *tmp)), stream) == 0
        torch.cuda.synchronize(cuda)
        before = torch.cuda.memory_allocated(cuda)
        free_before = torch.cuda.mem_get_info(cuda)[0]
        assert lib.wk_gemm_mxfp8_noalloc(ctypes.byref(_args(a, b, sa, sb, got, got_q, got_s)), stream) == 0
        assert lib.wk_gemm_mxfp8_noalloc_status() == 0
        assert torch.cuda.mem_get_info(cuda)[0] == free_before
        assert torch.cuda.memory_allocated(cuda) == before
        assert torch.equal(got, want) and torch.equal(got_q, want_q) and torch.equal(got_s, want_s)


def test_noalloc_rejects_problems_beyond_its_scratch(cuda):
    from warpy_kernels_b200 import _lib

    lib = _lib.lib()
    limit = lib.wk_gemm_mxfp8_noalloc_max_bytes()
    assert limit == 8 << 20
    # (M + N) * K / 32 just over the limit; nothing is launched, so small dummy buffers are enough
    m, n, k = 128 * 1024, 128 * 1024, 1152
    assert (m + n) * (k // 32) + 32 > limit
    dummy = torch.zeros(256, device=cuda, dtype=torch.uint8)
    x = _args(dummy.view(1, 256), dummy.view(1, 256), None, None, dummy)
    x.m, x.n, x.k = m, n, k
    code = lib.wk_gemm_mxfp8_noalloc(ctypes.byref(x), _lib.stream_ptr(cuda))
    assert code == -4
    assert b"too large" in lib.wk_error_string(code)
