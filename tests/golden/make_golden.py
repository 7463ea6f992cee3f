"""Generate the golden fixtures in this directory from the REFERENCE's own test oracle.

Run in a container that has the reference checkout (its path in the ``WARPY_REFERENCE``
environment variable)::

    python tests/golden/make_golden.py

The reference's GPU kernels cannot run here, but its oracle is plain torch: ``tests/fixtures.py`` (``reference``,
``quantize_qkv``, ``dequantize_qkv``, ``rel_l2``, ``row_p99``) and ``tests/gemm/test_gemm.py`` (``_mx_dequant``).  This
script imports those files unmodified (``import warpy_kernels`` inside them resolves to this repository's alias
package), evaluates them on seeded CPU inputs and stores inputs and outputs as ``.npz``.  ``tests/test_oracle.py``
replays the fixtures against ``oracle/reference_math.py``; the GPU tests compare the kernels with the same files.
"""

import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("WARPY_REFERENCE")  # checkout of the reference repository (tan0210/warpy-kernels)
if not REF or not os.path.isdir(os.path.join(REF, "tests")):
    raise SystemExit("set WARPY_REFERENCE to a checkout of the reference repository (its tests/fixtures.py is imported)")


def _load_reference_tests():
    sys.path.insert(0, REPO)  # `import warpy_kernels` -> this repository's alias package
    pkg = types.ModuleType("tests")
    pkg.__path__ = [os.path.join(REF, "tests")]
    sys.modules["tests"] = pkg
    mods = {}
    for name in ("registry", "fixtures"):
        spec = importlib.util.spec_from_file_location(f"tests.{name}", os.path.join(REF, "tests", f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"tests.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    # test_gemm.py needs the reference's JIT package at import time; take only the function we need, by source
    src = open(os.path.join(REF, "tests", "gemm", "test_gemm.py")).read()
    start = src.index("def _mx_dequant")
    end = src.index("\n\n", start)
    ns = {"torch": torch}
    exec(compile(src[start:end], "test_gemm.py:_mx_dequant", "exec"), ns)
    return mods["fixtures"], ns["_mx_dequant"]


def _u8(x):
    return x.view(torch.uint8).numpy()


ATTN_CASES = {
    # name: (B, Hq, Hkv, Nq, Nk, d, causal, seed)
    "attn_mha_causal": (1, 2, 2, 256, 256, 128, True, 0),
    "attn_gqa_ragged_causal": (1, 4, 2, 200, 333, 128, True, 1),
    "attn_gqa_noncausal": (2, 4, 1, 128, 192, 128, False, 2),
    "attn_short_q_causal": (1, 2, 1, 300, 100, 128, True, 3),  # rows without a visible key
}


def make_attention(fx):
    for name, (B, Hq, Hkv, Nq, Nk, d, causal, seed) in ATTN_CASES.items():
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, Hq, Nq, d, generator=g)
        k = torch.randn(B, Hkv, Nk, d, generator=g)
        v = torch.randn(B, Hkv, Nk, d, generator=g)
        k = k - k.mean(dim=2, keepdim=True)  # as tests/fixtures.py:72-78 (randn_qkv)
        v = v - v.mean(dim=2, keepdim=True)
        dout = torch.randn(B, Hq, Nq, d, generator=torch.Generator().manual_seed(7)).bfloat16()
        q8, k8, v8, sq, sk, sv = fx.quantize_qkv(q, k, v)
        qd, kd, vd = [x.requires_grad_() for x in fx.dequantize_qkv(q8, k8, v8, sq, sk, sv)]
        out, lse = fx.reference(qd, kd, vd, causal)
        out.backward(dout.float())
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"),
            shape=np.array([B, Hq, Hkv, Nq, Nk, d, int(causal), seed]),
            q8=_u8(q8), k8=_u8(k8), v8=_u8(v8),
            sq=sq.numpy(), sk=sk.numpy(), sv=sv.numpy(),
            dout_bf16=dout.view(torch.int16).numpy(),
            out=out.detach().numpy().astype(np.float16),  # |out| < 8 here; fp16 keeps 11 bits, far below tolerances
            lse=lse.detach().numpy(),
            dq=qd.grad.numpy().astype(np.float32), dk=kd.grad.numpy().astype(np.float32),
            dv=vd.grad.numpy().astype(np.float32),
            q_f32_head=q[0, 0, :4].numpy(), k_f32_head=k[0, 0, :4].numpy(),
        )
        print(name, "out", tuple(out.shape))


def make_metrics(fx):
    g = torch.Generator().manual_seed(11)
    a = torch.randn(64, 96, generator=g)
    b = a + 0.01 * torch.randn(64, 96, generator=g)
    np.savez_compressed(
        os.path.join(HERE, "metrics.npz"), a=a.numpy(), b=b.numpy(),
        rel_l2=np.float64(fx.rel_l2(a, b)), row_p99=np.float64(fx.row_p99(a, b)),
    )


def make_mx_dequant(mx_dequant):
    g = torch.Generator().manual_seed(5)
    m, n, k = 128, 128, 256
    a = torch.randn(m, k, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, generator=g).to(torch.float8_e4m3fn)
    sa = torch.randint(118, 136, (m, k // 32), generator=g, dtype=torch.uint8)  # as tests/gemm/test_gemm.py:199-201
    sb = torch.randint(120, 134, (n, k // 32), generator=g, dtype=torch.uint8)
    want_a = mx_dequant(a, sa) @ b.float().T  # the reference's mx_input product, tests/gemm/test_gemm.py:203
    want_ab = mx_dequant(a, sa) @ mx_dequant(b, sb).T
    np.savez_compressed(
        os.path.join(HERE, "gemm_mx.npz"), a8=_u8(a), b8=_u8(b), sa=sa.numpy(), sb=sb.numpy(),
        deq_a=mx_dequant(a, sa).numpy(), want_a=want_a.numpy(), want_ab=want_ab.numpy(),
    )


if __name__ == "__main__":
    torch.set_num_threads(8)
    fixtures, mx_dequant = _load_reference_tests()
    make_attention(fixtures)
    make_metrics(fixtures)
    make_mx_dequant(mx_dequant)
    print("golden fixtures written to", HERE)
