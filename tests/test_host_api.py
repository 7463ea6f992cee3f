"""CPU: the C-ABI library loads and exports every symbol the header declares; host-side validation mirrors the
reference's error behaviour (``warpy_kernels/gemm/api.py:125-164``, ``warpy_kernels/arch.py:69-116``)."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "warpy_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from warpy_kernels_b200 import _lib

    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 5
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/warpy_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_query_and_error_strings():
    from warpy_kernels_b200 import _lib

    lib = _lib.lib()
    assert lib.wk_query(b"gemm_mx") == 1
    assert lib.wk_query(b"attn_fwd_fp8") == 1
    assert lib.wk_query(b"gemm_gelu") == 1
    assert lib.wk_query(b"attn_fwd") == 1 and lib.wk_query(b"attn_bwd") == 1
    assert lib.wk_query(b"no_such_feature") == -1
    assert b"rejected" in lib.wk_error_string(-1)


def test_import_surface_matches_reference():
    import warpy_kernels
    from warpy_kernels import attn_bwd, attn_fwd, autotune_gemm, device_arch, gemm, make_gemm, supports  # noqa: F401
    import warpy_kernels.attn  # noqa: F401
    from warpy_kernels.utils import time_launch_ms, round_up, check_descale, tune_key  # noqa: F401

    assert set(warpy_kernels.__all__) >= {
        "attn_bwd", "attn_fwd", "autotune_gemm", "device_arch", "gemm", "make_gemm", "supports",
    }


def test_supports_feature_table():
    from warpy_kernels import supports

    assert supports("gemm_mx", 100) and supports("attn_fwd_fp8", 100)
    assert supports("gemm_gelu", 100) and supports("gemm_accum", 100)
    assert supports("attn_fwd", 100) and supports("attn_bwd", 100)
    assert not supports("gemm_mx", 90)  # other architectures are the reference's business
    with pytest.raises(ValueError):
        supports("bogus")
    if not torch.cuda.is_available():
        assert supports("gemm") is False  # no device: False, not an exception (arch.py:69-94)


def test_gemm_rejects_bad_dtypes_before_touching_the_device():
    from warpy_kernels import gemm

    a = torch.zeros(128, 64, dtype=torch.float32)
    with pytest.raises(ValueError):
        gemm(a, a)
    with pytest.raises(ValueError):
        gemm(torch.zeros(128, 64, dtype=torch.bfloat16), torch.zeros(128, 64, dtype=torch.float16))


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("CPU-only check")
    from warpy_kernels import gemm, quantize_mx

    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        gemm(a, a)
    with pytest.raises(NotImplementedError):
        quantize_mx(a)


def test_product_never_imports_the_oracle():
    for pkg in ("warpy_kernels_b200", "warpy_kernels"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, pkg)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".h")):
                    text = open(os.path.join(dirpath, f)).read()
                    assert "oracle" not in text.replace("oracle for", ""), f"{pkg}/{f} mentions the oracle"


def test_tune_cache_uses_the_reference_file_format(tmp_path, monkeypatch):
    """Keys and file layout of the reference's tune cache (``warpy_kernels/utils/__init__.py:229-273``)."""
    import json

    from warpy_kernels_b200 import utils

    path = tmp_path / "cache" / "tune.json"
    monkeypatch.setattr(utils, "TUNE_CACHE_PATH", str(path))
    key = utils.tune_key("fwd", 128, True, 4096, 4000, 4)
    assert key == "fwd|d=128|causal=1|nq=4096|nk=4096|rep=4|sm100"
    assert utils.tune_key("bwd_bf16", 64, False, 5, 1025, 1, arch=120) == "bwd_bf16|d=64|causal=0|nq=1024|nk=2048|rep=1"
    assert utils.tune_lookup(key) is None
    utils.tune_store(key, {"num_stages": 3})
    assert json.load(open(path)) == {key: {"num_stages": 3}}
    utils.forget_tune_cache()  # a new process reads the file back
    assert utils.tune_lookup(key) == {"num_stages": 3}
    best, results = utils.autotune("fwd", 128, False, 10, 10, 1, [{"a": 1}], lambda cfg: (lambda: None), 1, False) \
        if torch.cuda.is_available() else ({"a": 1}, [])
    assert best == {"a": 1}
