"""Host-side helpers of the B200 build: argument checks, launch timing and the on-disk tune cache.

What the reference's API contract fixes is kept: the names ``round_up``, ``check_descale``, ``cached_tensor``,
``time_launch_ms``, ``time_candidates``, ``tune_key``, ``tune_lookup``, ``tune_store`` and ``autotune``
(``warpy_kernels/utils/__init__.py:113-273``), the error type of ``check_descale``, the ``(best, results)`` return
of the tuners, and the tune cache's file name, JSON layout and key format (keys carry an ``|sm100`` suffix, so one
cache file can serve this library and the reference side by side).  The reference's JIT compile cache has no
counterpart: the kernels here are compiled ahead of time.
"""

import json
import os

import torch

_constants = {}


def cached_tensor(key, make):
    """A read-only constant tensor, built by ``make()`` the first time ``key`` is seen."""
    try:
        return _constants[key]
    except KeyError:
        return _constants.setdefault(key, make())


def check_descale(x, batch, h_kv, name):
    """Accept ``None`` or a CUDA tensor shaped ``[B, Hkv]`` as a dequantisation scale.

    Raises:
        ValueError: For any other shape, or a tensor that is not on a CUDA device.
    """
    if x is None:
        return
    want = (batch, h_kv)
    if tuple(x.shape) == want and x.is_cuda:
        return
    raise ValueError(f"{name}: expected a CUDA tensor [B, Hkv] = {list(want)}, got {list(x.shape)} on {x.device}")


def round_up(x, m):
    """Smallest multiple of ``m`` that is not below ``x``."""
    return -(-x // m) * m


# ---- timing ------------------------------------------------------------------------------------------------------
def time_launch_ms(fn, iters=10, warmup=3):
    """Milliseconds per call of ``fn`` on the current stream: the whole run of ``iters`` calls between two CUDA
    events, divided by ``iters`` (launches overlap as they would in a real loop)."""
    stream = torch.cuda.current_stream()
    for _ in range(max(0, warmup)):
        fn()
    stream.synchronize()
    first, last = (torch.cuda.Event(enable_timing=True) for _ in range(2))
    first.record(stream)
    n = max(1, iters)
    for _ in range(n):
        fn()
    last.record(stream)
    last.synchronize()
    return first.elapsed_time(last) / n


def time_candidates(candidates, build, iters, verbose, what):
    """Time ``build(cfg)()`` for every candidate config.

    A candidate whose ``build`` or launch raises ``ValueError``, ``NotImplementedError`` or ``RuntimeError`` is
    recorded with the error text instead of a time and cannot win.

    Returns:
        ``(best_config, results)`` with ``results`` a list of ``(config, milliseconds or error string)``.

    Raises:
        RuntimeError: If every candidate failed.
    """
    results, best_cfg, best_ms = [], None, float("inf")
    for cfg in candidates:
        try:
            outcome = time_launch_ms(build(cfg), iters)
            if outcome < best_ms:
                best_cfg, best_ms = cfg, outcome
            shown = f"{outcome:.3f} ms"
        except (ValueError, NotImplementedError, RuntimeError) as err:
            outcome = shown = f"{type(err).__name__}: {str(err)[:120]}"
        results.append((cfg, outcome))
        if verbose:
            print(f"  {what} tune {cfg}: {shown}", flush=True)
    if best_cfg is None:
        raise RuntimeError(f"no {what} config ran: {results}")
    return best_cfg, results


# ---- tune cache ---------------------------------------------------------------------------------------------------
# One JSON object on disk, key -> config dict, shared with the reference (same default path and environment
# variable).  TUNE_CACHE_PATH is read at every access so tests and callers may repoint it.
TUNE_CACHE_PATH = os.environ.get("WARPY_KERNELS_TUNE_CACHE", os.path.expanduser("~/.cache/warpy_kernels_tune.json"))
_loaded = {"path": None, "entries": {}}


def _entries():
    if _loaded["path"] != TUNE_CACHE_PATH:
        entries = {}
        try:
            with open(TUNE_CACHE_PATH) as f:
                data = json.load(f)
            if isinstance(data, dict):
                entries = data
        except (OSError, ValueError):
            pass  # a missing or unreadable file is an empty cache
        _loaded.update(path=TUNE_CACHE_PATH, entries=entries)
    return _loaded["entries"]


def forget_tune_cache():
    """Drop the in-memory copy so the next lookup reads the file again."""
    _loaded.update(path=None, entries={})


def tune_key(kind, d, causal, nq, nk, rep, arch=100):
    """Cache key: kernel kind, head dimension, mask, sequence lengths rounded up to a power of two (at least 1024)
    and GQA ratio; every architecture but the reference's SM120 appends ``|sm<arch>``."""
    lengths = [max(1024, 1 << (int(n) - 1).bit_length()) for n in (nq, nk)]
    parts = [kind, f"d={d}", f"causal={int(bool(causal))}", f"nq={lengths[0]}", f"nk={lengths[1]}", f"rep={rep}"]
    if arch != 120:
        parts.append(f"sm{arch}")
    return "|".join(parts)


def gemm_tune_key(kind, m, n, k, arch=100):
    """Cache key of a GEMM shape (exact sizes: the best kernel depends on how the tiles fill the SMs)."""
    return f"{kind}|m={m}|n={n}|k={k}|sm{arch}"


def tune_lookup(key):
    """The config stored under ``key``, or ``None``."""
    return _entries().get(key)


def tune_store(key, cfg):
    """Store ``cfg`` under ``key`` and write the whole cache back; a file that cannot be written is skipped."""
    entries = _entries()
    entries[key] = cfg
    folder = os.path.dirname(TUNE_CACHE_PATH)
    try:
        if folder:
            os.makedirs(folder, exist_ok=True)
        with open(TUNE_CACHE_PATH, "w") as f:
            json.dump(entries, f, indent=1, sort_keys=True)
    except OSError:
        pass


def autotune(kind, d, causal, nq, nk, rep, candidates, build, iters, verbose, arch=100):
    """Time the candidates and remember the fastest under the shape's key; returns ``(best_config, results)``."""
    best, results = time_candidates(candidates, build, iters, verbose, kind)
    tune_store(tune_key(kind, d, causal, nq, nk, rep, arch), best)
    return best, results
