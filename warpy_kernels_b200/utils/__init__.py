"""Host-side helpers with the semantics of the reference's ``warpy_kernels/utils/__init__.py``.

Only the pieces the hot path uses are here: ``round_up``/``pad_rows`` (``:170-179``), ``check_descale``
(``:151-167``), ``cached_tensor`` (``:113-126``), ``time_launch_ms``/``time_candidates`` (``:182-226``) and the JSON
tune cache (``:229-273``: same file, same keys with an ``|sm100`` suffix, so one cache file can serve both
libraries).  The reference's JIT compile cache has no counterpart: kernels here are compiled ahead of time.
"""

import json
import os

import torch
import torch.nn.functional as F

_cached = {}


def cached_tensor(key, make):
    """Return a constant tensor made once per ``key`` (callers must not write to it)."""
    t = _cached.get(key)
    if t is None:
        t = _cached[key] = make()
    return t


def check_descale(x, batch, h_kv, name):
    """Check that a dequantization scale is ``None`` or a ``[B, Hkv]`` tensor on a CUDA device.

    Raises:
        ValueError: Otherwise.
    """
    if x is not None and (tuple(x.shape) != (batch, h_kv) or not x.is_cuda):
        raise ValueError(
            f"{name} must be a CUDA tensor of shape [B, Hkv] = [{batch}, {h_kv}], "
            f"got {tuple(x.shape)} on {x.device}"
        )


def round_up(x, m):
    return (x + m - 1) // m * m


def pad_rows(x, n_pad, value=0):
    n = x.shape[-2] if x.dim() == 4 else x.shape[-1]  # row count
    if n == n_pad:
        return x.contiguous()
    pad = (0, 0, 0, n_pad - n) if x.dim() == 4 else (0, n_pad - n)
    return F.pad(x, pad, value=value).contiguous()


def time_launch_ms(fn, iters=10, warmup=3):
    """Mean milliseconds per call of ``fn`` between two CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def time_candidates(candidates, build, iters, verbose, what):
    """Time every candidate config and pick the fastest.

    Returns:
        ``(best_config, results)``, where ``results`` is a list of ``(config, milliseconds or error string)``.

    Raises:
        RuntimeError: If no candidate runs.
    """
    results = []
    for cfg in candidates:
        try:
            results.append((cfg, time_launch_ms(build(cfg), iters)))
        except (ValueError, NotImplementedError, RuntimeError) as e:
            results.append((cfg, f"{type(e).__name__}: {str(e)[:120]}"))
        if verbose:
            t = results[-1][1]
            print(f"  {what} tune {cfg}: {t if isinstance(t, str) else f'{t:.3f} ms'}", flush=True)
    timed = [(c, t) for c, t in results if not isinstance(t, str)]
    if not timed:
        raise RuntimeError(f"no {what} config ran: {results}")
    return min(timed, key=lambda ct: ct[1])[0], results


# ---- tune cache: best config per (kernel, head dim, causal, length bucket, GQA ratio), one JSON object on disk ----
TUNE_CACHE_PATH = os.environ.get("WARPY_KERNELS_TUNE_CACHE", os.path.expanduser("~/.cache/warpy_kernels_tune.json"))
_tune_cache = None


def tune_key(kind, d, causal, nq, nk, rep, arch=100):
    """Cache key in the reference's format; lengths fall into power-of-two buckets of at least 1024."""
    bucket = lambda n: 1 << max(10, (int(n) - 1).bit_length())
    key = f"{kind}|d={d}|causal={int(causal)}|nq={bucket(nq)}|nk={bucket(nk)}|rep={rep}"
    return key if arch == 120 else f"{key}|sm{arch}"


def tune_lookup(key):
    """The stored config for ``key``, or ``None``. An unreadable cache file counts as empty."""
    global _tune_cache
    if _tune_cache is None:
        try:
            with open(TUNE_CACHE_PATH) as f:
                _tune_cache = json.load(f)
        except (OSError, ValueError):
            _tune_cache = {}
    return _tune_cache.get(key)


def tune_store(key, cfg):
    """Remember ``cfg`` for ``key`` and rewrite the cache file (silently skipped if the file cannot be written)."""
    tune_lookup(key)
    _tune_cache[key] = cfg
    try:
        os.makedirs(os.path.dirname(TUNE_CACHE_PATH) or ".", exist_ok=True)
        with open(TUNE_CACHE_PATH, "w") as f:
            json.dump(_tune_cache, f, indent=1, sort_keys=True)
    except OSError:
        pass


def autotune(kind, d, causal, nq, nk, rep, candidates, build, iters, verbose, arch=100):
    """Time the candidates, store the winner under the shape's key, and return ``(best_config, results)``."""
    best, results = time_candidates(candidates, build, iters, verbose, kind)
    tune_store(tune_key(kind, d, causal, nq, nk, rep, arch), best)
    return best, results
