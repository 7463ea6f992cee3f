"""Host-side helpers with the semantics of the reference's ``warpy_kernels/utils/__init__.py``.

Only the pieces the hot path uses are here: ``round_up``/``pad_rows`` (``:170-179``), ``check_descale``
(``:151-167``), ``cached_tensor`` (``:113-126``), and ``time_launch_ms``/``time_candidates`` (``:182-226``).  The
reference's JIT compile cache and JSON tune cache have no counterpart: kernels here are compiled ahead of time.
"""

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
