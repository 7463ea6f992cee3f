"""Shared input recipes for the GPU tests (the reference's ``tests/fixtures.py:58-88`` recipes, seeded on the
device) and the comparison against the oracle."""

import math

import numpy as np
import torch

from oracle import reference_math as R


def randn_qkv(B, Hq, Hkv, Nq, Nk, d, seed=0, device="cuda"):
    """Random float32 ``q, k, v`` with ``k`` and ``v`` centred over the sequence (``tests/fixtures.py:72-78``)."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(B, Hq, Nq, d, device=device, generator=g)
    k = torch.randn(B, Hkv, Nk, d, device=device, generator=g)
    v = torch.randn(B, Hkv, Nk, d, device=device, generator=g)
    return q, k - k.mean(dim=2, keepdim=True), v - v.mean(dim=2, keepdim=True)


def hard_inputs(B, Hq, Hkv, Nq, Nk, d, seed=0, logit_std=4.0, dout_spread=1.5, device="cuda"):
    """Peaky-softmax inputs and log-normal dO row norms (``tests/fixtures.py:58-69``)."""
    q, k, v = randn_qkv(B, Hq, Hkv, Nq, Nk, d, seed, device)
    g = torch.Generator(device=device).manual_seed(seed + 1000)
    dout = torch.randn(B, Hq, Nq, d, device=device, generator=g)
    dout = dout * torch.exp(dout_spread * torch.randn(B, Hq, Nq, 1, device=device, generator=g))
    s = math.sqrt(logit_std)
    return q * s, k * s, v, dout


def sink_qkv(Nq, Nk, d, gap_nats, seed=1, device="cuda"):
    """One key ``gap_nats`` above a long near-uniform tail (``tests/fixtures.py:81-88``)."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = 1.0 + 0.1 * torch.randn(1, 1, Nq, d, device=device, generator=g)
    k = 0.01 * torch.randn(1, 1, Nk, d, device=device, generator=g)
    k[:, :, 0, :] = gap_nats / math.sqrt(d)
    v = torch.randn(1, 1, Nk, d, device=device, generator=g)
    return q, k, v


def load_golden(path, device):
    z = np.load(path)
    B, Hq, Hkv, Nq, Nk, d, causal, seed = [int(x) for x in z["shape"]]
    f8 = lambda a: torch.from_numpy(a).to(device).view(torch.float8_e4m3fn)
    t = dict(
        q8=f8(z["q8"]), k8=f8(z["k8"]), v8=f8(z["v8"]),
        sq=torch.from_numpy(z["sq"]).to(device), sk=torch.from_numpy(z["sk"]).to(device),
        sv=torch.from_numpy(z["sv"]).to(device),
        dout=torch.from_numpy(z["dout_bf16"]).to(device).view(torch.bfloat16), causal=bool(causal),
        out=torch.from_numpy(z["out"].astype(np.float32)), lse=torch.from_numpy(z["lse"]),
        dq=torch.from_numpy(z["dq"]), dk=torch.from_numpy(z["dk"]), dv=torch.from_numpy(z["dv"]),
    )
    return t


def fwd_errors(out, lse, out_ref, lse_ref, Nq, Nk, causal):
    """Errors the reference's ``_errors`` records (``tests/fixtures.py:188-228``) plus cosine and max-abs."""
    out, lse, out_ref, lse_ref = out.float().cpu(), lse.float().cpu(), out_ref.float().cpu(), lse_ref.float().cpu()
    visible = torch.ones(Nq, dtype=torch.bool)
    if causal:
        visible = (torch.arange(Nq) + Nk - Nq) >= 0
    errs = {
        "out": R.rel_l2(out[:, :, visible], out_ref[:, :, visible]),
        "lse": (lse[:, :, visible] - lse_ref[:, :, visible]).abs().max().item() if visible.any() else 0.0,
        "cos": R.cosine(out[:, :, visible], out_ref[:, :, visible]) if visible.any() else 1.0,
        "max_abs": R.max_abs(out[:, :, visible], out_ref[:, :, visible]) if visible.any() else 0.0,
    }
    assert bool((out[:, :, ~visible] == 0).all()), "rows without a visible key must give O = 0"
    assert not torch.isfinite(lse[:, :, ~visible]).any().item(), "rows without a visible key need a non-finite lse"
    assert not torch.isnan(out).any().item()
    return errs
