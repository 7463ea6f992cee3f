"""Multi-GPU sharding of the hot path: one process per GPU, no data-path collective.

The reference has no multi-GPU code.  Every kernel here works on independent units, so one problem is split
before the call and each rank runs the unchanged single-GPU entry points on its slice:

* attention forward / backward: the units are the ``B * Hkv`` (batch, KV head) pairs in row-major order; all query
  heads that share a KV head stay on one rank, so dK / dV need no reduction.  A rank owns a contiguous range of
  units, which is at most three rectangular pieces ``(b0, b1, h0, h1)`` of the input tensors (a partial batch item,
  whole batch items, a partial batch item): one kernel call per piece;
* GEMM and quantiser: by rows of ``a`` (tokens) in multiples of the 128-row tile; ``b`` (the weights) is replicated.

Only when a caller wants one full tensor back is a collective used: ``gather_rows`` and ``gather_heads`` are one
``all_gather_into_tensor`` each (NCCL over NVLink on GPUs, gloo in the CPU tests) when the shards are equal, which
they are whenever the unit count divides by the world size (else the shards are padded to equal length for the one
collective).  In both layouts a rank's shard is one contiguous block of the full tensor, so equal shards are
gathered in place, with nothing staged or copied around the call.
"""

import torch
import torch.distributed as dist


def split_range(n, world, rank):
    """Contiguous near-even split of ``range(n)``; the first ``n % world`` ranks get one extra unit."""
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def attention_units(B, Hkv, world, rank):
    """``(start, stop)`` of this rank's (batch, KV head) units, numbered ``b * Hkv + h``."""
    return split_range(B * Hkv, world, rank)


def attention_shard(B, Hkv, world, rank):
    """This rank's units as rectangular pieces ``(b0, b1, h0, h1)``: batch items ``[b0, b1)`` x KV heads ``[h0, h1)``.

    In unit order; whole batch items are merged into one piece, so a rank that owns everything (world size 1) makes a
    single call on the whole tensors.
    """
    lo, hi = attention_units(B, Hkv, world, rank)
    pieces = []
    u = lo
    while u < hi:
        b, h0 = divmod(u, Hkv)
        if h0 == 0 and hi - u >= Hkv:
            whole = (hi - u) // Hkv
            pieces.append((b, b + whole, 0, Hkv))
            u += whole * Hkv
        else:
            h1 = min(Hkv, h0 + (hi - u))
            pieces.append((b, b + 1, h0, h1))
            u += h1 - h0
    return pieces


def slice_attention_inputs(q, k, v, descales, piece):
    """Views of ``q, k, v`` and the ``[B, Hkv]`` descales for one ``(b0, b1, h0, h1)`` piece."""
    b0, b1, h0, h1 = piece
    group = q.shape[1] // k.shape[1]
    qs = q[b0:b1, h0 * group : h1 * group]
    ks, vs = k[b0:b1, h0:h1], v[b0:b1, h0:h1]
    ds = tuple(None if s is None else s[b0:b1, h0:h1] for s in descales)
    return qs, ks, vs, ds


def local_head_slab(shape, Hkv, world, rank, dtype, device):
    """Buffer for this rank's part of a ``[B, Hq, N, d]`` tensor plus a view of it per piece.

    Returns:
        ``(slab, views)``: ``slab`` is ``[units, Hq / Hkv, N, d]``, one entry per owned (batch, KV head) unit in unit
        order -- the block ``gather_heads`` sends; ``views[i]`` is the ``[b1 - b0, (h1 - h0) * Hq / Hkv, N, d]`` window
        of piece ``i``, to be passed as the kernel's ``out=``.
    """
    B, Hq, N, d = shape
    group = Hq // Hkv
    lo, hi = attention_units(B, Hkv, world, rank)
    slab = torch.empty(hi - lo, group, N, d, dtype=dtype, device=device)
    views = []
    for b0, b1, h0, h1 in attention_shard(B, Hkv, world, rank):
        u0 = b0 * Hkv + h0 - lo
        n_units = (b1 - b0) * (h1 - h0)
        views.append(slab[u0 : u0 + n_units].view(b1 - b0, (h1 - h0) * group, N, d))
    return slab, views


def gemm_shard(M, world, rank, tile=128):
    """Rows ``[start, stop)`` of ``a`` for this rank; shards are multiples of the 128-row tile."""
    if M % tile:
        raise ValueError(f"M must be a multiple of {tile}")
    lo, hi = split_range(M // tile, world, rank)
    return lo * tile, hi * tile


def _gather_blocks(full_rows, local, spans, group):
    """All-gather ``local`` (rows ``spans[rank]`` of ``full_rows``) into ``full_rows`` with one collective.

    Equal shards land in place.  Unequal ones (the unit count does not divide by the world size) are padded to the
    longest shard, gathered into a temporary and copied out, since not every backend gathers unequal tensors.
    """
    local = local.contiguous()
    sizes = [b - a for a, b in spans]
    if len(set(sizes)) == 1:
        dist.all_gather_into_tensor(full_rows, local, group=group)
        return
    longest = max(sizes)
    padded = local.new_zeros((longest,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    staged = local.new_empty((len(spans) * longest,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(staged, padded, group=group)
    for r, (a, b) in enumerate(spans):
        full_rows[a:b] = staged[r * longest : r * longest + (b - a)]


def gather_rows(local, M, group=None):
    """All-gather row shards of a ``[rows, N]`` tensor (split by ``gemm_shard``) into the full ``[M, N]`` tensor."""
    world = dist.get_world_size(group)
    full = torch.empty((M,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    _gather_blocks(full, local, [gemm_shard(M, world, r) for r in range(world)], group)
    return full


def gather_heads(local, shape, Hkv, group=None):
    """All-gather per-rank attention outputs back into one ``[B, Hq, N, d]`` tensor.

    Args:
        local: This rank's ``[units, Hq / Hkv, N, d]`` slab (``local_head_slab``), or a list of per-piece tensors in
            the order of ``attention_shard`` (they are concatenated, which costs a copy the slab avoids).
        shape: Full output shape ``(B, Hq, N, d)``.
        Hkv: Number of KV heads (the split granularity).
    """
    B, Hq, N, d = shape
    world = dist.get_world_size(group)
    units, per_unit = B * Hkv, (Hq // Hkv, N, d)
    if not torch.is_tensor(local):
        local = torch.cat([t.reshape(-1, *per_unit) for t in local]) if local else None
    spans = [split_range(units, world, r) for r in range(world)]
    if local is None:
        raise ValueError("a rank without units cannot take part in the gather: use at most B * Hkv ranks")
    full = torch.empty(units, *per_unit, dtype=local.dtype, device=local.device)
    _gather_blocks(full, local.reshape(-1, *per_unit), spans, group)
    return full.view(B, Hq, N, d)
