"""Multi-GPU sharding of the hot path: one process per GPU, no data-path collective.

The reference has no multi-GPU code.  Every kernel here works on independent units, so the work is split before the
call and each rank runs the unchanged single-GPU entry points on its slice:

* attention forward / backward: by (batch, KV-head group) -- all query heads that share a KV head stay on one rank,
  so dK/dV need no reduction;
* GEMM and quantiser: by rows of ``a`` (tokens); ``b`` (the weights) is replicated.

Only when a caller wants one full tensor back is a collective used: ``gather_rows`` /``gather_heads`` call
``torch.distributed.all_gather`` (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""

import torch
import torch.distributed as dist


def split_range(n, world, rank):
    """Contiguous near-even split of ``range(n)``; the first ``n % world`` ranks get one extra unit."""
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def attention_shard(B, Hkv, world, rank):
    """Units of work are the ``B * Hkv`` (batch, KV head) pairs.

    Returns:
        List of ``(b, hkv_start, hkv_stop)`` slices owned by ``rank``; consecutive KV heads of one batch item are merged.
    """
    lo, hi = split_range(B * Hkv, world, rank)
    out = []
    u = lo
    while u < hi:
        b, h0 = divmod(u, Hkv)
        h1 = min(Hkv, h0 + (hi - u))
        out.append((b, h0, h1))
        u += h1 - h0
    return out


def slice_attention_inputs(q, k, v, descales, piece):
    """Views of ``q, k, v`` and the ``[B, Hkv]`` descales for one ``(b, hkv_start, hkv_stop)`` piece."""
    b, h0, h1 = piece
    group = q.shape[1] // k.shape[1]
    qs = q[b : b + 1, h0 * group : h1 * group]
    ks, vs = k[b : b + 1, h0:h1], v[b : b + 1, h0:h1]
    ds = tuple(None if s is None else s[b : b + 1, h0:h1] for s in descales)
    return qs, ks, vs, ds


def gemm_shard(M, world, rank, tile=128):
    """Rows ``[start, stop)`` of ``a`` for this rank; shards are multiples of the 128-row tile."""
    if M % tile:
        raise ValueError(f"M must be a multiple of {tile}")
    lo, hi = split_range(M // tile, world, rank)
    return lo * tile, hi * tile


def gather_rows(local, M, group=None):
    """All-gather row shards of a ``[rows, N]`` tensor (split by ``gemm_shard``) into the full ``[M, N]`` tensor."""
    world = dist.get_world_size(group)
    sizes = [gemm_shard(M, world, r) for r in range(world)]
    full = torch.empty((M,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pieces = [full[a:b] for a, b in sizes]
    if all(p.shape == pieces[0].shape for p in pieces):
        dist.all_gather_into_tensor(full, local.contiguous(), group=group)
    else:
        dist.all_gather(pieces, local.contiguous(), group=group)
    return full


def gather_heads(local_pieces, shape, B, Hkv, dtype, device, group=None):
    """All-gather per-rank attention outputs back into one ``[B, Hq, N, d]`` tensor.

    Args:
        local_pieces: This rank's list of ``(piece, tensor)`` as produced from ``attention_shard``.
        shape: Full output shape ``(B, Hq, N, d)``.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    full = torch.zeros(shape, dtype=dtype, device=device)
    group_size = shape[1] // Hkv
    for r in range(world):
        for piece in attention_shard(B, Hkv, world, r):
            b, h0, h1 = piece
            dst = full[b, h0 * group_size : h1 * group_size]
            if r == rank:
                src = dict((p, t) for p, t in local_pieces)[piece]
                dst.copy_(src.reshape(dst.shape))
            buf = dst.contiguous()
            dist.broadcast(buf, src=r if group is None else dist.get_global_rank(group, r), group=group)
            if r != rank:
                dst.copy_(buf)
    return full
