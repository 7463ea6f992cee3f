"""CPU: the multi-GPU sharding logic, with two gloo ranks standing in for two GPUs."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from warpy_kernels_b200 import shard


def test_split_range_covers_everything():
    for n in (1, 7, 8, 128, 129):
        for world in (1, 2, 3, 8):
            spans = [shard.split_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("B,Hkv,world", [(4, 32, 8), (4, 32, 1), (4, 32, 3), (1, 8, 8), (1, 8, 4), (2, 3, 4), (1, 8, 3),
                                          (5, 2, 3)])
def test_attention_shard_partitions_batch_times_kv_heads(B, Hkv, world):
    seen = []
    for r in range(world):
        pieces = shard.attention_shard(B, Hkv, world, r)
        assert len(pieces) <= 3
        mine = []
        for b0, b1, h0, h1 in pieces:
            assert 0 <= b0 < b1 <= B and 0 <= h0 < h1 <= Hkv
            assert b1 - b0 == 1 or (h0, h1) == (0, Hkv)  # only whole batch items are merged
            mine += [b * Hkv + h for b in range(b0, b1) for h in range(h0, h1)]
        lo, hi = shard.attention_units(B, Hkv, world, r)
        assert mine == list(range(lo, hi))  # in unit order, contiguous
        seen += mine
    assert seen == list(range(B * Hkv))
    if world == 1:
        assert shard.attention_shard(B, Hkv, 1, 0) == [(0, B, 0, Hkv)]  # one call on the whole tensors


def test_gemm_shard_is_tile_aligned():
    for world in (1, 2, 4, 8):
        spans = [shard.gemm_shard(8192, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 8192
        assert all(a % 128 == 0 and b % 128 == 0 for a, b in spans)
    with pytest.raises(ValueError):
        shard.gemm_shard(100, 2, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # GEMM by rows: each rank computes its slab of a @ b.T, the gather reassembles the full product
        g = torch.Generator().manual_seed(0)
        a, b = torch.randn(512, 64, generator=g), torch.randn(96, 64, generator=g)
        lo, hi = shard.gemm_shard(512, world, rank)
        full = shard.gather_rows(a[lo:hi] @ b.T, 512)
        assert torch.equal(full, torch.cat([a[s:e] @ b.T for s, e in (shard.gemm_shard(512, world, r) for r in range(world))]))
        # attention by (batch, KV head): stand-in "kernel" = a per-head function; GQA groups stay together
        B, Hq, Hkv, N, d = 2, 6, 3, 8, 4
        q = torch.randn(B, Hq, N, d, generator=g)
        k, v = torch.randn(B, Hkv, N, d, generator=g), torch.randn(B, Hkv, N, d, generator=g)
        sq = torch.rand(B, Hkv, generator=g)

        def fake_attn(qs, ks, vs, ds):
            rep = qs.shape[1] // ks.shape[1]
            return qs * ds[0].repeat_interleave(rep, 1)[:, :, None, None] + ks.repeat_interleave(rep, 1) - vs.repeat_interleave(rep, 1)

        want = fake_attn(q, k, v, (sq, None, None))
        # (a) the kernel writes into this rank's slab through per-piece views: nothing is copied before the gather
        slab, views = shard.local_head_slab(want.shape, Hkv, world, rank, want.dtype, want.device)
        pieces = shard.attention_shard(B, Hkv, world, rank)
        for piece, view in zip(pieces, views):
            qs, ks, vs, ds = shard.slice_attention_inputs(q, k, v, (sq, None, None), piece)
            view.copy_(fake_attn(qs, ks, vs, ds))
        assert torch.equal(shard.gather_heads(slab, want.shape, Hkv), want)
        # (b) a list of per-piece tensors works too
        mine = [fake_attn(*shard.slice_attention_inputs(q, k, v, (sq, None, None), piece)[:3],
                          shard.slice_attention_inputs(q, k, v, (sq, None, None), piece)[3]) for piece in pieces]
        assert torch.equal(shard.gather_heads(mine, want.shape, Hkv), want)
        # uneven split: 5 batch items x 1 KV head over 2 ranks
        q5 = torch.randn(5, 2, N, d, generator=g)
        lo5, hi5 = shard.attention_units(5, 1, world, rank)
        assert torch.equal(shard.gather_heads([q5[lo5:hi5] * 2], q5.shape, 1), q5 * 2)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_with_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
