"""GPU (two or more devices): one problem split over two ranks through ``warpy_kernels_b200.shard``, the real kernels
on each shard, one NCCL all-gather, and the gathered tensor compared bit for bit with the single-GPU result.

The ranks are child processes, one per GPU; no kernel reads another GPU's memory and NCCL is the only cross-GPU
traffic.  Skipped on a box with a single GPU (two NCCL ranks cannot share a device).
"""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist

    import warpy_kernels as wk
    from oracle import reference_math as R
    from warpy_kernels_b200 import _lib, shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # ---- FP8 GQA attention forward, causal: by (batch, KV head) -------------------------------------------
        B, Hq, Hkv, N, d = 2, 12, 3, 640, 128
        g = torch.Generator(device=dev).manual_seed(0)  # the same inputs on every rank
        q = torch.randn(B, Hq, N, d, device=dev, generator=g)
        k = torch.randn(B, Hkv, N, d, device=dev, generator=g)
        v = torch.randn(B, Hkv, N, d, device=dev, generator=g)
        q8, k8, v8, sq, sk, sv = R.quantize_qkv(q, k, v)
        slab, views = shard.local_head_slab((B, Hq, N, d), Hkv, world, rank, torch.bfloat16, dev)
        for piece, view in zip(shard.attention_shard(B, Hkv, world, rank), views):
            qs, ks, vs, ds = shard.slice_attention_inputs(q8, k8, v8, (sq, sk, sv), piece)
            out, _, _ = wk.attn_fwd(qs, ks, vs, *ds, causal=True, out=view)
            assert out.data_ptr() == view.data_ptr()  # written in place: nothing to copy before the gather
        full = shard.gather_heads(slab, (B, Hq, N, d), Hkv)
        whole, _, _ = wk.attn_fwd(q8, k8, v8, sq, sk, sv, causal=True)
        assert torch.equal(full, whole), "sharded attention differs from the single-GPU result"

        # ---- MXFP8 GEMM: by rows of a ----------------------------------------------------------------------------
        m, n, k_ = 1024, 512, 1024
        a8, sa = wk.quantize_mx(torch.randn(m, k_, device=dev, generator=g).bfloat16())
        b8, sb = wk.quantize_mx(torch.randn(n, k_, device=dev, generator=g).bfloat16())
        lo, hi = shard.gemm_shard(m, world, rank)
        local = wk.gemm(a8[lo:hi], b8, a_scale_mx=sa[lo:hi], b_scale_mx=sb)
        assert torch.equal(shard.gather_rows(local, m), wk.gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb))

        # ---- quantiser: by rows -----------------------------------------------------------------------------------
        x = torch.randn(m, k_, device=dev, generator=g).bfloat16()
        ql, sl = wk.quantize_mx(x[lo:hi])
        qw, sw = wk.quantize_mx(x)
        assert torch.equal(shard.gather_rows(ql.view(torch.uint8), m), qw.view(torch.uint8))
        assert torch.equal(shard.gather_rows(sl, m), sw)
        _lib.device_status()
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_sharded_kernels_match_single_gpu(tmp_path):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
