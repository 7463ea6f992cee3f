"""Benchmark of the warpy-kernels hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.  Its headline (``metric``, ``value``,
``e2e``, ``roofline``, ``cpu_baseline``) is the FP8 causal attention forward, batch 4, 32 heads, sequence 4096, head
dim 128 -- the configuration the metric is quoted on.  Under ``"workloads"`` the same line carries every other
configuration of the hot path, measured in the same process: BF16 GEMM 2048^3, the FP8 attention backward of the
headline shape, the MXFP8 GEMM at M 8192 with (N 14336, K 4096) and (N 4096, K 14336), the FP8 GQA forward at
32768 keys, and the MXFP8 quantiser.  ``--workload NAME`` measures one of them alone (profiling runs).

Per workload:
  value       device-timed: K steps between two CUDA events on the launching stream, inputs resident in HBM
  sustained   the same launch repeated back to back for about 1.5 s, with the SM clock sampled inside that region
              (``clocks`` comes from here: the K-step burst is far shorter than one nvidia-smi period)
  e2e         through the public Python API with HOST buffers: pinned host -> device copies of the step's inputs, the
              kernel(s), device -> host copy of the results, split into chunks over three streams so that the copies
              in both directions overlap the kernels
  roofline    achieved / measured peak, plus the fraction of the nominal dense peak
  cpu_baseline  the reference's CPU path for that workload (its torch fp32 test oracle, restated under ``oracle/``)
              on the host cores, bounded sample

Multi-GPU (launched by ``torch.distributed.run``): ONE problem of the stated size is split over the ranks through
``warpy_kernels_b200.shard`` -- attention by (batch, KV head), GEMM and quantiser by rows of ``a`` -- with no
data-path collective, so the scaling is strong: value = the whole problem's work / the slowest rank's time.
``with_gather`` adds the optional NCCL all-gather that assembles one full output tensor.  BF16 GEMM 2048^3 is too
small to shard: every rank computes it whole (replicas).

``--impl reference`` times the reference's CPU path on the host cores, K bounded-sample steps, rank 0 only.
"""

import argparse
import datetime
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

# the bench's tuner runs write their winners here, not into the user's cache file
os.environ.setdefault("WARPY_KERNELS_TUNE_CACHE",
                      os.path.join(tempfile.gettempdir(), f"warpy_kernels_bench_tune_{os.getpid()}.json"))

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL = {"fp8": 4500.0, "bf16": 2250.0}  # dense TFLOP/s, B200 data sheet
NOMINAL_HBM_GBS = 7700.0
ALL_CPUS = os.sched_getaffinity(0)  # before any binding near a GPU
HEADLINE = "attn_fwd"
ALL = ["attn_fwd", "gemm_bf16", "attn_bwd", "gemm_mx", "gemm_mx_b", "attn_gqa", "quant"]

# dram__bytes_read.sum + dram__bytes_write.sum per step on one GPU, from ncu captures (attention figures: captured
# at a fraction of the batch / heads and scaled, traffic grows with batch x heads)
DRAM_TRAFFIC_BYTES = {
    # persistent kernel + the two-term launch for the short query blocks (the flag scan moves a few KB)
    "attn_fwd": 2 * (96.5e6 + 31.9e6 + 12.6e6),
    "attn_fwd_small": 96.5e6 + 31.9e6 + 12.6e6,
    "attn_gqa": 4 * (83.2e6 + 85.2e6),
    "attn_gqa_small": 83.2e6 + 85.2e6,
    # prep + dK/dV + dQ
    "attn_bwd": 2 * (155.4e6 + 226.7e6 + 177.3e6),
    "attn_bwd_small": 155.4e6 + 226.7e6 + 177.3e6,
    "gemm_mx": 292.8e6 + 201.3e6,
    "gemm_bf16_8k": 1083.5e6 + 127.0e6,
    "gemm_bf16_8k_pair": 1083.5e6 + 127.0e6,
    "gemm_bf16_8k_single": 1377.2e6 + 128.6e6,
    "quant": 234.9e6 + 82.3e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------------------
# SM clock log: one nvidia-smi for the whole run, every line stamped; regions are cut out by wall-clock time
# ------------------------------------------------------------------------------------------------------------
class ClockLog:
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.samples, self.proc = [], None  # (epoch seconds, sm MHz, max MHz, watts, [reasons])
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, mx = float(parts[1]), float(parts[2])
                watts = float(parts[3])
            except ValueError:
                continue
            active = [n for n, v in zip(self.REASONS, parts[4:8]) if v.lower().startswith("active")]
            self.samples.append((stamp, sm, mx, watts, active))

    def wait_first(self, limit_s=3.0):
        t0 = time.time()
        while self.proc is not None and not self.samples and time.time() - t0 < limit_s:
            time.sleep(0.05)

    def window(self, t0, t1):
        """Median SM clock and the throttle reasons seen between wall-clock times t0 and t1."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.15)  # let the line that covers the end of the region arrive
        rows = [s for s in self.samples if t0 + 0.1 <= s[0] <= t1]
        sm = sorted(r[1] for r in rows)
        reasons = sorted({x for r in rows for x in r[4]})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": rows[0][2] if rows else None,
                "reasons": reasons, "samples": len(rows), "power_w_max": max((r[3] for r in rows), default=None)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()


def bind_near_gpu(index):
    """Pin this process to the CPUs nearest to GPU ``index`` (NVML's affinity mask), so that the pinned host
    buffers allocated afterwards land on that socket's memory.  Returns what was done, for the JSON line."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return {"cpus": f"{min(cpus)}-{max(cpus)}", "count": len(cpus)}
    except Exception as err:  # noqa: BLE001  (no NVML, no permission: run unbound)
        return {"cpus": None, "note": f"unbound ({type(err).__name__})"}
    return {"cpus": None, "note": "unbound"}


# ------------------------------------------------------------------------------------------------------------
# host <-> device pipelining for the end-to-end number
# ------------------------------------------------------------------------------------------------------------
class Pipeline:
    """Runs chunk callables round-robin on a few side streams; the calling stream waits for all of them.

    Each chunk enqueues its own host -> device copies, kernels and device -> host copies on the stream it is given,
    so the H2D copy of one chunk, the kernel of another and the D2H copy of a third run at the same time.
    """

    def __init__(self, dev, n_streams=None):
        n_streams = n_streams or E2E_STREAMS
        self.dev = dev
        self.streams = [torch.cuda.Stream(dev) for _ in range(n_streams)]

    def run(self, chunks, first=None):
        main = torch.cuda.current_stream(self.dev)
        start = main.record_event()
        ready = None
        if first is not None:  # work every chunk depends on (e.g. the weights of a GEMM), on the first side stream
            self.streams[0].wait_event(start)
            with torch.cuda.stream(self.streams[0]):
                first()
                ready = self.streams[0].record_event()
        for i, chunk in enumerate(chunks):
            s = self.streams[i % len(self.streams)]
            s.wait_event(start)
            if ready is not None:
                s.wait_event(ready)
            with torch.cuda.stream(s):
                chunk()
        for s in self.streams:
            main.wait_stream(s)


def pinned(t):
    return t.cpu().pin_memory()


def copy_floor_ms(dev, h2d_bytes, d2h_bytes, reps=4):
    """What the link between host and GPU allows for the step's bytes, with no kernel at all: the host -> device
    bytes as one big copy, the device -> host bytes as one big copy, and both at the same time on two streams.
    Returns the three times in milliseconds (best of ``reps``)."""
    if h2d_bytes + d2h_bytes == 0:
        return 0.0, 0.0, 0.0
    up_src = torch.zeros(max(h2d_bytes, 1), dtype=torch.uint8).pin_memory()
    up_dst = torch.empty(max(h2d_bytes, 1), dtype=torch.uint8, device=dev)
    down_src = torch.zeros(max(d2h_bytes, 1), dtype=torch.uint8, device=dev)
    down_dst = torch.zeros(max(d2h_bytes, 1), dtype=torch.uint8).pin_memory()
    main = torch.cuda.current_stream(dev)
    s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def once(up, down):
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for on, stream, dst, src in ((up, s_up, up_dst, up_src), (down, s_down, down_dst, down_src)):
            if on:
                stream.wait_stream(main)
                with torch.cuda.stream(stream):
                    dst.copy_(src, non_blocking=True)
                main.wait_stream(stream)
        e1.record(main)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    return tuple(min(once(up, down) for _ in range(reps)) for up, down in ((True, False), (False, True), (True, True)))


def split_even(n, parts):
    parts = max(1, min(parts, n))
    base, extra = divmod(n, parts)
    out, lo = [], 0
    for i in range(parts):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


# ------------------------------------------------------------------------------------------------------------
# workloads.  Each builder makes THIS RANK's shard of the stated problem and returns a dict:
#   step       enqueue the shard's kernels on the current stream (inputs resident)
#   e2e_step   the same through the public API from pinned host buffers, pipelined
#   gather     (world > 1) the optional all-gather into one full tensor
#   work       algorithmic work of the WHOLE problem (flop or bytes); work_local: this rank's part
# ------------------------------------------------------------------------------------------------------------
def quantize_per_tensor(x):
    scale = x.abs().amax().clamp_min(1e-12) / 448.0
    return (x / scale).to(torch.float8_e4m3fn), scale


E2E_CHUNKS = int(os.environ.get("WK_BENCH_E2E_CHUNKS", "8"))
E2E_STREAMS = int(os.environ.get("WK_BENCH_E2E_STREAMS", "3"))


def _e2e_subpieces(piece, target=None):
    """Split one rectangular piece (b0, b1, h0, h1) into about ``target`` chunks for the copy / compute pipeline:
    by batch item first, then by KV head inside a batch item."""
    b0, b1, h0, h1 = piece
    target = target or E2E_CHUNKS
    per_item = max(1, -(-target // (b1 - b0)))
    return [(b, b + 1, h0 + lo, h0 + hi) for b in range(b0, b1) for lo, hi in split_even(h1 - h0, per_item)]


def make_attn(dev, world, rank, B, Hq, Hkv, N, d, causal, seed, bf16=False, backward=False):
    import warpy_kernels as wk
    from warpy_kernels.attn import make_attn_bwd, make_attn_fwd
    from warpy_kernels_b200 import shard

    group = Hq // Hkv
    pieces = shard.attention_shard(B, Hkv, world, rank)
    g = torch.Generator(device=dev).manual_seed(seed + 17 * rank)
    slab, views = shard.local_head_slab((B, Hq, N, d), Hkv, world, rank, torch.bfloat16, dev)
    per_piece, launches, keep = [], [], []
    local_units = 0
    for piece, out_view in zip(pieces, views):
        b0, b1, h0, h1 = piece
        nb, nh = b1 - b0, h1 - h0
        local_units += nb * nh
        mk = lambda h: torch.randn(nb, h, N, d, device=dev, generator=g).bfloat16()
        q, k, v = mk(nh * group), mk(nh), mk(nh)
        if bf16:
            qx, kx, vx, ds = q, k, v, (None, None, None)
        else:
            (qx, sq), (kx, sk), (vx, sv) = (quantize_per_tensor(t.float()) for t in (q, k, v))
            ds = tuple(torch.full((nb, nh), float(s), device=dev) for s in (sq, sk, sv))
        del q, k, v
        entry = dict(piece=piece, q=qx, k=kx, v=vx, ds=ds, out=out_view)
        if not backward:
            launch, out, lse, pmax = make_attn_fwd(qx, kx, vx, *ds, causal=causal, out=out_view)
            launches.append(launch)
        else:
            out, lse, pmax = wk.attn_fwd(qx, kx, vx, *ds, causal=causal, out=out_view)
            dout = torch.randn(nb, nh * group, N, d, device=dev,
                               generator=torch.Generator(device=dev).manual_seed(7 + rank)).bfloat16()
            launch, finish = make_attn_bwd(qx, kx, vx, out, lse, pmax, dout, *ds, causal=causal)
            launches.append(launch)
            entry.update(lse=lse, pmax=pmax, dout=dout, grads=finish())
        per_piece.append(entry)
    keep.append(per_piece)

    def step():
        for launch in launches:
            launch()

    # ---- end to end: pinned host inputs -> device -> kernels -> pinned host results, pipelined over chunks
    pipe = Pipeline(dev)
    chunks, h2d, d2h = [], 0, 0
    as_u8 = (lambda t: t) if bf16 else (lambda t: t.view(torch.uint8))
    from_u8 = (lambda t: t) if bf16 else (lambda t: t.view(torch.float8_e4m3fn))
    for e in per_piece:
        b0, b1, h0, h1 = e["piece"]
        for sb0, sb1, sh0, sh1 in _e2e_subpieces(e["piece"]):
            bs, hs = slice(sb0 - b0, sb1 - b0), slice(sh0 - h0, sh1 - h0)
            qs = slice((sh0 - h0) * group, (sh1 - h0) * group)
            dsc = tuple(None if s is None else s[bs, hs].contiguous() for s in e["ds"])
            if not backward:
                host_in = [pinned(as_u8(t).contiguous()) for t in (e["q"][bs, qs], e["k"][bs, hs], e["v"][bs, hs])]
                dev_in = [torch.empty_like(t, device=dev) for t in host_in]
                host_out = torch.empty(sb1 - sb0, (sh1 - sh0) * group, N, d, dtype=torch.bfloat16).pin_memory()
                h2d += sum(t.numel() * t.element_size() for t in host_in)
                d2h += host_out.numel() * 2

                # prepared once, as a serving loop would: the launch reads the device buffers the copies fill
                run, o, _, _ = make_attn_fwd(*(from_u8(t) for t in dev_in), *dsc, causal=causal)

                def chunk(host_in=host_in, dev_in=dev_in, host_out=host_out, run=run, o=o):
                    for d_, h_ in zip(dev_in, host_in):
                        d_.copy_(h_, non_blocking=True)
                    run()
                    host_out.copy_(o, non_blocking=True)
            else:
                # the forward's saved tensors stay on the device; dout arrives from the host, gradients go back
                qc, kc, vc = e["q"][bs, qs], e["k"][bs, hs], e["v"][bs, hs]
                oc, lc, pc = e["out"][bs, qs], e["lse"][bs, qs], e["pmax"][bs, qs]
                host_do = pinned(e["dout"][bs, qs].contiguous())
                dev_do = torch.empty_like(host_do, device=dev)
                host_g = [torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (qc, kc, vc)]
                h2d += host_do.numel() * 2
                d2h += sum(t.numel() * 2 for t in host_g)

                run, finish = make_attn_bwd(qc, kc, vc, oc, lc, pc, dev_do, *dsc, causal=causal)

                def chunk(host_do=host_do, dev_do=dev_do, host_g=host_g, run=run, grads=finish()):
                    dev_do.copy_(host_do, non_blocking=True)
                    run()
                    for h_, g_ in zip(host_g, grads):
                        h_.copy_(g_, non_blocking=True)
            chunks.append(chunk)

    def gather():
        if backward:
            return None  # dq / dk / dv would be three gathers of the same kind; the forward's stands for them
        return shard.gather_heads(slab, (B, Hq, N, d), Hkv)

    per_unit = (10.0 if backward else 4.0) * group * N * N * d * (0.5 if causal else 1.0)
    return dict(step=step, e2e_step=lambda: pipe.run(chunks), gather=gather, work=per_unit * B * Hkv,
                work_local=per_unit * local_units, bound="tensor", dtype="bf16" if bf16 else "fp8",
                launches=3 * len(launches), h2d=h2d, d2h=d2h, e2e_chunks=len(chunks),
                gather_bytes=0 if backward else B * Hq * N * d * 2, keep=keep, shard=f"{local_units} of {B * Hkv} (batch, KV head) units")


def make_gemm_bf16(dev, world, rank, m, n, k, seed, cta_pair=None, sharded=True):
    import warpy_kernels as wk
    from warpy_kernels_b200 import shard

    lo, hi = shard.gemm_shard(m, world, rank) if sharded else (0, m)
    g = torch.Generator(device=dev).manual_seed(seed + 17 * rank)
    a = torch.randn(hi - lo, k, device=dev, generator=g).bfloat16()
    b = torch.randn(n, k, device=dev, generator=torch.Generator(device=dev).manual_seed(seed + 1)).bfloat16()
    launch, out = wk.make_gemm(a, b, cta_pair=cta_pair)
    pipe = Pipeline(dev)
    hb, db = pinned(b), torch.empty_like(b)
    chunks, h2d, d2h = [], hb.numel() * 2, 0
    for r0, r1 in ((128 * x, 128 * y) for x, y in split_even((hi - lo) // 128, 8)):
        ha, da = pinned(a[r0:r1]), torch.empty(r1 - r0, k, dtype=a.dtype, device=dev)
        ho = torch.empty(r1 - r0, n, dtype=torch.bfloat16).pin_memory()
        h2d, d2h = h2d + ha.numel() * 2, d2h + ho.numel() * 2

        def chunk(ha=ha, da=da, ho=ho):
            da.copy_(ha, non_blocking=True)
            ho.copy_(wk.gemm(da, db, cta_pair=cta_pair), non_blocking=True)
        chunks.append(chunk)
    first = lambda: db.copy_(hb, non_blocking=True)
    return dict(step=launch, e2e_step=lambda: pipe.run(chunks, first), gather=lambda: shard.gather_rows(out, m),
                work=2.0 * m * n * k, work_local=2.0 * (hi - lo) * n * k, bound="tensor",
                dtype="bf16", launches=1, h2d=h2d, d2h=d2h, e2e_chunks=len(chunks), gather_bytes=m * n * 2,
                keep=(a, b, out), shard=f"rows {lo}:{hi} of {m}" if sharded else "replica (whole problem per rank)",
                replicas=not sharded)


def make_gemm_mx(dev, world, rank, m, n, k, seed, cta_pair=None):
    import warpy_kernels as wk
    from warpy_kernels_b200 import shard

    lo, hi = shard.gemm_shard(m, world, rank)
    g = torch.Generator(device=dev).manual_seed(seed + 17 * rank)
    a8, sa = wk.quantize_mx(torch.randn(hi - lo, k, device=dev, generator=g).bfloat16())
    b8, sb = wk.quantize_mx(torch.randn(n, k, device=dev,
                                        generator=torch.Generator(device=dev).manual_seed(seed + 1)).bfloat16())
    tuned = None
    if cta_pair is None:
        # untimed set-up, like the reference's tuner: time the two kernels once for this shape; make_gemm then
        # finds the winner in the tune cache
        tuned, _ = wk.autotune_gemm(a8, b8, iters=5, verbose=False, a_scale_mx=sa, b_scale_mx=sb)
    launch, out = wk.make_gemm(a8, b8, a_scale_mx=sa, b_scale_mx=sb, cta_pair=cta_pair)
    pipe = Pipeline(dev)
    u8 = lambda t: t.view(torch.uint8)
    f8 = lambda t: t.view(torch.float8_e4m3fn)
    hb, hsb = pinned(u8(b8)), pinned(sb)
    db, dsb = torch.empty_like(hb, device=dev), torch.empty_like(hsb, device=dev)
    chunks, h2d, d2h = [], hb.numel() + hsb.numel(), 0
    for r0, r1 in ((128 * x, 128 * y) for x, y in split_even((hi - lo) // 128, 8)):
        ha, hs = pinned(u8(a8[r0:r1])), pinned(sa[r0:r1])
        da, dsa = torch.empty_like(ha, device=dev), torch.empty_like(hs, device=dev)
        ho = torch.empty(r1 - r0, n, dtype=torch.bfloat16).pin_memory()
        h2d, d2h = h2d + ha.numel() + hs.numel(), d2h + ho.numel() * 2

        def chunk(ha=ha, hs=hs, da=da, dsa=dsa, ho=ho):
            da.copy_(ha, non_blocking=True)
            dsa.copy_(hs, non_blocking=True)
            ho.copy_(wk.gemm(f8(da), f8(db), a_scale_mx=dsa, b_scale_mx=dsb, cta_pair=cta_pair), non_blocking=True)
        chunks.append(chunk)

    def first():
        db.copy_(hb, non_blocking=True)
        dsb.copy_(hsb, non_blocking=True)

    return dict(step=launch, e2e_step=lambda: pipe.run(chunks, first), gather=lambda: shard.gather_rows(out, m),
                work=2.0 * m * n * k, work_local=2.0 * (hi - lo) * n * k, bound="tensor", dtype="fp8", launches=3,
                h2d=h2d, d2h=d2h, e2e_chunks=len(chunks), gather_bytes=m * n * 2, keep=(a8, b8, sa, sb, out),
                shard=f"rows {lo}:{hi} of {m}", tuned=tuned)


def make_quant(dev, world, rank, m, k, seed):
    import warpy_kernels as wk
    from warpy_kernels_b200 import shard

    lo, hi = shard.gemm_shard(m, world, rank)
    rows = hi - lo
    x = torch.randn(rows, k, device=dev, generator=torch.Generator(device=dev).manual_seed(seed + 17 * rank)).bfloat16()
    q = torch.empty(rows, k, dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty(rows, k // 32, dtype=torch.uint8, device=dev)
    pipe = Pipeline(dev)
    chunks, h2d, d2h = [], 0, 0
    for r0, r1 in ((128 * a, 128 * b) for a, b in split_even(rows // 128, 8)):
        hx, dx = pinned(x[r0:r1]), torch.empty(r1 - r0, k, dtype=x.dtype, device=dev)
        hq = torch.empty(r1 - r0, k, dtype=torch.uint8).pin_memory()
        hs = torch.empty(r1 - r0, k // 32, dtype=torch.uint8).pin_memory()
        h2d, d2h = h2d + hx.numel() * 2, d2h + hq.numel() + hs.numel()

        def chunk(hx=hx, dx=dx, hq=hq, hs=hs):
            dx.copy_(hx, non_blocking=True)
            cq, cs = wk.quantize_mx(dx)
            hq.copy_(cq.view(torch.uint8), non_blocking=True)
            hs.copy_(cs, non_blocking=True)
        chunks.append(chunk)
    per_row = k * (2 + 1 + 1 / 32)
    return dict(step=lambda: wk.quantize_mx(x, q, s), e2e_step=lambda: pipe.run(chunks),
                gather=lambda: shard.gather_rows(q.view(torch.uint8), m), work=m * per_row, work_local=rows * per_row,
                bound="hbm", dtype="u8", launches=1, h2d=h2d, d2h=d2h, e2e_chunks=len(chunks), gather_bytes=m * k,
                keep=(x, q, s), shard=f"rows {lo}:{hi} of {m}")


WORKLOADS = {
    "attn_fwd": dict(desc="FP8 causal attention forward B4 H32 N4096 d128", unit="TFLOP/s",
                     make=lambda dev, w, r: make_attn(dev, w, r, 4, 32, 32, 4096, 128, True, 0)),
    "attn_fwd_small": dict(desc="FP8 causal attention forward B2 H32 N4096 d128 (profiling size)", unit="TFLOP/s",
                           make=lambda dev, w, r: make_attn(dev, w, r, 2, 32, 32, 4096, 128, True, 0)),
    "attn_bwd": dict(desc="FP8 causal attention backward B4 H32 N4096 d128", unit="TFLOP/s",
                     make=lambda dev, w, r: make_attn(dev, w, r, 4, 32, 32, 4096, 128, True, 0, backward=True)),
    "attn_bwd_small": dict(desc="FP8 causal attention backward B2 H32 N4096 d128 (profiling size)", unit="TFLOP/s",
                           make=lambda dev, w, r: make_attn(dev, w, r, 2, 32, 32, 4096, 128, True, 0, backward=True)),
    "attn_fwd_bf16": dict(desc="BF16 causal attention forward B4 H32 N4096 d128", unit="TFLOP/s",
                          make=lambda dev, w, r: make_attn(dev, w, r, 4, 32, 32, 4096, 128, True, 0, bf16=True)),
    "attn_bwd_bf16": dict(desc="BF16 causal attention backward B4 H32 N4096 d128", unit="TFLOP/s",
                          make=lambda dev, w, r: make_attn(dev, w, r, 4, 32, 32, 4096, 128, True, 0, bf16=True,
                                                           backward=True)),
    "attn_gqa": dict(desc="FP8 GQA causal attention forward B1 Hq64 Hkv8 N32768 d128", unit="TFLOP/s",
                     make=lambda dev, w, r: make_attn(dev, w, r, 1, 64, 8, 32768, 128, True, 0)),
    "attn_gqa_small": dict(desc="FP8 GQA causal attention forward B1 Hq16 Hkv2 N32768 d128 (profiling size)",
                           unit="TFLOP/s", make=lambda dev, w, r: make_attn(dev, w, r, 1, 16, 2, 32768, 128, True, 0)),
    "attn_fwd_d64": dict(desc="FP8 causal attention forward B4 H32 N4096 d64", unit="TFLOP/s",
                         make=lambda dev, w, r: make_attn(dev, w, r, 4, 32, 32, 4096, 64, True, 0)),
    "gemm_bf16": dict(desc="BF16 GEMM M=N=K=2048", unit="TFLOP/s", flush=True,
                      make=lambda dev, w, r: make_gemm_bf16(dev, w, r, 2048, 2048, 2048, 0, sharded=False)),
    "gemm_bf16_8k": dict(desc="BF16 GEMM M=N=K=8192", unit="TFLOP/s",
                         make=lambda dev, w, r: make_gemm_bf16(dev, w, r, 8192, 8192, 8192, 0)),
    "gemm_bf16_8k_single": dict(desc="BF16 GEMM M=N=K=8192 on single CTAs (128 x 256 tiles)", unit="TFLOP/s",
                                make=lambda dev, w, r: make_gemm_bf16(dev, w, r, 8192, 8192, 8192, 0, cta_pair=False)),
    "gemm_bf16_8k_pair": dict(desc="BF16 GEMM M=N=K=8192 on CTA pairs (cta_group::2)", unit="TFLOP/s",
                              make=lambda dev, w, r: make_gemm_bf16(dev, w, r, 8192, 8192, 8192, 0, cta_pair=True)),
    "gemm_mx": dict(desc="MXFP8 GEMM M8192 N14336 K4096 (E8M0 scales on A and B)", unit="TFLOP/s",
                    make=lambda dev, w, r: make_gemm_mx(dev, w, r, 8192, 14336, 4096, 0)),
    "gemm_mx_pair": dict(desc="MXFP8 GEMM M8192 N14336 K4096 on CTA pairs (cta_group::2)", unit="TFLOP/s",
                         make=lambda dev, w, r: make_gemm_mx(dev, w, r, 8192, 14336, 4096, 0, cta_pair=True)),
    "gemm_mx_b": dict(desc="MXFP8 GEMM M8192 N4096 K14336 (E8M0 scales on A and B)", unit="TFLOP/s",
                      make=lambda dev, w, r: make_gemm_mx(dev, w, r, 8192, 4096, 14336, 0)),
    "quant": dict(desc="MXFP8 quantiser [8192, 14336] bf16", unit="GB/s",
                  make=lambda dev, w, r: make_quant(dev, w, r, 8192, 14336, 0)),
}


# ------------------------------------------------------------------------------------------------------------
# CPU baseline: the reference's torch fp32 oracle on the host cores, bounded sample of the same workload
# ------------------------------------------------------------------------------------------------------------
def cpu_sample(workload, budget_s=6.0):
    """One bounded sample of the reference's CPU path for ``workload``: ``(work done, seconds, description)``."""
    import numpy as np

    from oracle import c_oracle
    from oracle import reference_math as R

    base = workload
    for stem in ("attn_fwd", "attn_bwd", "attn_gqa", "gemm_bf16", "gemm_mx", "quant"):
        if workload.startswith(stem):
            base = stem
    g = torch.Generator().manual_seed(0)
    if base in ("attn_fwd", "attn_gqa", "attn_bwd"):
        N, d = (32768, 128) if base == "attn_gqa" else (4096, 128)
        rows = 4096  # one (batch, head) slice; for 32768 keys the last 4096 queries of a head
        q = torch.randn(1, 1, rows, d, generator=g)
        k, v = torch.randn(1, 1, N, d, generator=g), torch.randn(1, 1, N, d, generator=g)
        vis = sum(min(N, r + N - rows + 1) for r in range(rows))  # visible (query, key) pairs, bottom-right causal
        slices, used = 0, 0.0
        if base != "attn_bwd":
            while used < budget_s and slices < 8:
                t0 = time.perf_counter()
                R.attention_reference_chunked(q, k, v, True, q_chunk=1024)
                used += time.perf_counter() - t0
                slices += 1
            return 4.0 * vis * d * slices, used, (f"{slices} (batch, head) slices of {rows} queries x {N} keys, causal, "
                                                  "torch fp32 oracle")
        dout = torch.randn(1, 1, rows, d, generator=g).bfloat16().float()
        while used < budget_s and slices < 8:
            qd, kd, vd = (t.clone().requires_grad_() for t in (q, k, v))
            out, _ = R.attention_reference(qd, kd, vd, True)  # the forward that builds the graph is not timed
            t0 = time.perf_counter()
            out.backward(dout)
            used += time.perf_counter() - t0
            slices += 1
        return 10.0 * vis * d * slices, used, (f"{slices} (batch, head) slices of {rows} x {N}, causal: autograd "
                                               "backward through the torch fp32 oracle (its forward untimed)")
    if base == "gemm_bf16":
        m = n = k = 2048
        a, b = torch.randn(m, k, generator=g).bfloat16(), torch.randn(n, k, generator=g).bfloat16()
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < min(budget_s, 4.0) or reps == 0:
            R.gemm_reference(a, b).bfloat16()
            reps += 1
        return 2.0 * m * n * k * reps, time.perf_counter() - t0, f"{reps} x (a.float() @ b.float().T) at 2048^3"
    if base == "gemm_mx":
        n, k = (4096, 14336) if workload.endswith("_b") else (14336, 4096)
        rows = 1024
        a8 = torch.randn(rows, k, generator=g).to(torch.float8_e4m3fn)
        b8 = torch.randn(n, k, generator=g).to(torch.float8_e4m3fn)
        sa = torch.randint(120, 134, (rows, k // 32), generator=g, dtype=torch.uint8)
        sb = torch.randint(120, 134, (n, k // 32), generator=g, dtype=torch.uint8)
        reps, t0 = 0, time.perf_counter()
        while (time.perf_counter() - t0 < budget_s and reps < 8) or reps == 0:
            (R.mx_dequant(a8, sa) @ R.mx_dequant(b8, sb).T).bfloat16()
            reps += 1
        return 2.0 * rows * n * k * reps, time.perf_counter() - t0, (
            f"{reps} slabs of {rows} rows of M: mx_dequant(a, sa) @ mx_dequant(b, sb).T at N{n} K{k}, dequantisation "
            "of both operands inside the timed region")
    if base == "quant":
        m, k = 8192, 14336
        x = torch.randn(m, k, generator=g).bfloat16()
        xb = x.view(torch.int16).numpy().view(np.uint16)
        cores = len(ALL_CPUS)
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < min(budget_s, 4.0) or reps == 0:
            c_oracle.quantize_mx(xb, threads=cores)
            reps += 1
        return m * k * (2 + 1 + 1 / 32) * reps, time.perf_counter() - t0, (
            f"{reps} x C restatement of the quantiser on [{m}, {k}] bf16, {cores} pthreads")
    raise ValueError(workload)


def cpu_baseline(workload, unit, budget_s=6.0):
    os.sched_setaffinity(0, ALL_CPUS)  # the GPU arm may have bound this process to the CPUs near its GPU
    torch.set_num_threads(len(ALL_CPUS))  # torchrun pins OMP_NUM_THREADS=1; the CPU arm may use every core
    cpu_sample(workload, budget_s=0.5)  # warm-up (thread pools, page faults)
    work, seconds, what = cpu_sample(workload, budget_s)
    scale = 1e12 if unit == "TFLOP/s" else 1e9
    return {"value": work / seconds / scale, "unit": unit, "cores": len(ALL_CPUS), "kind": "port", "sample": what}


# ------------------------------------------------------------------------------------------------------------
# measurement of one workload
# ------------------------------------------------------------------------------------------------------------
def measure(name, args, dev, dist, world, rank, clocks):
    from warpy_kernels_b200 import _lib

    wl = WORKLOADS[name]
    w = wl["make"](dev, world, rank)
    stream = torch.cuda.current_stream(dev)
    warmup = max(3, args.warmup)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if wl.get("flush") else None

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, warm, flush=True):
        for _ in range(warm):
            fn()
        barrier()
        if flush_buf is None or not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
            return e0.elapsed_time(e1) / steps
        per = []  # inputs + outputs fit in L2: flush it and time each launch on its own
        for _ in range(steps):
            flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            torch.cuda.synchronize(dev)
            per.append(e0.elapsed_time(e1))
        barrier()
        return sum(per) / len(per)

    kernel_ms = timed(w["step"], args.steps, warmup)
    # sustained: the same launch back to back for about sustain_s seconds; clocks sampled inside this region
    reps = max(10, int(math.ceil(args.sustain_s * 1e3 / max(kernel_ms, 1e-3))))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record(stream)
    for _ in range(reps):
        w["step"]()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    t1 = time.time()
    sustained_ms = e0.elapsed_time(e1) / reps
    clk = clocks.window(t0, t1) if clocks is not None else None
    if clk is not None:
        clk["sampled"] = "inside the sustained region"
    barrier()
    gather_ms = None
    if world > 1 and not w.get("replicas") and w["gather_bytes"]:
        def with_gather():
            w["step"]()
            w["gather"]()
        gather_ms = timed(with_gather, max(3, args.steps // 2), 2)
    # the end-to-end step brings its inputs from the host, so there is nothing to flush
    e2e_ms = timed(w["e2e_step"], max(3, args.steps // 4), 2, flush=False)
    _lib.device_status()
    up_ms, down_ms, floor_ms = copy_floor_ms(dev, w["h2d"], w["d2h"])

    if args.per_rank:
        print(f"[rank {rank}] {name}: burst {kernel_ms:.4f} ms, sustained {sustained_ms:.4f} ms, e2e {e2e_ms:.4f} ms, "
              f"with gather {gather_ms}", file=sys.stderr, flush=True)
    t = torch.tensor([kernel_ms, sustained_ms, e2e_ms, gather_ms or 0.0], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(w["h2d"]), float(w["d2h"])], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the slowest rank's device time
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    kernel_ms, sustained_ms, e2e_ms, gather_ms = t.tolist()
    h2d, d2h = (int(x) for x in sums.tolist())

    scale = 1e12 if wl["unit"] == "TFLOP/s" else 1e9
    replicas = bool(w.get("replicas")) and world > 1
    total_work = w["work"] * (world if replicas else 1)
    rate = lambda ms: total_work / (ms * 1e-3) / scale
    per_gpu = (w["work"] if replicas else w["work_local"]) / (kernel_ms * 1e-3) / scale  # this rank's own kernel rate
    peaks = measured_peaks()
    if w["bound"] == "tensor":
        # no measured fp8 peak exists; the measured bf16 cuBLAS burst figure is doubled for fp8 operands
        peak, unit = peaks["bf16_tflops"] * (2.0 if w["dtype"] == "fp8" else 1.0), "TFLOP/s"
        nominal = NOMINAL[w["dtype"]]
    else:
        peak, unit, nominal = peaks["hbm_gbs"], "GB/s", NOMINAL_HBM_GBS
    res = {
        "workload": wl["desc"], "value": rate(kernel_ms), "unit": wl["unit"], "ms_per_step": kernel_ms,
        "dtype": w["dtype"], "shard": w["shard"],
        "scaling": "weak (replicas)" if replicas else "strong",
        "l2": "explicit flush between launches" if flush_buf is not None else "inputs and outputs larger than L2",
        "roofline": {"bound": w["bound"], "achieved": per_gpu, "peak": peak, "unit": unit, "frac": per_gpu / peak,
                     "traffic": DRAM_TRAFFIC_BYTES.get(name) if world == 1 else None,
                     "peak_source": peaks["source"] + (" bf16 cuBLAS burst x2 for fp8" if w["dtype"] == "fp8" else ""),
                     "frac_of_nominal": per_gpu / nominal},
        "sustained": {"value": rate(sustained_ms), "ms_per_step": sustained_ms, "steps": reps,
                      "seconds": sustained_ms * reps * 1e-3,
                      "sm_mhz_median": clk["sm_mhz"] if clk else None,
                      "ms_x_mhz": sustained_ms * clk["sm_mhz"] if clk and clk["sm_mhz"] else None,
                      "l2": "back-to-back launches, no flush" if flush_buf is not None else "larger than L2"},
        "e2e": {"value": rate(e2e_ms), "unit": wl["unit"], "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "chunks_per_rank": w["e2e_chunks"], "streams": E2E_STREAMS,
                "copies_alone_ms": {"h2d": up_ms, "d2h": down_ms, "both_at_once": floor_ms},
                "note": "copies_alone_ms: rank 0's bytes as one big copy per direction, no kernel: what the link allows"},
        "gpu_launches": w["launches"] * args.steps,
        "clocks": clk,
    }
    if w.get("tuned") is not None:
        res["autotuned"] = w["tuned"]
    if gather_ms:
        res["with_gather"] = {"value": rate(gather_ms), "ms_per_step": gather_ms, "gathered_bytes": w["gather_bytes"],
                              "collective": "one NCCL all_gather_into_tensor per step, after the kernels"}
    del w
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------------------------
def reference_arm(args, rank):
    """The reference's CPU path (its torch fp32 test oracle) on the host cores: K bounded-sample steps."""
    if rank != 0:
        return
    names = [args.workload] if args.workload != "all" else [HEADLINE]
    name = names[0]
    wl = WORKLOADS[name]
    torch.set_num_threads(len(ALL_CPUS))
    scale = 1e12 if wl["unit"] == "TFLOP/s" else 1e9
    budget = 1.0  # seconds of CPU work per step
    for _ in range(max(0, args.warmup)):
        cpu_sample(name, budget_s=0.3)
    work = seconds = 0.0
    what = ""
    for _ in range(max(1, args.steps)):
        w_, s_, what = cpu_sample(name, budget_s=budget)
        work, seconds = work + w_, seconds + s_
    value = work / seconds / scale
    base = {"value": value, "unit": wl["unit"], "cores": len(ALL_CPUS), "kind": "port",
            "sample": f"per step: {what}"}
    line = {
        "impl": "reference", "metric": f"{wl['desc']} throughput", "value": value, "unit": wl["unit"],
        "n_gpus": args.gpus, "steps": max(1, args.steps), "warmup": max(0, args.warmup),
        "ms_per_step": 1e3 * seconds / max(1, args.steps), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_block(wl, args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.workload == "all":
        line["workloads"] = {n: cpu_baseline(n, WORKLOADS[n]["unit"], budget_s=3.0) for n in ALL if n != HEADLINE}
    print(json.dumps(line))


def config_block(wl, world):
    return {"workload": wl["desc"], "l2": "inputs and outputs larger than L2",
            "sharding": "one problem split over the ranks by (batch, KV head), no data-path collective"
            if world > 1 else "single GPU"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="all", choices=["all"] + sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustain-s", type=float, default=1.5, dest="sustain_s")
    ap.add_argument("--per-rank", action="store_true", help="print every rank's own times to stderr")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    numa = bind_near_gpu(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    clocks = ClockLog(local)
    clocks.wait_first()
    names = ALL if args.workload == "all" else [args.workload]
    head_name = names[0]
    results = {}
    for name in names:
        results[name] = measure(name, args, dev, dist, world, rank, clocks if rank == 0 else None)
    clocks.stop()

    if rank == 0:
        head = results[head_name]
        wl = WORKLOADS[head_name]
        line = {
            "metric": f"{wl['desc']} throughput",
            "value": head["value"],
            "unit": wl["unit"],
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(3, args.warmup),
            "ms_per_step": head["ms_per_step"],
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": head["dtype"],
            "data": "synthetic",
            "config": config_block(wl, world),
            "host_binding": numa,
            "roofline": head["roofline"],
            "sustained": head["sustained"],
            "e2e": head["e2e"],
            "gpu_launches": head["gpu_launches"],
            "clocks": head["clocks"],
        }
        if "with_gather" in head:
            line["with_gather"] = head["with_gather"]
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(head_name, wl["unit"], budget_s=12.0)
            for name in names[1:]:
                results[name]["cpu_baseline"] = cpu_baseline(name, WORKLOADS[name]["unit"], budget_s=5.0)
        if len(names) > 1:
            line["workloads"] = {n: results[n] for n in names[1:]}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
