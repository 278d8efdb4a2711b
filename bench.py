#!/usr/bin/env python
"""Benchmark of the MXFP8 sparse-attention path.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...        # the CPU arm: torch dequantise-and-gather on host cores

Workload (config.workload).  N = 1: the reference's headline prefill point -- 65 536 query tokens, 64 heads, one
512-wide MXFP8 KV head, kv_len 16 384, pair-shared rows of 4096 distinct indices (BASELINE configuration 1).
N > 1: BASELINE configuration 4 -- ONE problem of 524 288 query tokens whose query pairs are sharded contiguously
over the ranks (mxdsa_b200.sharding), KV replicated, the last 10 % of every index row -1, nothing exchanged.
Inputs are synthetic with the reference benchmark's distributions (N(0,1) values through the packers); no
dataset exists for this path.  One "step" = one call of the prefill entry point over the rank's tokens.

Printed JSON (one line, rank 0):
  value      whole-job MXFP8 TFLOP/s, algorithmic flops 2*s_q*64*topk*(512+512) per step (x 0.9 with the masked
             tails of configuration 4), inputs resident in HBM, CUDA-event time, max over ranks
  e2e        same metric through the package's host-buffer entry point: pinned Q / KV / indices copied in and
             out / lse / max_logits copied back inside the timed region
  roofline   the attention kernel against the tensor-core roof.  peak = the MXFP8 rate MEASURED on this GPU by an
             issue-only loop of the library's own block-scaled MMA shapes (mxfp8_peak); the fractions of 2 x the
             measured bf16 GEMM rates and of the nominal 4.5 PFLOP/s are given beside it.  traffic = recorded ncu
             DRAM bytes of a small case (profiles/traffic.json), scaled
  cpu_baseline  the torch dequantise-and-gather CPU path on a bounded sample (rank 0, N = 1)
  prefill_sweep / decode_sweep  (N = 1) the reference benchmark's tables: ours and the compiled, unmodified
             reference kernel (oracle/_ref/mxdsa_ext.so, when present) in the same loop, CUDA-graph replay with a
             256 MiB L2 flush before every timed replay, median / P20 / P80, SM clock of each arm
  decode     the decode headline (batch 128, sq 6, main 128 + extra 4096 of 16 384): latency of both kernels,
             gathered GB/s against the measured HBM roof, and the host-buffer e2e latency
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

S_Q, S_KV, TOPK, HEADS = 65536, 16384, 4096, 64
METRIC = "prefill sparse-attn MXFP8 TFLOP/s (sq=65536/GPU, kv=16384, topk=4096)"


def prefill_flops(s_q: int, topk: int) -> float:
    return 2.0 * s_q * HEADS * topk * (512 + 512)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        d = json.load(open(path))
        return dict(source="measured", hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])))
    return dict(source="fallback", hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v == "Active"})
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def make_prefill_inputs(torch, s_q: int, seed: int):
    from mxdsa_b200 import packing as P
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.empty((s_q, HEADS, 528), dtype=torch.uint8, device="cuda")
    for i in range(0, s_q, 1024):
        n = min(1024, s_q - i)
        q[i:i + n] = P.pack_dual_q64(torch.randn(n, HEADS, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((S_KV, 1), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    idx = torch.empty((s_q // 2, 1, TOPK), dtype=torch.int32, device="cuda")
    for i in range(0, s_q // 2, 2048):
        n = min(2048, s_q // 2 - i)
        idx[i:i + n, 0] = torch.rand(n, S_KV, device="cuda", generator=g).argsort(dim=1)[:, :TOPK].int()
    return q, kv, idx, w1, w2


def time_steps(torch, fn, steps, warmup, dist=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return evs[0].elapsed_time(evs[steps]), per


def cpu_baseline(torch, q, kv, idx, w1, w2, target_s=20.0):
    """torch dequantise-and-gather on host cores over a bounded sample of the same workload."""
    from oracle import cpu_baseline as cb
    cores = os.cpu_count() or 1
    k, v = cb.dequant_prefill_kv(kv.cpu(), w1, w2)
    tokens = 32
    cb.prefill_cpu(q[:tokens].cpu(), k, v, idx[:tokens // 2].cpu(), 512 ** -0.5, cores)   # warm the thread pool
    t0 = time.time()
    cb.prefill_cpu(q[:tokens].cpu(), k, v, idx[:tokens // 2].cpu(), 512 ** -0.5, cores)
    probe = max(time.time() - t0, 1e-3)
    tokens = int(min(32768, max(32, 2 * round(tokens * target_s / probe / 2))))
    qs, ids = q[:tokens].cpu(), idx[:tokens // 2].cpu()
    t0 = time.time()
    cb.prefill_cpu(qs, k, v, ids, 512 ** -0.5, cores)
    dt = time.time() - t0
    return dict(value=prefill_flops(tokens, TOPK) / dt / 1e12, unit="TFLOP/s", cores=cores, kind="port",
                sample=f"{tokens} of {q.shape[0]} query tokens at topk={TOPK}, {dt:.1f} s, torch fp32 "
                       f"dequantise-and-gather on {cores} threads"), dt


def run_reference_arm(args):
    """The CPU arm.  The reference has no CPU implementation of its kernels; the host-core
    comparator that its inputs define is the torch dequantise-and-gather path (oracle port)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from mxdsa_b200 import packing as P
    from oracle import cpu_baseline as cb
    torch.manual_seed(0)
    cores = os.cpu_count() or 1
    tokens = 2048      # upper bound of the per-step sample; cut down below if the box is slow
    q = P.pack_dual_q64(torch.randn(tokens, HEADS, 512))[0]
    kvf, w1, w2 = P.make_rank1_kv((S_KV, 1))
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    idx = torch.stack([torch.randperm(S_KV)[:TOPK] for _ in range(tokens // 2)]).int().view(tokens // 2, 1, TOPK)
    # N > 1 is BASELINE configuration 4 (this arm's config follows the other arm's): the last 10 % of every index row
    # is -1, and only the attended 90 % is counted
    config4 = args.gpus > 1
    counted = 0.9 if config4 else 1.0
    if config4:
        idx[:, :, TOPK - TOPK // 10:] = -1
    k, v = cb.dequant_prefill_kv(kv, w1, w2)
    t0 = time.time()
    cb.prefill_cpu(q[:8], k, v, idx[:4], 512 ** -0.5, cores)
    probe = max(time.time() - t0, 1e-3) / 8
    # bound the whole run to a few minutes: (steps + warmup) * sample_time <= ~120 s
    budget = 120.0 / max(args.steps + args.warmup, 1)
    tokens = int(min(tokens, max(2, 2 * int(budget / probe / 2))))
    fn = lambda: cb.prefill_cpu(q[:tokens], k, v, idx[:tokens // 2], 512 ** -0.5, cores)
    for _ in range(args.warmup):
        fn()
    t0 = time.time()
    for _ in range(args.steps):
        fn()
    dt = (time.time() - t0) / args.steps
    val = prefill_flops(tokens, TOPK) * counted / dt / 1e12
    sample = (f"{tokens} query tokens per step at topk={TOPK}, kv_len={S_KV}"
              f"{', last 10 % of every index row -1 (counted x 0.9)' if config4 else ''}: torch fp32 dequantise-and-gather "
              f"(oracle port; the reference ships no CPU implementation) on {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if config4 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": (f"prefill sq={args.total_sq} kv_len=16384 topk=4096 heads=64 dim=512, last 10% of every "
                                "index row = -1 (BASELINE configuration 4), bounded sample on rank 0's host cores"
                                if config4 else
                                "prefill sq=65536 kv_len=16384 topk=4096 heads=64 dim=512 (BASELINE configuration 1 at "
                                "its headline topk), bounded sample"),
                   "sample_tokens": tokens, "counted_flop_fraction": counted},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def load_reference():
    """The compiled, unmodified reference extension (oracle/_ref/mxdsa_ext.so), or None where it is not present."""
    import importlib.util
    path = os.path.join(ROOT, "oracle", "_ref", "mxdsa_ext.so")
    if not os.path.isfile(path):
        return None
    try:
        spec = importlib.util.spec_from_file_location("mxdsa_ext", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        return ref
    except Exception:   # the comparator is optional
        return None


_FLUSH = {}


def graph_latency(torch, fn, timed=20, warm=5):
    """The reference benchmark's method (tests/benchmark.py:41-67): a few eager calls, capture into a CUDA graph,
    warm replays, then timed replays with 256 MiB written before each one so that nothing of the previous replay
    is left in L2.  Returns median / P20 / P80 in milliseconds and the clocks sampled during the timed replays."""
    dev = torch.cuda.current_device()
    if dev not in _FLUSH:
        _FLUSH[dev] = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush = _FLUSH[dev]
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    ts = []
    with ClockSampler(dev) as clocks:
        for _ in range(timed):
            flush.zero_()
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(e))
    ts.sort()
    pick = lambda f: ts[min(len(ts) - 1, int(f * len(ts)))]
    c = clocks.summary()
    return dict(ms=statistics.median(ts), p20_ms=pick(0.2), p80_ms=pick(0.8), sm_mhz=c["sm_mhz"], reasons=c["reasons"])


def mxfp8_peak(torch):
    """Issue-only rate of the library's own block-scaled E4M3 MMA shapes on this GPU (mxdsa_selftest_mma_rate):
    every CTA pair issues tcgen05.mma kind::mxf8f6f4 back to back on operands resident in shared memory.  The mean
    of the QK shape (N = 128) and the PV shape (N = 256) -- an attention tile spends the same flops in each -- is
    the measured MXFP8 roof that the attention kernel's fraction is quoted against."""
    from mxdsa_b200 import capi
    L = capi.lib()
    data = torch.randint(0, 255, (1 << 17,), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    out = {}
    for n in (128, 256):
        iters = 6000 if n == 128 else 3000         # about 8 ms each: long enough to settle under the power cap
        capi.check(L.mxdsa_selftest_mma_rate(data.data_ptr(), n, 200, st), "mma rate probe")
        torch.cuda.synchronize()
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        capi.check(L.mxdsa_selftest_mma_rate(data.data_ptr(), n, iters, st), "mma rate probe")
        e.record()
        torch.cuda.synchronize()
        out[n] = (sms // 2) * iters * 64 * 2.0 * 128 * n * 32 / a.elapsed_time(e) / 1e9
    # equal flops in each shape -> harmonic mean of the two rates
    both = 2.0 / (1.0 / out[128] + 1.0 / out[256])
    return dict(tflops=both, qk_shape_tflops=out[128], pv_shape_tflops=out[256],
                how="issue-only tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale loop, M128 x N128/N256 x K32, "
                    "operands in shared memory, all SMs, CUDA-event time")


def prefill_sweep(torch, M, ref, q, kv, idx_full, w1, w2, topks, peak_tflops):
    """ours and the reference kernel at every topk of the list, same inputs, same loop, graph replay + L2 flush."""
    sc = 512 ** -0.5
    s_q = q.shape[0]
    rows = []
    for topk in topks:
        idx = idx_full[:, :, :topk].contiguous()
        ours = graph_latency(torch, lambda: M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None))
        row = dict(topk=topk, ours=ours, tflops=prefill_flops(s_q, topk) / ours["ms"] / 1e9)
        row["frac_of_measured_mxfp8_peak"] = row["tflops"] / peak_tflops
        if ref is not None:
            r = graph_latency(torch, lambda: ref.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, list(w1), list(w2),
                                                                                      None, None))
            row["reference"] = r
            row["ours_over_reference_time"] = ours["ms"] / r["ms"]
        rows.append(row)
        del idx
    return rows


def make_decode_inputs(torch, b, extra_max):
    """Reference tests/benchmark.py:119-147: per request a main cache of 128 keys (2 pages, topk 128, all of them,
    permuted) and an extra cache of 16 384 keys (256 pages) of its own; indices are pool offsets."""
    from mxdsa_b200 import packing as P
    s_q = 6
    g = torch.Generator(device="cuda").manual_seed(3)
    q = P.pack_dual_q64(torch.randn(b * s_q, HEADS, 512, device="cuda", generator=g))[0].view(b, s_q, HEADS, 528)
    kvf, w1, w2 = P.make_rank1_kv((2 * b, 64, 1), device="cuda", generator=g)
    kv = P.pack_dual_decode_kv_pages(kvf)[0]
    pool = P.pack_dual_decode_kv_pages(torch.randn(256, 64, 1, 512, device="cuda", generator=g))[0]
    ekv = pool.repeat(b, 1, 1, 1)                      # b x 8.65 MB: every request has its own pages
    off = torch.arange(b, device="cuda", dtype=torch.int32)[:, None, None]
    idx = (torch.rand(b * s_q, 128, device="cuda", generator=g).argsort(1).int().view(b, s_q, 128) + off * 128).contiguous()
    eidx = (torch.rand(b * s_q, 16384, device="cuda", generator=g).argsort(1)[:, :extra_max].int()
            .view(b, s_q, extra_max) + off * 16384).contiguous()
    return q, kv, idx, ekv, eidx, w1, w2


def decode_sweep(torch, M, ref, peaks, batches, extras):
    """Decode latency (attention + combine, scheduling info computed once and reused) for every batch / extra topk:
    ours and the reference kernel, graph replay + L2 flush; gathered GB/s against the measured HBM roof."""
    sc = 512 ** -0.5
    out = []
    for b in batches:
        q, kv, idx, ekv, eidx_full, w1, w2 = make_decode_inputs(torch, b, max(extras))
        pairs = (q.shape[1] + 1) // 2
        for extra in extras:
            ek, ei = (ekv, eidx_full[:, :, :extra].contiguous()) if extra > 0 else (None, None)
            first = M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, ek, ei, None, 512, 512, sc, w1, w2)
            meta, splits = first[2], first[3]
            ours = graph_latency(torch, lambda: M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, meta, splits, ek, ei,
                                                                               None, 512, 512, sc, w1, w2), timed=30)
            gathered = b * pairs * (128 + extra) * 528       # each selected row once per query pair
            gbs = gathered / ours["ms"] / 1e6
            row = dict(b=b, extra_topk=extra, ours=ours, latency_us=ours["ms"] * 1e3, gathered_bytes=gathered, gbs=gbs,
                       frac_of_measured_hbm=gbs / peaks["hbm_gbs"])
            # the opt-in operator without a combine pass (whole requests per part; one launch, no scratch)
            wf = M.dual_mxfp8_sparse_decode_fwd_whole(q, kv, idx, None, None, None, None, ek, ei, None, 512, 512, sc, w1, w2)
            whole = graph_latency(torch, lambda: M.dual_mxfp8_sparse_decode_fwd_whole(q, kv, idx, None, None, wf[2], wf[3], ek,
                                                                                     ei, None, 512, 512, sc, w1, w2), timed=30)
            row["whole_request_latency_us"] = whole["ms"] * 1e3
            if ref is not None:
                rf = ref.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, ek, ei, None, 512, 512, sc,
                                                      list(w1), list(w2))
                r = graph_latency(torch, lambda: ref.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, rf[2], rf[3], ek, ei,
                                                                                  None, 512, 512, sc, list(w1), list(w2)),
                                  timed=30)
                row["reference"] = r
                row["reference_latency_us"] = r["ms"] * 1e3
                row["ours_over_reference_time"] = ours["ms"] / r["ms"]
            out.append(row)
        del q, kv, idx, ekv, eidx_full
        torch.cuda.empty_cache()
    return out


def decode_e2e(torch, M, steps=10):
    """Decode headline through host buffers: the KV caches live in HBM (they are the serving state), what a step
    brings from the host is the packed queries and the index rows, what goes back is out and lse."""
    sc = 512 ** -0.5
    b, extra = 128, 4096
    q, kv, idx, ekv, eidx, w1, w2 = make_decode_inputs(torch, b, extra)
    first = M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, ekv, eidx, None, 512, 512, sc, w1, w2)
    meta, splits = first[2], first[3]
    hq, hidx, heidx = q.cpu().pin_memory(), idx.cpu().pin_memory(), eidx.cpu().pin_memory()
    h_out = torch.empty(first[0].shape, dtype=torch.bfloat16).pin_memory()
    h_lse = torch.empty((b, 6, HEADS), dtype=torch.float32).pin_memory()

    def step():
        dq, di, de = hq.cuda(non_blocking=True), hidx.cuda(non_blocking=True), heidx.cuda(non_blocking=True)
        o, lse, _, _ = M.dual_mxfp8_sparse_decode_fwd(dq, kv, di, None, None, meta, splits, ekv, de, None, 512, 512, sc,
                                                      w1, w2)
        h_out.copy_(o, non_blocking=True)
        h_lse.copy_(lse.transpose(1, 2), non_blocking=True)

    total, _ = time_steps(torch, step, steps, 3)
    ms = total / steps
    return dict(latency_us=ms * 1e3, h2d_bytes_per_step=hq.numel() + 4 * (hidx.numel() + heidx.numel()),
                d2h_bytes_per_step=2 * h_out.numel() + 4 * h_lse.numel(),
                how="pinned q / index rows copied in, attention + combine, out / lse copied back; KV caches resident in HBM")


def pack_headline(torch, peaks, steps, warmup):
    """The step in front of the path: fused quantise-and-pack of Q (16 384 tokens x 64 heads of bf16
    activations, 1.07 GB in, 0.55 GB out) and of a 65 536-token KV cache, against the HBM roof; the torch
    kernel chain that the reference's helper launches for the same tensor is timed beside it."""
    from mxdsa_b200 import packing as P, quantize as Z
    g = torch.Generator(device="cuda").manual_seed(9)
    out = {}
    for name, shape, fused, chain in (
            ("pack_q", (16384, HEADS, 512), Z.pack_dual_q64, lambda t: P.pack_dual_q64(t)[0]),
            ("pack_kv", (65536 * 8, 1, 512), Z.pack_dual_prefill_kv64, lambda t: P.pack_dual_prefill_kv64(t)[0])):
        x = torch.randn(shape, device="cuda", generator=g).bfloat16()
        rows = x.numel() // 512
        alg_bytes = rows * (512 * 2 + 528)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

        def timed(fn, n):
            for _ in range(warmup):
                fn(x)
            ts = []
            for _ in range(n):
                flush.zero_()
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn(x)
                e.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(e))
            return statistics.median(ts)

        ms = timed(fused, steps)
        ms_chain = timed(chain, 3)
        gbs = alg_bytes / ms / 1e6
        out[name] = dict(rows=rows, ms=ms, torch_chain_ms=ms_chain, algorithmic_bytes=alg_bytes,
                         roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                       frac=gbs / peaks["hbm_gbs"], traffic=None))
        del x
        torch.cuda.empty_cache()
    return out


def topk_headline(torch, peaks, steps, warmup):
    """The producer of the path's other input: index selection for 8192 query pairs (score rows of both
    tokens, 16 384 keys each, 1.07 GB read) -> 4096 ascending indices per pair, against the HBM roof;
    torch.topk + sort on the pair-merged scores is timed beside it."""
    from mxdsa_b200.indexer import select_topk_indices
    g = torch.Generator(device="cuda").manual_seed(11)
    pairs, s_kv, topk = 8192, S_KV, TOPK
    scores = torch.randn((2 * pairs, s_kv), device="cuda", generator=g)
    alg_bytes = 2 * pairs * s_kv * 4 + pairs * topk * 4
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def chain(x):
        return torch.topk(torch.maximum(x[0::2], x[1::2]), topk, dim=1).indices.sort(dim=1).values.int()

    def timed(fn, n):
        for _ in range(warmup):
            fn(scores)
        ts = []
        for _ in range(n):
            flush.zero_()
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(scores)
            e.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(e))
        return statistics.median(ts)

    ms = timed(lambda x: select_topk_indices(x, topk, pair=True), steps)
    ms_chain = timed(chain, 3)
    gbs = alg_bytes / ms / 1e6
    return dict(pairs=pairs, s_kv=s_kv, topk=topk, ms=ms, torch_chain_ms=ms_chain, algorithmic_bytes=alg_bytes,
                roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                              frac=gbs / peaks["hbm_gbs"],
                              # DRAM bytes of one launch: the recorded ncu capture (2048 pairs), scaled by the pairs
                              traffic=(recorded_traffic("topk_2048_pairs") or {}).get("dram_bytes", 0) * pairs / 2048 or None,
                              traffic_source="profiles/traffic.json (a record, not measured in this run)"))


def run_profile_case(which: str):
    """Three launches of a small case of one kernel: inputs larger than L2, well under a GB on the
    device, each launch a millisecond or two -- the size a multi-pass profiler capture wants."""
    import torch
    import mxdsa_b200 as M
    torch.cuda.set_device(0)
    if which == "prefill":
        s_q = 4096                                     # Q = 138 MB; same kv_len / topk as the headline
        q, kv, idx, w1, w2 = make_prefill_inputs(torch, s_q, seed=100)
        for _ in range(3):
            M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
        case = {"kernel": "mxdsa_attn_kernel<prefill,128>", "s_q": s_q, "kv_len": S_KV, "topk": TOPK}
    elif which == "topk":
        from mxdsa_b200.indexer import select_topk_indices
        scores = torch.randn((2 * 2048, S_KV), device="cuda")              # 268 MB of scores
        for _ in range(3):
            select_topk_indices(scores, TOPK, pair=True)
        case = {"kernel": "mxdsa_topk_rows_kernel<2>", "pairs": 2048, "s_kv": S_KV, "topk": TOPK}
    elif which == "pack":
        from mxdsa_b200 import quantize as Z
        x = torch.randn((4096, HEADS, 512), device="cuda").bfloat16()     # 268 MB in, 138 MB out
        kv = torch.randn((262144, 1, 512), device="cuda").bfloat16()
        for _ in range(3):
            Z.pack_dual_q64(x)
            Z.pack_dual_prefill_kv64(kv)
        case = {"kernel": "mxdsa_pack_rows_kernel<bf16, Q> and <bf16, KV>", "rows": 262144}
    else:
        from mxdsa_b200 import packing as P
        b, s_q, extra = 32, 6, 4096                    # 32 requests x 8.65 MB of private extra pages = 277 MB
        g = torch.Generator(device="cuda").manual_seed(3)
        q = P.pack_dual_q64(torch.randn(b * s_q, HEADS, 512, device="cuda", generator=g))[0].view(b, s_q, HEADS, 528)
        kvf, w1, w2 = P.make_rank1_kv((2 * b, 64, 1), device="cuda", generator=g)
        kv = P.pack_dual_decode_kv_pages(kvf)[0]
        pool = P.pack_dual_decode_kv_pages(torch.randn(256, 64, 1, 512, device="cuda", generator=g))[0]
        ekv = pool.repeat(b, 1, 1, 1)
        off = torch.arange(b, device="cuda", dtype=torch.int32)[:, None, None]
        idx = (torch.rand(b * s_q, 128, device="cuda", generator=g).argsort(1).int().view(b, s_q, 128) + off * 128).contiguous()
        eidx = (torch.rand(b * s_q, 16384, device="cuda", generator=g).argsort(1)[:, :extra].int()
                .view(b, s_q, extra) + off * 16384).contiguous()
        for _ in range(3):
            M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, ekv, eidx, None, 512, 512, 512 ** -0.5,
                                           w1, w2)
        case = {"kernel": "mxdsa_attn_kernel<decode,64> + mxdsa_combine_kernel", "b": b, "s_q": s_q, "extra_topk": extra}
    torch.cuda.synchronize()
    M.device_fault()
    print(json.dumps({"profile_case": which, **case, "launches": 3}))


def recorded_traffic(key: str):
    """DRAM bytes of one launch of a small case, as captured by ncu (profiles/traffic.json: a record, not a
    measurement of this run).  Returns the entry or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        return json.load(open(path)).get(key)
    except (OSError, ValueError):
        return None


def spread_cpu_affinity(local: int, world: int):
    """One slice of the host cores per rank, so that the ranks' copy threads and pinned buffers (first touch) do
    not pile up on the same cores and memory controller.  Returns the cores this rank now runs on."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        if world > 1 and len(cores) >= world:
            n = len(cores) // world
            mine = cores[local * n:(local + 1) * n]
            os.sched_setaffinity(0, mine)
            return mine
        return cores
    except (AttributeError, OSError):
        return []


def make_config4_shard(torch, rank: int, world: int, total_sq: int):
    """BASELINE configuration 4: ONE prefill problem of total_sq query tokens whose query pairs are sharded
    contiguously over the ranks (mxdsa_b200.sharding), KV replicated; the last 10 % of every index row is -1."""
    from mxdsa_b200 import sharding
    t0, t1 = sharding.shard_query_tokens(total_sq, rank, world)
    q, kv, idx, w1, w2 = make_prefill_inputs(torch, t1 - t0, seed=4000 + rank)
    idx[:, :, TOPK - TOPK // 10:] = -1
    return (t0, t1), q, kv, idx, w1, w2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sq", type=int, default=S_Q, help="query tokens of the N = 1 workload (default: the headline 65536)")
    ap.add_argument("--total-sq", type=int, default=524288, help="query tokens of the sharded problem at N > 1")
    ap.add_argument("--no-extras", action="store_true", help="only the headline line: no e2e, sweeps, decode, CPU baseline")
    ap.add_argument("--full-sweep", action="store_true", help="all 32 prefill topk points and all 33 decode extra-topk points")
    ap.add_argument("--profile-case", choices=["prefill", "decode", "pack", "topk"], default=None,
                    help="launch a small case of one kernel a few times and exit (for profiler captures; no timing)")
    args = ap.parse_args()
    if args.profile_case:
        return run_profile_case(args.profile_case)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import mxdsa_b200 as M
    from mxdsa_b200 import host, sharding
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cores = spread_cpu_affinity(local, world)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = measured_peaks()
    sc = 512 ** -0.5
    if world == 1:
        s_q = args.sq
        q, kv, idx, w1, w2 = make_prefill_inputs(torch, s_q, seed=100)
        counted = 1.0
        workload = (f"prefill sq={s_q} kv_len={S_KV} topk={TOPK} heads=64 dim=512 (BASELINE configuration 1 at its "
                    f"headline topk), one GPU")
        scaling = "weak"
    else:
        (t0, t1), q, kv, idx, w1, w2 = make_config4_shard(torch, rank, world, args.total_sq)
        s_q = t1 - t0
        counted = 0.9          # the masked tail of every index row does no counted work
        workload = (f"prefill sq={args.total_sq} kv_len={S_KV} topk={TOPK} heads=64 dim=512, last 10% of every index "
                    f"row = -1 (BASELINE configuration 4): query pairs sharded contiguously over {world} GPUs "
                    f"({s_q} tokens on rank 0), KV replicated, no collective on the timed path")
        scaling = "strong"
    fn = lambda: M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None)

    with ClockSampler(local) as clocks:
        total_ms, per = time_steps(torch, fn, args.steps, args.warmup, dist)
    M.device_fault()
    job_ms = sharding.max_over_ranks(total_ms)
    ms_per_step = job_ms / args.steps
    total_tokens = s_q if world == 1 else args.total_sq
    flops = prefill_flops(total_tokens, TOPK) * counted
    value = flops / ms_per_step / 1e9

    # ---- roofline of the attention kernel (the only kernel of a prefill step)
    kern_ms = statistics.median(per)
    achieved = prefill_flops(s_q, TOPK) * counted / kern_ms / 1e9
    mx = mxfp8_peak(torch) if rank == 0 else None
    peak = mx["tflops"] if mx else 2.0 * peaks["bf16_tflops_sustained"]
    rec = recorded_traffic("prefill_sq4096_topk4096")
    traffic = None
    if rec:   # the KV bytes do not grow with the query tokens; the rest does
        traffic = (rec["dram_read_bytes"] - S_KV * 528 + rec["dram_write_bytes"]) * (s_q / rec["s_q"]) + S_KV * 528
    roofline = dict(bound="tensor", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak, traffic=traffic,
                    traffic_source=("profiles/traffic.json (ncu capture of `bench.py --profile-case prefill`, scaled by "
                                    "query tokens; a record, not measured in this run)") if rec else None,
                    algorithmic_bytes=s_q * (HEADS * 528 + TOPK * 2 + HEADS * 512 * 2 + HEADS * 8) + S_KV * 528,
                    peak_source="measured: issue-only block-scaled E4M3 MMA loop of this library (mxfp8_peak)" if mx
                    else f"2 x {peaks['source']} sustained bf16 GEMM TFLOP/s",
                    frac_of_2x_sustained_bf16=achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                    frac_of_2x_burst_bf16=achieved / (2.0 * peaks["bf16_tflops"]),
                    frac_of_nominal_4500=achieved / 4500.0)
    if mx:
        roofline["mxfp8_peak"] = mx

    result = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "latency_us": ms_per_step * 1e3,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "mxfp8(e4m3+ue8m0)->f32",
        "data": "synthetic",
        "config": {"workload": workload, "tokens_per_gpu": s_q, "counted_flop_fraction": counted,
                   "l2": "inputs (Q 2.2 GB, indices 0.5 GB per 65536 tokens) are larger than L2; KV (8.65 MB) is "
                         "L2-resident by design of the workload",
                   "note": ("N = 1 is configuration 1 (the metric's configuration); N > 1 is configuration 4, whose "
                            "masked 10 % of every index row is gathered and multiplied like the rest but not counted")},
        "roofline": roofline, "gpu_launches": args.steps,
    }
    if rank == 0:
        result["clocks"] = clocks.summary()

    if not args.no_extras:
        # ---- end to end through the package's host-buffer entry point: every byte crosses PCIe inside the step
        hq, hkv, hidx = q.cpu().pin_memory(), kv.cpu().pin_memory(), idx.cpu().pin_memory()
        h_out = torch.empty((s_q, HEADS, 512), dtype=torch.bfloat16).pin_memory()
        h_lse = torch.empty((s_q, HEADS), dtype=torch.float32).pin_memory()
        h_mxl = torch.empty((s_q, HEADS), dtype=torch.float32).pin_memory()
        e2e_step = lambda: host.prefill_from_host(hq, hkv, hidx, sc, w1, w2, h_out, h_mxl, h_lse)
        e_steps = min(args.steps, 3)
        e_total, _ = time_steps(torch, e2e_step, e_steps, 1, dist)
        e_ms_rank = e_total / e_steps
        e_ms = sharding.max_over_ranks(e_total) / e_steps
        h2d = hq.numel() + hkv.numel() + hidx.numel() * 4
        d2h = h_out.numel() * 2 + h_lse.numel() * 4 + h_mxl.numel() * 4
        result["e2e"] = {"value": flops / e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e_ms,
                         "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e_steps,
                         "rank0_h2d_plus_d2h_gbs": (h2d + d2h) / e_ms_rank / 1e6,
                         "slowest_rank_over_rank0": e_ms / e_ms_rank, "rank0_cores": len(cores),
                         "how": "mxdsa_b200.host.prefill_from_host: chunks of 8192 tokens, H2D / attention / D2H of "
                                "neighbouring chunks overlapped on three streams; ranks run on disjoint host cores"}
        del hq, hidx, h_out
        if rank == 0 and world == 1:
            ref = load_reference()
            result["cpu_baseline"], _ = cpu_baseline(torch, q, kv, idx, w1, w2)
            # ---- the BASELINE tables: ours and the reference kernel in the same loop (graph replay, L2 flushed)
            topks = list(range(128, 4097, 128)) if args.full_sweep else [128, 256, 512, 1024, 2048, 3968, 4096]
            # The reference kernel forms the address of a token's Q scales as int32 token * int32 stride
            # (reference csrc/attention/prefill_kernel.cuh:266-269), which overflows from token 63 551 on: at the
            # headline's 65 536 tokens it reads 2 GiB below the tensor (an illegal address on this pool unless that
            # memory happens to be mapped).  It is therefore run on at most 63 488 tokens; the sweep uses 16 384.
            n_sw = min(16384, s_q)
            result["prefill_sweep"] = dict(s_q=n_sw, kv_len=S_KV, rows=prefill_sweep(
                torch, M, ref, q[:n_sw], kv, idx[:n_sw // 2], w1, w2, topks, peak))
            if ref is not None:
                n_ref = min(63488, s_q)
                head = prefill_sweep(torch, M, ref, q[:n_ref], kv, idx[:n_ref // 2], w1, w2, [TOPK], peak)[0]
                result["reference_gpu"] = dict(what=f"unmodified reference kernel (sm_100f build) on the first {n_ref} query "
                                                    "tokens of the same inputs, ours beside it in the same loop "
                                                    "(CUDA-graph replay, L2 flushed); above 63 550 tokens the reference's "
                                                    "int32 address arithmetic overflows",
                                               s_q=n_ref, ms_per_step=head["reference"]["ms"],
                                               value=prefill_flops(n_ref, TOPK) / head["reference"]["ms"] / 1e9,
                                               unit="TFLOP/s", ours_ms_same_method=head["ours"]["ms"],
                                               ours_value_same_method=head["tflops"],
                                               reference_sm_mhz=head["reference"]["sm_mhz"], ours_sm_mhz=head["ours"]["sm_mhz"])
            del q, idx
            torch.cuda.empty_cache()
            extras = list(range(0, 4097, 128)) if args.full_sweep else [0, 512, 2048, 4096]
            result["decode_sweep"] = decode_sweep(torch, M, ref, peaks, (64, 128), extras)
            head = [r for r in result["decode_sweep"] if r["b"] == 128 and r["extra_topk"] == 4096][0]
            drec = recorded_traffic("decode_b32_extra4096")
            dtraffic = None
            if drec:
                dtraffic = (drec["dram_read_bytes"] + drec["dram_write_bytes"]) * (128.0 / drec["b"])
            result["decode"] = dict(workload="decode b=128 sq=6 main 128 + extra 4096 of 16384 (BASELINE configuration 3)",
                                    latency_us=head["latency_us"], reference_latency_us=head.get("reference_latency_us"),
                                    gathered_bytes=head["gathered_bytes"], gbs=head["gbs"],
                                    roofline=dict(bound="hbm", achieved=head["gbs"], peak=peaks["hbm_gbs"], unit="GB/s",
                                                  frac=head["gbs"] / peaks["hbm_gbs"], traffic=dtraffic,
                                                  traffic_source="profiles/traffic.json (ncu capture of `bench.py "
                                                                 "--profile-case decode`, b = 32, scaled by requests)"
                                                  if drec else None),
                                    launches_per_step=2, e2e=decode_e2e(torch, M))
            torch.cuda.empty_cache()
            result["pack"] = pack_headline(torch, peaks, 10, 3)
            result["topk_select"] = topk_headline(torch, peaks, 10, 3)
            result["gpu_launches_note"] = "prefill step = 1 attention kernel; decode step = attention + combine"
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
