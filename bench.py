#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: KV append + split-K GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one decode token: for every layer, append the token's K/V to the cache, then
attend over the whole context.  The default workload is the FP8 Qwen3-8B-like case
(36 layers, 32 q / 8 kv / 128, batch 1, context 8192, 16 splits).  Prints ONE JSON line.

value     device-timed, inputs resident in HBM, microseconds per token per layer
e2e       the same from pinned HOST buffers through vfkv_decode_token_host_submit / _wait with two
          tokens in flight (every step's copies inside the timed region); the synchronous
          vfkv_decode_token_host is reported beside it
roofline  the attention split kernel: algorithmic KV bytes per launch / its mean launch time,
          against the measured HBM copy bandwidth
cpu_baseline  the CPU oracle (a C port of the reference's CPU attention and store code, the
          reference itself is Rust and cannot be built here) on a bounded sample

Under torchrun every rank runs the headline workload on its own sequence(s) and GPU (sharding
by sequence, no collective on the data path; times are the max over ranks), and the two sharded
configurations are measured as well -- the long context cut by position over the ranks (partials
exchanged by peer stores inside the attention kernel, output checked against one GPU), the same
context cut by kv-head group (no exchange) and the ragged batch of 64 dealt out by sequence --
each beside its one-GPU time from the same run.  They
are the last key of the line ("sharded").
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: n_layers, Hq, Hkv, D, dtype, batch, context, n_splits, window pattern, softcap
    "qwen3_8b_fp8_ctx8192_b1": dict(n_layers=36, hq=32, hkv=8, d=128, dtype="F8", batch=1, ctx=8192,
                                    n_splits=16, softcap=0.0, windows=None),
    "llama3_8b_f16_ctx2048_b1": dict(n_layers=32, hq=32, hkv=8, d=128, dtype="F16", batch=1, ctx=2048,
                                     n_splits=0, softcap=0.0, windows=None),
    # two layers each: consecutive launches then touch different layers, as in a forward pass
    "batch64_fp8_ctx8192": dict(n_layers=2, hq=32, hkv=8, d=128, dtype="F8", batch=64, ctx=8192,
                                n_splits=0, softcap=0.0, windows=None),
    "batch64_fp8_ragged_512_16384": dict(n_layers=2, hq=32, hkv=8, d=128, dtype="F8", batch=64, ctx=16384,
                                         n_splits=0, softcap=0.0, windows=None, ragged=(512, 16384)),
    "gemma_f16_ctx32768_b8": dict(n_layers=6, hq=16, hkv=8, d=256, dtype="F16", batch=8, ctx=32768,
                                  n_splits=0, softcap=50.0, windows=[1024, 1024, 1024, 1024, 1024, 0]),
    "long_fp8_ctx131072_b1": dict(n_layers=8, hq=64, hkv=8, d=128, dtype="F8", batch=1, ctx=131072,
                                  n_splits=0, softcap=0.0, windows=None, shard="positions"),
}
DEFAULT_WORKLOAD = "qwen3_8b_fp8_ctx8192_b1"
METRIC = "kv_append_decode_attn_us_per_token_layer"
UNIT = "us/token/layer"
ES = {"F32": 4, "F16": 2, "F8": 1}
DT = {"F32": 0, "F16": 1, "F8": 2}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel, from the ncu
# captures summarised under profiles/ (one file per kernel and workload; a capture cannot run inside
# a timed run, so these are read off the summaries; workloads without a capture report null)
NCU_TRAFFIC_BYTES = {"qwen3_8b_fp8_ctx8192_b1": 16_900_000, "batch64_fp8_ctx8192": 1_079_900_000}


def config_of(name, w):
    """The workload as both arms print it (identical dictionaries, so the two lines can be matched)."""
    return {"workload": name, "n_layers": w["n_layers"], "n_q_heads": w["hq"], "n_kv_heads": w["hkv"],
            "head_dim": w["d"], "kv_dtype": w["dtype"], "batch_per_gpu": w["batch"], "context": w["ctx"],
            "n_splits": w["n_splits"], "softcap": w["softcap"], "windows": w["windows"],
            "ragged": list(w["ragged"]) if "ragged" in w else None}


def algorithmic_bytes(w, lens, layer):
    """Bytes one layer-step must move: KV rows read + Q + new K/V (f32) in; appended rows + O out."""
    e = ES[w["dtype"]]
    win = (w["windows"] or [0] * w["n_layers"])[layer]
    total = 0
    for L in lens:
        eff = min(int(L), win) if win else int(L)
        total += 2 * eff * w["hkv"] * w["d"] * e + w["hq"] * w["d"] * 4 + 2 * w["hkv"] * w["d"] * 4
        total += 2 * w["hkv"] * w["d"] * e + w["hq"] * w["d"] * 4
    return total


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Dense bf16 TFLOP/s of a library GEMM timed alone (MEASURED_PEAKS.json), else the fallback figure."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path)).get("bf16_tflops", 1590.0))
    return 1590.0


def copy_bandwidth_here(n_bytes=1 << 31, reps=10):
    """The same measurement MEASURED_PEAKS.json's hbm_gbs comes from (a device-to-device copy of
    bf16 elements, read + write bytes, best of `reps`, CUDA events), on the GPU this run got: boards of
    one pool differ by several per cent, and the fractions printed here divide by the pool's figure."""
    import torch
    a = torch.empty(n_bytes // 2, dtype=torch.bfloat16, device="cuda").normal_()
    b = torch.empty_like(a)
    best = 0.0
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        b.copy_(a)
        e1.record()
        torch.cuda.synchronize()
        best = max(best, 2.0 * n_bytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    del a, b
    torch.cuda.empty_cache()
    return best


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._halt.wait(0.02)

    def finish(self):
        self._halt.set()
        self.join(timeout=1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ----------------------------------------------------------------------------------------------
def run_reference(args, w, rank, world):
    """The reference arm: the CPU code of the path (C port of the reference's CPU attention,
    tests/correctness.rs:2567-2617, and store, fp8_ext.rs:126-211) on all host threads, on a
    bounded sample of the same workload."""
    if rank != 0:
        return
    import oracle
    cores = oracle.use_all_host_threads()           # before anything is timed: launchers export OMP_NUM_THREADS=1
    dt = DT[w["dtype"]]
    rng = np.random.default_rng(1234)
    lens = make_lens(w, rng)
    # bounded sample: at most `layers` distinct layer slabs, cycled; each step = one layer-step
    b = min(w["batch"], 8)
    lens = lens[:b]
    slab = int(max(lens))
    st = oracle.NP_DTYPE[dt]
    n_slabs = 2
    ks, vs = [], []
    for _ in range(n_slabs):
        kf = rng.standard_normal((b, slab, w["hkv"], w["d"]), dtype=np.float32)
        ks.append(oracle.store(kf, dt).reshape(kf.shape).astype(st, copy=False))
        vs.append(oracle.store(kf[::-1].copy(), dt).reshape(kf.shape).astype(st, copy=False))
    q = rng.standard_normal((b, w["hq"], w["d"]), dtype=np.float32)
    kn = rng.standard_normal((b, w["hkv"], w["d"]), dtype=np.float32)
    vn = rng.standard_normal((b, w["hkv"], w["d"]), dtype=np.float32)
    win = (w["windows"] or [0] * w["n_layers"])

    def layer_step(i):
        wl = win[i % len(win)]
        starts = np.array([max(0, int(L) - wl) if wl else 0 for L in lens], np.uint32)
        oracle.decode_step(q, kn, vn, ks[i % n_slabs], vs[i % n_slabs], dt, b, slab, w["hq"], w["hkv"], w["d"],
                           np.asarray(lens, np.uint32), starts, None, w["softcap"])

    layer_step(0)
    t0 = time.perf_counter(); layer_step(1); one = time.perf_counter() - t0
    # keep the whole run within a couple of minutes: ~1 s of CPU work per step
    per_step = max(1, min(w["n_layers"], int(1.0 / max(one, 1e-6))))
    for i in range(args.warmup):
        layer_step(i)
    t0 = time.perf_counter()
    for s in range(args.steps):
        for i in range(per_step):
            layer_step(s * per_step + i)
    dt_s = time.perf_counter() - t0
    us = dt_s * 1e6 / (args.steps * per_step * b)
    sample = (f"{args.steps} steps x {per_step} layer-steps of {b} sequence(s) at the workload's shapes "
              f"({w['dtype']} cache, context {slab}), {cores} OpenMP threads")
    line = {"metric": METRIC, "value": us, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s * 1e3 / args.steps,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_of(args.workload, w),
            "cpu_baseline": {"value": us, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def make_lens(w, rng):
    if "ragged" in w:
        lo, hi = w["ragged"]
        return [int(x) for x in rng.integers(lo, hi + 1, w["batch"])]
    return [w["ctx"]] * w["batch"]


def cpu_baseline_sample(w, budget_s=12.0):
    """Oracle timing on the host cores for the JSON line's cpu_baseline object."""
    import oracle
    cores = oracle.use_all_host_threads()           # before anything is timed
    dt = DT[w["dtype"]]
    rng = np.random.default_rng(99)
    b = min(w["batch"], 4)
    lens = make_lens(w, rng)[:b]
    slab = int(max(lens))
    st = oracle.NP_DTYPE[dt]
    kf = rng.standard_normal((b, slab, w["hkv"], w["d"]), dtype=np.float32)
    k = oracle.store(kf, dt).reshape(kf.shape).astype(st, copy=False)
    v = oracle.store(kf[:, ::-1].copy(), dt).reshape(kf.shape).astype(st, copy=False)
    q = rng.standard_normal((b, w["hq"], w["d"]), dtype=np.float32)
    kn = rng.standard_normal((b, w["hkv"], w["d"]), dtype=np.float32)
    win = (w["windows"] or [0])
    n, t0 = 0, time.perf_counter()
    oracle.decode_step(q, kn, kn, k, v, dt, b, slab, w["hq"], w["hkv"], w["d"], np.asarray(lens, np.uint32))
    t0 = time.perf_counter()
    while True:
        wl = win[n % len(win)]
        starts = np.array([max(0, int(L) - wl) if wl else 0 for L in lens], np.uint32)
        oracle.decode_step(q, kn, kn, k, v, dt, b, slab, w["hq"], w["hkv"], w["d"], np.asarray(lens, np.uint32),
                           starts, None, w["softcap"])
        n += 1
        el = time.perf_counter() - t0
        if el > budget_s or n >= 20000:
            break
    return {"value": el * 1e6 / (n * b), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} layer-steps of {b} sequence(s), {w['dtype']} cache, context {slab}, "
                      f"{cores} OpenMP threads, {el:.1f} s"}


# ----------------------------------------------------------------------------------------------
class Job:
    """Cache + inputs of one rank, resident on its GPU.  `lens` overrides the workload's sequence
    lengths (a rank's share of a ragged batch)."""

    def __init__(self, w, device, seed, ctx=None, lens=None):
        import torch
        import vulkanforge_b200 as vf
        self.vf, self.torch, self.w = vf, torch, w
        torch.cuda.set_device(device)
        self.own_ctx = ctx is None
        self.ctx = ctx if ctx is not None else vf.Context(device)
        rng = np.random.default_rng(seed)
        self.lens = list(lens) if lens is not None else make_lens(w, rng)
        B, L = len(self.lens), w["ctx"]
        self.batch = B
        self.cache = vf.KvCache(self.ctx, vf.KvCacheConfig(w["n_layers"], w["hkv"], w["d"], L, n_slots=B),
                                vf.KvDtype[w["dtype"]])
        sliding = [i for i, x in enumerate(w["windows"] or []) if x]
        window = max(w["windows"]) if w["windows"] else 0
        self.fwd = vf.CudaForward(self.ctx, self.cache, n_heads=w["hq"], max_batch=B, n_splits=w["n_splits"],
                                  softcap=w["softcap"], sliding_window=window, sliding_layers=sliding)
        g = torch.Generator(device="cuda").manual_seed(seed)
        fp8 = w["dtype"] == "F8"
        chunk = 4096
        row = w["hkv"] * w["d"]
        # pre-fill every slab through the product's own prefill append (N(0,1); 1 % x20 outliers for FP8)
        for layer in range(w["n_layers"]):
            for s in range(B):
                n = self.lens[s] - 1
                for p in range(0, n, chunk):
                    m = min(chunk, n - p)
                    kv = torch.randn(2, m, row, device="cuda", generator=g)
                    if fp8:
                        mask = torch.rand(2, m, row, device="cuda", generator=g) < 0.01
                        kv = torch.where(mask, kv * 20.0, kv)
                    self.fwd.b_step_kv_write(layer, kv[0], kv[1], m, p, s)
        nl = w["n_layers"]
        self.q = torch.randn(nl, B, w["hq"], w["d"], device="cuda", generator=g)
        self.k = torch.randn(nl, B, w["hkv"], w["d"], device="cuda", generator=g)
        self.v = torch.randn(nl, B, w["hkv"], w["d"], device="cuda", generator=g)
        self.out = torch.zeros(nl, B, w["hq"], w["d"], device="cuda")
        self.pos = torch.tensor([x - 1 for x in self.lens], dtype=torch.int32, device="cuda")
        self.max_len = max(self.lens)
        # pinned host copies for the end-to-end leg
        self.h_q, self.h_k, self.h_v = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
        self.h_out = torch.zeros_like(self.out, device="cpu").pin_memory()
        self.h_out2 = torch.zeros_like(self.out, device="cpu").pin_memory()
        self.h_pos = np.array([x - 1 for x in self.lens], np.uint32)
        torch.cuda.synchronize()
        self.ctx.poll()
        # the timed work runs on its own stream (CUDA graphs cannot capture the default stream)
        self.stream = torch.cuda.Stream(device=device)
        self.fwd.stream = self.stream.cuda_stream
        self.graph = None
        self.launches_per_step = 0

    def step(self):
        """One token: every layer's append + attention, recorded by one library call."""
        self.fwd.decode_token(self.q, self.k, self.v, self.out, None, self.pos, self.batch, self.max_len)

    def count_launches(self):
        n0 = self.ctx.launch_count()
        with self.torch.cuda.stream(self.stream):
            self.step()
        self.torch.cuda.synchronize()
        self.launches_per_step = self.ctx.launch_count() - n0       # kernels of libvfkv.so per token
        return self.launches_per_step

    def capture(self):
        """Records one step into a CUDA graph, the counterpart of the reference's pre-recorded
        per-token command buffer (forward/decode.rs:169-259); positions stay device-side inputs."""
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            self.step()
        self.graph = g

    def close(self):
        self.torch.cuda.synchronize()
        self.graph = None
        self.fwd.workspace.destroy()
        self.cache.destroy()

    def step_host(self):
        self.fwd.decode_token_host(self.h_q, self.h_k, self.h_v, self.h_out, self.h_pos, self.batch)

    def steps_host_pipelined(self, steps):
        """`steps` tokens through vfkv_decode_token_host_submit / _wait with two in flight; every
        token's inputs come from pinned host memory and its outputs go back to it."""
        pending = []
        for i in range(steps):
            if len(pending) == 2:
                self.fwd.decode_token_host_wait(pending.pop(0))
            pending.append(self.fwd.decode_token_host_submit(self.h_q, self.h_k, self.h_v,
                                                             self.h_out if i % 2 == 0 else self.h_out2, self.h_pos,
                                                             self.batch))
        for t in pending:
            self.fwd.decode_token_host_wait(t)

    def h2d_bytes(self):
        return self.h_q.numel() * 4 + self.h_k.numel() * 4 + self.h_v.numel() * 4 + self.h_pos.nbytes

    def d2h_bytes(self):
        return self.h_out.numel() * 4

    def profile(self, steps):
        """Mean launch time of each kernel family over `steps` more steps (events around every launch)."""
        import ctypes as C
        L = self.ctx._lib
        L.vfkv_profile_enable(self.ctx.handle, 1)
        with self.torch.cuda.stream(self.stream):
            for _ in range(steps):
                self.step()
        self.torch.cuda.synchronize()
        res = {}
        for label, name in ((0, "kv_store"), (2, "fa_split"), (3, "fa_reduce")):
            n, tot, mn = C.c_uint64(), C.c_double(), C.c_double()
            L.vfkv_profile_collect(self.ctx.handle, label, C.byref(n), C.byref(tot), C.byref(mn), 0)
            if n.value:
                res[name] = {"launches": n.value, "mean_us": tot.value * 1e3 / n.value, "min_us": mn.value * 1e3}
        L.vfkv_profile_enable(self.ctx.handle, 0)
        return res


def timed_blocks(fn, stream, steps, warmup, dist=None, min_total_ms=500.0, max_blocks=400):
    """`warmup` untimed calls, then blocks of exactly `steps` calls each, every block bracketed by
    a barrier + synchronize on both sides and timed with CUDA events on `stream`; blocks repeat until
    the timed regions add up to `min_total_ms` (so that clocks can be sampled under load).  With
    several ranks every block's time is the maximum over the ranks.  Returns (median block ms, number
    of blocks, total timed ms)."""
    import torch

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def block():
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
    barrier()
    first = block()
    n_blocks = int(min(max_blocks, max(1, np.ceil(min_total_ms / max(first, 1e-3)))))   # same on every rank
    blocks = [first] + [block() for _ in range(n_blocks - 1)]
    return float(np.median(blocks)), len(blocks), float(np.sum(blocks))


def roofline_of(w, lens, us_per_launch, peak, peak_kind, traffic=None):
    """Roofline object of the attention kernel for launches that take `us_per_launch` on average."""
    per_launch = float(np.mean([algorithmic_bytes(w, lens, l) for l in range(w["n_layers"])]))
    achieved = per_launch / (us_per_launch * 1e-6) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic, "algorithmic_bytes_per_launch": per_launch, "mean_launch_us": us_per_launch,
            "peak_source": f"{peak_kind} copy bandwidth", "frac_of_8000_nominal": achieved / 8000.0}


def measure_workload(name, device, args, ctx=None, lens=None, seed=77, min_total_ms=200.0):
    """One GPU, one workload: a CUDA graph of one token (every layer's fused kernel), device-timed.
    Returns (us per token per layer, us per launch, job's sequence lengths, launches per step)."""
    import gc
    import torch
    w = dict(WORKLOADS[name])
    gc.collect()
    torch.cuda.empty_cache()      # hand the previous workload's blocks back before the cache is allocated
    job = Job(w, device, seed=seed, ctx=ctx, lens=lens)
    try:
        job.ctx.set_dependent_launch(args.pdl)
        with torch.cuda.stream(job.stream):
            for _ in range(2):
                job.step()
        torch.cuda.synchronize()
        launches = job.count_launches()
        job.capture()
        sampler = ClockSampler(physical_gpu_index(device))
        sampler.start()
        ms, _, _ = timed_blocks(job.graph.replay, job.stream, args.steps, 3, None, min_total_ms)
        measure_workload.last_clocks = sampler.finish()
        job.ctx.poll()
        us_step = ms * 1e3 / args.steps
        return us_step / (job.batch * w["n_layers"]), us_step / max(launches, 1), job.lens, launches
    finally:
        job.close()


def other_workloads(ctx, args, peak, peak_kind):
    """The remaining configurations on one GPU, each with the roofline of its attention launches."""
    out = {}
    for name in ("llama3_8b_f16_ctx2048_b1", "batch64_fp8_ctx8192", "batch64_fp8_ragged_512_16384",
                 "gemma_f16_ctx32768_b8", "long_fp8_ctx131072_b1"):
        w = WORKLOADS[name]
        time.sleep(1.0)       # let the board's power average settle: these kernels run at the power cap
        us_tl, us_launch, lens, launches = measure_workload(name, ctx.device, args, ctx=ctx)
        fused = launches == w["n_layers"]
        out[name] = {"us_per_token_layer": us_tl, "launches_per_step": launches,
                     "clocks": measure_workload.last_clocks,
                     "roofline": roofline_of(w, lens, us_launch, peak, peak_kind, NCU_TRAFFIC_BYTES.get(name))
                     if fused else None}
    return out


def next_rows(ctx, args, peak, tensor_peak):
    """The callers either side of the hot path, measured on their own: chunked-prefill causal
    attention over the cache (a 2048-token chunk ending at position 16384, FP8, 32 q / 8 kv / 128:
    tensor-bound, takes the tcgen05 kernel) and RoPE fused with the append of a 512-token chunk."""
    import torch
    import vulkanforge_b200 as vf
    hq, hkv, d, m, q_start = 32, 8, 128, 2048, 14336
    L = q_start + m
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        g = torch.Generator(device="cuda").manual_seed(5)
        for p in range(0, L, 4096):
            kv = torch.randn(2, 4096, hkv * d, device="cuda", generator=g)
            fwd.b_step_kv_write(0, kv[0], kv[1], 4096, p, 0)
        q = torch.randn(m, hq, d, device="cuda", generator=g)
        out = torch.zeros(m, hq, d, device="cuda")
        kv = torch.randn(2, 512, hkv * d, device="cuda", generator=g)

        def timed(fn, reps):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / reps

        time.sleep(1.0)       # let the board's power average settle after the decode workloads
        us_attn = timed(lambda: fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0), 30)
        us_rope = timed(lambda: fwd.rope_kv_write(0, kv[0], kv[1], 512, q_start, freq_base=500000.0), 20)
        # the same launches replayed from a CUDA graph: device time without the host's call overhead
        side = torch.cuda.Stream()
        fwd.stream = side.cuda_stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fwd.rope_kv_write(0, kv[0], kv[1], 512, q_start, freq_base=500000.0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(20):
                fwd.rope_kv_write(0, kv[0], kv[1], 512, q_start, freq_base=500000.0)
        fwd.stream = None
        us_rope_graph = timed(graph.replay, 5) / 20
        flops = 4.0 * hq * d * (m * q_start + m * (m + 1) // 2)              # causal: query i sees q_start + i + 1 rows
        # a short chunk late in a long context: 32 (kv-head, row block) items, which one CTA per item
        # would run on 32 SMs (with the shares switched off the tcgen05 kernel runs one CTA per item)
        few = prefill_extra(ctx, tensor_peak, timed, "F8", 256, 60000, (4, 3, "us_without_even_shares"))
        # F16 rows: K/V tiles by TMA in the specialised form, against the pipelined form
        f16 = prefill_extra(ctx, tensor_peak, timed, "F16", 2048, 14336, (4, 2, "us_pipelined_form"))
        rope_bytes = 2 * 512 * hkv * d * (4 + 1)                             # f32 in, one byte out, K and V
        tf = flops / (us_attn * 1e-6) / 1e12
        gbs = rope_bytes / (us_rope_graph * 1e-6) / 1e9                      # device time: the graph replay
        return {"prefill_attention": {"workload": "2048 queries at positions 14336..16383, FP8 cache, 32/8/128",
                                      "us": us_attn, "bound": "tensor", "achieved": tf, "unit": "TFLOP/s",
                                      "peak": tensor_peak, "frac": tf / tensor_peak if tensor_peak else None,
                                      "note": "tcgen05.mma kernel (roles on separate warps, one CTA per SM with an even "
                                              "share of all K/V tiles), S, P and O in tensor memory"},
                "prefill_attention_few_items": few,
                "prefill_attention_f16": f16,
                "rope_append": {"workload": "512 tokens x 8 kv-heads x 128, FP8 cache, K rotated", "us": us_rope,
                                "us_in_graph": us_rope_graph,
                                "bound": "hbm", "achieved": gbs, "unit": "GB/s", "peak": peak, "frac": gbs / peak,
                                "note": "5 MiB per launch: launch latency, not bandwidth, sets the time; "
                                        "us = one library call per launch from Python, us_in_graph = graph replay"}}
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def prefill_extra(ctx, tensor_peak, timed, dtype, m, q_start, compare):
    """One more prefill-attention case, 32 q / 8 kv / 128: `compare` = (warps, stages, key) times the
    same call with that tuning beside the automatic choice."""
    import torch
    import vulkanforge_b200 as vf
    hq, hkv, d = 32, 8, 128
    L = q_start + m
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        g = torch.Generator(device="cuda").manual_seed(6)
        for p in range(0, L, 4096):
            n = min(4096, L - p)
            kv = torch.randn(2, n, hkv * d, device="cuda", generator=g)
            fwd.b_step_kv_write(0, kv[0], kv[1], n, p, 0)
        q = torch.randn(m, hq, d, device="cuda", generator=g)
        out = torch.zeros(m, hq, d, device="cuda")
        us = timed(lambda: fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0), 20)
        ctx.set_attn_tuning(compare[0], compare[1])
        us_other = timed(lambda: fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0), 5)
        ctx.set_attn_tuning(0, 0)
        tf = 4.0 * hq * d * (m * q_start + m * (m + 1) // 2) / (us * 1e-6) / 1e12
        return {"workload": f"{m} queries at positions {q_start}..{L - 1}, {dtype} cache, 32/8/128", "us": us,
                compare[2]: us_other, "bound": "tensor", "achieved": tf, "unit": "TFLOP/s",
                "peak": tensor_peak, "frac": tf / tensor_peak if tensor_peak else None}
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def run_probe(args):
    """One kernel on its own, for profiling (the commands of profiles/*.md).  `--probe prefill`: the
    chunked-prefill attention (`--probe-dtype` cache, 32 q / 8 kv / 128, `--probe-m` queries ending
    at position `--probe-ctx`); `rope`: RoPE fused with the append of a 512-token chunk; `append`: the plain
    append of a 512-token chunk; `fp8_to_f16`: the cache read of `--probe-ctx` positions of one layer;
    `generic`: the CUDA-core split kernel + merge kernel on an F32 cache of `--probe-ctx` positions;
    `decode`: `--workload`'s fused decode kernel, one layer-step per launch over all its layers;
    `exchange`: the one-launch form of the position-sharded step (attention + fan-out + merge of the
    ranks' blocks) in a group of one rank, 64 q / 8 kv / 128, FP8, `--probe-ctx` positions."""
    import torch
    import vulkanforge_b200 as vf
    ctx = vf.Context(0)
    hq, hkv, d, m, L = 32, 8, 128, args.probe_m, args.probe_ctx
    if args.probe == "decode":
        w = dict(WORKLOADS[args.workload])
        if args.probe_batch:
            w["batch"] = args.probe_batch
        job = Job(w, 0, seed=77, ctx=ctx)
        ctx.set_dependent_launch(args.pdl)
        fn, work, unit = job.step, sum(algorithmic_bytes(w, job.lens, l) for l in range(w["n_layers"])) / 1e9, "GB/s"
        stream = job.stream
    else:
        stream = torch.cuda.current_stream()
        q_start = L - m
        dtype = vf.KvDtype.F32 if args.probe == "generic" else vf.KvDtype[args.probe_dtype]
        cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), dtype)
        fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=16 if args.probe == "generic" else 0)
        g = torch.Generator(device="cuda").manual_seed(5)
        for p in range(0, L, 4096):
            n = min(4096, L - p)
            kv = torch.randn(2, n, hkv * d, device="cuda", generator=g)
            fwd.b_step_kv_write(0, kv[0], kv[1], n, p, 0)
        q = torch.randn(m, hq, d, device="cuda", generator=g)
        out = torch.zeros(m, hq, d, device="cuda")
        kv = torch.randn(2, 512, hkv * d, device="cuda", generator=g)
        if args.probe == "prefill":
            fn = lambda: fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0)
            work, unit = 4.0 * hq * d * (m * q_start + m * (m + 1) // 2) / 1e12, "TFLOP/s"
        elif args.probe == "rope":
            fn = lambda: fwd.rope_kv_write(0, kv[0], kv[1], 512, q_start, freq_base=500000.0)
            work, unit = 2 * 512 * hkv * d * 5 / 1e9, "GB/s"
        elif args.probe == "append":
            fn = lambda: fwd.b_step_kv_write(0, kv[0], kv[1], 512, q_start, 0)
            work, unit = 2 * 512 * hkv * d * 5 / 1e9, "GB/s"
        elif args.probe == "fp8_to_f16":
            k16 = torch.empty(L, hkv, d, dtype=torch.float16, device="cuda")
            v16 = torch.empty_like(k16)
            fn = lambda: ctx.check(ctx._lib.vfkv_fp8_to_f16(cache.handle, 0, 0, L, k16.data_ptr(), v16.data_ptr(), None))
            work, unit = 2 * L * hkv * d * 3 / 1e9, "GB/s"
        elif args.probe == "exchange":
            fwd.workspace.destroy()
            fwd = vf.CudaForward(ctx, cache, n_heads=64)
            ex = vf.PeerExchange(ctx, 1, 0, 64, d)
            q64 = torch.randn(64, d, device="cuda", generator=g)
            out64 = torch.zeros(64, d, device="cuda")
            fn = lambda: fwd.attend_exchange(ex, 0, q64, 0, L, out64)
            work, unit = 2 * L * hkv * d / 1e9, "GB/s"
        else:                                      # generic: CUDA-core split kernel + merge kernel, F32 cache
            fn = lambda: fwd.run_flash_attn_split_reduce(q[0], out[0], 0, L - 1, 16, 0, 0)
            work, unit = 2 * L * hkv * d * 4 / 1e9, "GB/s"
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
    torch.cuda.synchronize()
    ctx.poll()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"probe": args.probe, "workload": args.workload if args.probe == "decode" else None, "m": m,
                      "context": L, "us_per_call": us, "achieved": work / (us * 1e-6), "unit": unit,
                      "steps": args.steps}), flush=True)


# ----------------------------------------------------------------------------------------------
def page_rows(page, hkv, d, seed=4000):
    """K and V rows of one 256-position page of the long-context workload: the same on whichever
    rank generates them (N(0,1), 1 % of the elements x20)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed + page)
    kv = torch.randn(2, 256, hkv * d, device="cuda", generator=g)
    mask = torch.rand(2, 256, hkv * d, device="cuda", generator=g) < 0.01
    return torch.where(mask, kv * 20.0, kv)


def sharded_section(ctx, args, rank, world, local_rank, dist):
    """The two sharded configurations at `world` GPUs, each with its one-GPU time from the same run.

    long_fp8_ctx131072_b1: positions dealt round-robin in 256-row pages; per layer ONE launch per
    rank (owner's append + attention + split merge + peer stores of the partial into every rank's
    buffer + merge of all ranks' partials); the step is replayed from a CUDA graph.  Before timing,
    rank 0 checks layer 0's output against a single-GPU decode step over the unsharded rows.
    long_fp8_ctx131072_b1_by_kv_head_group: the same sequence with every position on every rank but
    only the rank's kv-heads (vfkv_shard_kv_heads) and their q-heads; nothing to exchange.
    batch64_fp8_ragged_512_16384: sequences dealt out by `assign_sequences`; no exchange at all."""
    import torch
    import vulkanforge_b200 as vf
    from vulkanforge_b200.shard import PositionShards, ShardedSequenceDecoder, assign_sequences
    res = {}
    peak, peak_kind = peaks()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- long context, sharded by position -------------------------------------------------
    name = "long_fp8_ctx131072_b1"
    w = WORKLOADS[name]
    L, hq, hkv, d, n_layers = w["ctx"], w["hq"], w["hkv"], w["d"], w["n_layers"]
    one_gpu_us = None
    if rank == 0:                                  # the same workload on one GPU, same run
        one_gpu_us, _, _, _ = measure_workload(name, local_rank, args, ctx=ctx)
    barrier()
    sh = PositionShards(world, 256)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, hkv, d, sh.local_capacity(L)), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=w["n_splits"])
    exchange = vf.PeerExchange(ctx, world, rank, hq, d)
    if dist is not None:
        exchange.connect()
    dec = ShardedSequenceDecoder(fwd, sh, rank, exchange=exchange)
    ctx.set_dependent_launch(args.pdl)
    n_pages = (L + 255) // 256
    for page in range(rank, n_pages, world):       # this rank's pages of the earlier tokens
        kv = page_rows(page, hkv, d)
        m = min(256, L - 1 - page * 256)
        if m <= 0:
            continue
        for layer in range(n_layers):
            fwd.b_step_kv_write(layer, kv[0, :m], kv[1, :m], m, sh.local_pos(page * 256), 0)
    g = torch.Generator(device="cuda").manual_seed(99)          # same inputs on every rank
    q = torch.randn(n_layers, hq, d, device="cuda", generator=g)
    kn = torch.randn(n_layers, 2, 1, hkv * d, device="cuda", generator=g)
    out = torch.zeros(n_layers, hq, d, device="cuda")
    stream = torch.cuda.Stream()
    fwd.stream = stream.cuda_stream

    def step():
        for layer in range(n_layers):
            dec.decode(layer, q[layer], kn[layer, 0], kn[layer, 1], out[layer], L - 1)

    with torch.cuda.stream(stream):
        step()
    barrier()
    n0 = ctx.launch_count()
    with torch.cuda.stream(stream):
        step()
    barrier()
    launches = ctx.launch_count() - n0
    ctx.poll()
    check = None
    ref = None
    if rank == 0:                                  # layer 0 against one GPU holding every row
        rc = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
        rf = vf.CudaForward(ctx, rc, n_heads=hq, n_splits=w["n_splits"])
        for page in range(n_pages):
            kv = page_rows(page, hkv, d)
            m = min(256, L - 1 - page * 256)
            if m > 0:
                rf.b_step_kv_write(0, kv[0, :m], kv[1, :m], m, page * 256, 0)
        ref = torch.zeros(hq, d, device="cuda")
        pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
        rf.decode_step(0, q[0], kn[0, 0], kn[0, 1], ref, None, pos, 1, L)
        torch.cuda.synchronize()
        check = float((out[0] - ref).abs().max() / ref.abs().max())
        rf.workspace.destroy()
        rc.destroy()
        if not check <= 1e-3:
            raise RuntimeError(f"position-sharded output differs from one GPU: relative error {check}")
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    ms, blocks, _ = timed_blocks(graph.replay, stream, args.steps, 3, dist, 200.0)
    ctx.poll()
    us = ms * 1e3 / args.steps / n_layers
    res[name] = {"us_per_token_layer": us, "one_gpu_us_per_token_layer": one_gpu_us, "n_gpus": world,
                 "launches_per_layer_per_rank": launches / n_layers,
                 "check_rel_err_vs_one_gpu": check,
                 "exchange": "peer stores from the attention kernel, merged in the same launch",
                 "exchanged_bytes_per_rank_per_layer": (d + 2) * hq * 8 * world}
    if one_gpu_us is not None:
        res[name]["speedup"] = one_gpu_us / us
        res[name]["efficiency"] = one_gpu_us / us / world
        res[name]["roofline_frac_per_gpu"] = (algorithmic_bytes(w, [L], 0) / world) / (us * 1e-6) / 1e9 / peak
    fwd.stream = None
    barrier()
    exchange.destroy()
    fwd.workspace.destroy()
    cache.destroy()

    # ---- the same long context, sharded by kv-head group ---------------------------------------
    # Rank r holds kv-heads [first, first + count) of every position and the q-heads that read them:
    # outputs are disjoint head ranges, there is nothing to exchange.  The split count is the
    # library's own choice for a few kv-heads with the GPU to themselves.
    import ctypes as C
    first, count = C.c_uint32(), C.c_uint32()
    ctx.check(ctx._lib.vfkv_shard_kv_heads(world, rank, hkv, C.byref(first), C.byref(count)))
    h0, nh, grp = first.value, count.value, hq // hkv
    if world <= hkv:                               # every rank has at least one kv-head
        cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, nh, d, L), vf.KvDtype.F8)
        fwd = vf.CudaForward(ctx, cache, n_heads=nh * grp, n_splits=0, max_splits=255)
        for page in range(n_pages):
            kv = page_rows(page, hkv, d)
            m = min(256, L - 1 - page * 256)
            if m <= 0:
                continue
            kv = kv.view(2, 256, hkv, d)[:, :m, h0:h0 + nh].contiguous()
            for layer in range(n_layers):
                fwd.b_step_kv_write(layer, kv[0], kv[1], m, page * 256, 0)
        qh = q.view(n_layers, hkv, grp, d)[:, h0:h0 + nh].reshape(n_layers, 1, nh * grp, d).contiguous()
        kh = kn.view(n_layers, 2, hkv, d)[:, :, h0:h0 + nh].contiguous()
        k_new = kh[:, 0].reshape(n_layers, 1, nh, d).contiguous()
        v_new = kh[:, 1].reshape(n_layers, 1, nh, d).contiguous()
        outh = torch.zeros(n_layers, 1, nh * grp, d, device="cuda")
        pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
        fwd.stream = stream.cuda_stream

        def step_heads():
            fwd.decode_token(qh, k_new, v_new, outh, None, pos, 1, L)

        with torch.cuda.stream(stream):
            step_heads()
        barrier()
        ctx.poll()
        check_heads = None
        if rank == 0 and ref is not None:
            mine = ref.view(hkv, grp, d)[h0:h0 + nh].reshape(nh * grp, d)
            check_heads = float((outh[0, 0] - mine).abs().max() / ref.abs().max())
            if not check_heads <= 1e-3:
                raise RuntimeError(f"kv-head-sharded output differs from one GPU: relative error {check_heads}")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step_heads()
        ms, _, _ = timed_blocks(graph.replay, stream, args.steps, 3, dist, 200.0)
        ctx.poll()
        us = ms * 1e3 / args.steps / n_layers
        key = name + "_by_kv_head_group"
        res[key] = {"us_per_token_layer": us, "one_gpu_us_per_token_layer": one_gpu_us, "n_gpus": world,
                    "kv_heads_per_rank": nh, "launches_per_layer_per_rank": 1.0,
                    "check_rel_err_vs_one_gpu": check_heads, "exchange": "none (disjoint q-head ranges)"}
        if one_gpu_us is not None:
            res[key]["speedup"] = one_gpu_us / us
            res[key]["efficiency"] = one_gpu_us / us / world
            res[key]["roofline_frac_per_gpu"] = (algorithmic_bytes(w, [L], 0) / world) / (us * 1e-6) / 1e9 / peak
        fwd.stream = None
        barrier()
        fwd.workspace.destroy()
        cache.destroy()

    # ---- ragged batch of 64, sharded by sequence ----------------------------------------------
    name = "batch64_fp8_ragged_512_16384"
    w = WORKLOADS[name]
    lens = make_lens(w, np.random.default_rng(1077))          # the same draw on every rank
    one_gpu_us = None
    if rank == 0:
        one_gpu_us, _, _, _ = measure_workload(name, local_rank, args, ctx=ctx, lens=lens)
    barrier()
    mine = assign_sequences(lens, world)[rank]
    job = Job(dict(w), local_rank, seed=2000 + rank, ctx=ctx, lens=[lens[i] for i in mine])
    ctx.set_dependent_launch(args.pdl)
    with torch.cuda.stream(job.stream):
        job.step()
    torch.cuda.synchronize()
    job.capture()
    ms, _, _ = timed_blocks(job.graph.replay, job.stream, args.steps, 3, dist, 200.0)
    ctx.poll()
    us = ms * 1e3 / args.steps / (len(lens) * w["n_layers"])
    res[name] = {"us_per_token_layer": us, "one_gpu_us_per_token_layer": one_gpu_us, "n_gpus": world,
                 "sequences_per_rank": [len(x) for x in assign_sequences(lens, world)],
                 "positions_per_rank": [int(sum(lens[i] for i in x)) for x in assign_sequences(lens, world)],
                 "exchange": "none"}
    if one_gpu_us is not None:
        res[name]["speedup"] = one_gpu_us / us
        res[name]["efficiency"] = one_gpu_us / us / world
    job.close()
    barrier()
    return res


def run_ours(args, w, rank, world, local_rank):
    import torch
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=300))
    job = Job(w, local_rank, seed=1000 + rank)
    job.ctx.set_dependent_launch(args.pdl)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(job.stream):
        for _ in range(args.warmup):
            job.step()
    barrier()
    job.count_launches()
    if not args.no_graph:
        job.capture()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    run = job.graph.replay if job.graph is not None else job.step
    ms, blocks, total_ms = timed_blocks(run, job.stream, args.steps, args.warmup, dist)
    clocks = sampler.finish()
    launches = job.launches_per_step * args.steps * blocks
    ms_stream = ms
    if job.graph is not None:                                  # same steps, one launch call per kernel
        ms_stream, _, _ = timed_blocks(job.step, job.stream, args.steps, 3, dist, 100.0)
    job.ctx.poll()

    # end-to-end leg: host buffers in, host buffers out, every step
    for _ in range(max(3, args.warmup)):
        job.step_host()
    e2e_blocks = []
    for _ in range(max(3, min(blocks, 50))):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            job.step_host()
        barrier()
        e2e_blocks.append((time.perf_counter() - t0) * 1e3)
    e2e_sync_ms = float(np.median(e2e_blocks))
    # the same with two tokens in flight (submit / wait): the copies of one token run beside the
    # layers of the other, as the reference's two command-buffer / fence pairs allow
    job.steps_host_pipelined(max(3, args.warmup))
    e2e_blocks = []
    for _ in range(max(3, min(blocks, 50))):
        barrier()
        t0 = time.perf_counter()
        job.steps_host_pipelined(args.steps)
        barrier()
        e2e_blocks.append((time.perf_counter() - t0) * 1e3)
    e2e_ms = float(np.median(e2e_blocks))

    if dist is not None:
        t = torch.tensor([e2e_ms, e2e_sync_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, e2e_sync_ms = float(t[0]), float(t[1])
        tot = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(tot)
        launches = int(tot[0])

    line = None
    if rank == 0:
        tokens = w["batch"] * world                       # tokens decoded per step, all ranks
        denom = args.steps * tokens * w["n_layers"]
        value = ms * 1e3 / denom
        prof = job.profile(min(args.steps, 20))
        peak, peak_kind = peaks()
        split = prof.get("fa_split")
        roofline = None
        if split:
            # The timed region launches one kernel per layer-step and nothing else (append and merge
            # are fused into it), so its mean launch duration inside the region is region time /
            # launches; consecutive launches overlap under dependent launch, which per-launch event
            # pairs (kept in "kernels", measured in a separate pass) cannot show.
            fused = job.launches_per_step == w["n_layers"]
            mean_us = ms * 1e3 / (args.steps * w["n_layers"]) if fused else split["mean_us"]
            roofline = roofline_of(w, job.lens, mean_us, peak, peak_kind, NCU_TRAFFIC_BYTES.get(args.workload))
            roofline["kernel"] = "attn_split_mma_kernel (fa_split: append + attention + merge)" if fused else "fa_split"
            roofline["mean_launch_us_isolated_events"] = split["mean_us"]
        step_bytes = sum(algorithmic_bytes(w, job.lens, l) for l in range(w["n_layers"]))
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32 (fp8/f16 storage)", "data": "synthetic",
                "config": config_of(args.workload, w),
                "run": {"l2": "each step streams the whole cache (larger than the 126 MB L2) before a layer repeats"
                              if step_bytes > 200e6 else "working set below L2: hot-L2 numbers",
                        "launch": "one CUDA graph replay per token" if job.graph is not None else "stream launches",
                        "dependent_launch_mode": args.pdl,
                        "parallelism": f"sequence-sharded x{world}, no collective",
                        "timed_blocks": blocks, "timed_region_ms": total_ms,
                        "value_is": "median over the blocks of (block time / steps); each block is exactly "
                                    "--steps steps between barrier + synchronize, max over ranks"},
                "value_stream_launches": ms_stream * 1e3 / denom,
                "tokens_per_s": tokens * args.steps / (ms * 1e-3),
                "achieved_gbs_whole_step": step_bytes * world * args.steps / (ms * 1e-3) / 1e9,
                "roofline": roofline, "kernels": prof, "clocks": clocks, "gpu_launches": launches,
                "e2e": {"value": e2e_ms * 1e3 / denom, "unit": UNIT, "h2d_bytes_per_step": job.h2d_bytes(),
                        "d2h_bytes_per_step": job.d2h_bytes(),
                        "call": "vfkv_decode_token_host_submit / _wait, two tokens in flight, pinned host buffers",
                        "value_one_token_at_a_time": e2e_sync_ms * 1e3 / denom,
                        "call_one_token_at_a_time": "vfkv_decode_token_host"}}
        if world == 1 and not args.no_extra and args.workload == DEFAULT_WORKLOAD:
            line["copy_gbs_this_gpu"] = copy_bandwidth_here()
            others = other_workloads(job.ctx, args, peak, peak_kind)
            line["roofline_batch64_ctx8192"] = dict(others["batch64_fp8_ctx8192"]["roofline"],
                                                    workload="batch64_fp8_ctx8192: 64 sequences x 8192 tokens, "
                                                             "32 q / 8 kv / 128, FP8, 2 layers")
            line["other_workloads"] = others
            line["next_rows"] = next_rows(job.ctx, args, peak, tensor_peak())
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_sample(w)
    ctx = job.ctx
    job.close()
    if args.workload == DEFAULT_WORKLOAD and not args.no_extra:
        sharded = sharded_section(ctx, args, rank, world, local_rank, dist)
        if line is not None:
            line["sharded"] = sharded                      # last key of the line
    if line is not None:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline sample")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the other workloads, the next rows and the sharded configurations")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a CUDA graph replay")
    ap.add_argument("--pdl", type=int, default=2, choices=[0, 1, 2],
                    help="programmatic dependent launch mode of the attention kernel (vfkv_ctx_set_dependent_launch)")
    ap.add_argument("--probe", default=None, choices=["prefill", "rope", "append", "fp8_to_f16", "generic", "decode", "exchange"],
                    help="run one kernel on its own (for profiling) and exit")
    ap.add_argument("--probe-m", type=int, default=2048)
    ap.add_argument("--probe-ctx", type=int, default=16384)
    ap.add_argument("--probe-dtype", default="F8", choices=["F8", "F16"], help="--probe prefill: cache element type")
    ap.add_argument("--probe-batch", type=int, default=0, help="--probe decode: override the workload's batch")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = dict(WORKLOADS[args.workload])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.probe:
        run_probe(args)
        return
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
