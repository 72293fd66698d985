#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: KV append + split-K GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one decode token: for every layer, append the token's K/V to the cache, then
attend over the whole context.  The default workload is the FP8 Qwen3-8B-like case
(36 layers, 32 q / 8 kv / 128, batch 1, context 8192, 16 splits).  Prints ONE JSON line.

value     device-timed, inputs resident in HBM, microseconds per token per layer
e2e       the same through vfkv_decode_token_host with pinned HOST buffers (copies inside the
          timed region)
roofline  the attention split kernel: algorithmic KV bytes per launch / its mean launch time,
          against the measured HBM copy bandwidth
cpu_baseline  the CPU oracle (a C port of the reference's CPU attention and store code, the
          reference itself is Rust and cannot be built here) on a bounded sample

Under torchrun every rank runs the same workload on its own sequence(s) and GPU (sharding by
sequence, no collective on the data path); times are the max over ranks.
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
    "batch64_fp8_ctx8192": dict(n_layers=1, hq=32, hkv=8, d=128, dtype="F8", batch=64, ctx=8192,
                                n_splits=0, softcap=0.0, windows=None),
    "batch64_fp8_ragged_512_16384": dict(n_layers=1, hq=32, hkv=8, d=128, dtype="F8", batch=64, ctx=16384,
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
# captures summarised under profiles/ (attn_split_mma_fp8_*.md)
NCU_TRAFFIC_BYTES = {"qwen3_8b_fp8_ctx8192_b1": 16_843_000, "batch64_fp8_ctx8192": 1_081_500_000}


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
            "data": "synthetic", "config": {"workload": args.workload, **{k: v for k, v in w.items() if k != "windows"}},
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
    """Cache + inputs of one rank, resident on its GPU."""

    def __init__(self, w, device, seed, ctx=None):
        import torch
        import vulkanforge_b200 as vf
        self.vf, self.torch, self.w = vf, torch, w
        torch.cuda.set_device(device)
        self.ctx = ctx if ctx is not None else vf.Context(device)
        rng = np.random.default_rng(seed)
        self.lens = make_lens(w, rng)
        B, L = w["batch"], w["ctx"]
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
        self.fwd.decode_token(self.q, self.k, self.v, self.out, None, self.pos, self.w["batch"], self.max_len)

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
        self.fwd.workspace.destroy()
        self.cache.destroy()

    def step_host(self):
        self.fwd.decode_token_host(self.h_q, self.h_k, self.h_v, self.h_out, self.h_pos, self.w["batch"])

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


def batch64_roofline(ctx, args, peak):
    """The same kernel where it is bandwidth-bound: 64 sequences x 8192 tokens, FP8, one layer
    (1 GiB of K/V per launch, far beyond L2).  Device events around `steps` launches."""
    import torch
    w = WORKLOADS["batch64_fp8_ctx8192"]
    job = None
    try:
        job = Job(w, ctx.device, seed=77, ctx=ctx)
        with torch.cuda.stream(job.stream):
            for _ in range(3):
                job.step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                job.step()
            e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        nbytes = algorithmic_bytes(w, job.lens, 0)
        achieved = nbytes / (us * 1e-6) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES["batch64_fp8_ctx8192"], "algorithmic_bytes_per_launch": nbytes,
                "mean_launch_us": us, "frac_of_8000_nominal": achieved / 8000.0,
                "workload": "batch64_fp8_ctx8192: 64 sequences x 8192 tokens, 32 q / 8 kv / 128, FP8, 1 layer"}
    finally:
        if job is not None:
            job.close()


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

        us_attn = timed(lambda: fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0), 10)
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
        rope_bytes = 2 * 512 * hkv * d * (4 + 1)                             # f32 in, one byte out, K and V
        tf = flops / (us_attn * 1e-6) / 1e12
        gbs = rope_bytes / (us_rope_graph * 1e-6) / 1e9                      # device time: the graph replay
        return {"prefill_attention": {"workload": "2048 queries at positions 14336..16383, FP8 cache, 32/8/128",
                                      "us": us_attn, "bound": "tensor", "achieved": tf, "unit": "TFLOP/s",
                                      "peak": tensor_peak, "frac": tf / tensor_peak if tensor_peak else None,
                                      "note": "tcgen05.mma kernel, S and O in tensor memory"},
                "rope_append": {"workload": "512 tokens x 8 kv-heads x 128, FP8 cache, K rotated", "us": us_rope,
                                "us_in_graph": us_rope_graph,
                                "bound": "hbm", "achieved": gbs, "unit": "GB/s", "peak": peak, "frac": gbs / peak,
                                "note": "5 MiB per launch: launch latency, not bandwidth, sets the time; "
                                        "us = one library call per launch from Python, us_in_graph = graph replay"}}
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def run_probe(args):
    """One kernel of the "next" rows on its own, for profiling: `--probe prefill` launches the
    chunked-prefill attention `--steps` times (FP8, 32 q / 8 kv / 128, `--probe-m` queries ending
    at position `--probe-ctx`); `--probe rope` the fused RoPE + append of a 512-token chunk."""
    import torch
    import vulkanforge_b200 as vf
    ctx = vf.Context(0)
    hq, hkv, d, m, L = 32, 8, 128, args.probe_m, args.probe_ctx
    q_start = L - m
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
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
    else:
        fn = lambda: fwd.rope_kv_write(0, kv[0], kv[1], 512, q_start, freq_base=500000.0)
        work, unit = 2 * 512 * hkv * d * 5 / 1e9, "GB/s"
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
    print(json.dumps({"probe": args.probe, "m": m, "context": L, "us_per_launch": us, "achieved": work / (us * 1e-6),
                      "unit": unit, "steps": args.steps}), flush=True)
    fwd.workspace.destroy()
    cache.destroy()
    ctx.destroy()


def run_ours(args, w, rank, world, local_rank):
    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    job = Job(w, local_rank, seed=1000 + rank)
    job.ctx.check(job.ctx._lib.vfkv_ctx_set_dependent_launch(job.ctx.handle, args.pdl))
    job.ctx.set_cluster_merge(bool(args.cluster))
    if args.tune:
        wt, st = (int(x) for x in args.tune.split("x"))
        job.ctx.check(job.ctx._lib.vfkv_ctx_set_attn_tuning(job.ctx.handle, wt, st))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        """W warm-up steps, then K steps between two events on the job's stream."""
        with torch.cuda.stream(job.stream):
            for _ in range(args.warmup):
                fn()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            barrier()
        return e0.elapsed_time(e1)

    with torch.cuda.stream(job.stream):
        for _ in range(args.warmup):
            job.step()
    barrier()
    n0 = job.ctx.launch_count()
    with torch.cuda.stream(job.stream):
        job.step()
    barrier()
    job.launches_per_step = job.ctx.launch_count() - n0       # kernels of libvfkv.so per token
    if not args.no_graph:
        job.capture()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms = timed(job.graph.replay if job.graph is not None else job.step)
    launches = job.launches_per_step * args.steps
    clocks = sampler.finish()
    ms_stream = timed(job.step) if job.graph is not None else ms      # same steps, one launch call per kernel
    job.ctx.poll()

    # end-to-end leg: host buffers in, host buffers out, every step
    for _ in range(max(3, args.warmup)):
        job.step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        job.step_host()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
        tot = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(tot)
        launches = int(tot[0])

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
            per_launch = float(np.mean([algorithmic_bytes(w, job.lens, l) for l in range(w["n_layers"])]))
            fused = job.launches_per_step == w["n_layers"]
            mean_us = ms * 1e3 / (args.steps * w["n_layers"]) if fused else split["mean_us"]
            achieved = per_launch / (mean_us * 1e-6) / 1e9
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                        "kernel": "attn_split_mma_kernel (fa_split: append + attention + merge)" if fused else "fa_split",
                        "algorithmic_bytes_per_launch": per_launch, "mean_launch_us": mean_us,
                        "mean_launch_us_isolated_events": split["mean_us"],
                        "peak_source": f"{peak_kind} copy bandwidth", "frac_of_8000_nominal": achieved / 8000.0}
        step_bytes = sum(algorithmic_bytes(w, job.lens, l) for l in range(w["n_layers"]))
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32 (fp8/f16 storage)", "data": "synthetic",
                "config": {"workload": args.workload, "n_layers": w["n_layers"], "n_q_heads": w["hq"],
                           "n_kv_heads": w["hkv"], "head_dim": w["d"], "kv_dtype": w["dtype"], "batch_per_gpu": w["batch"],
                           "context": w["ctx"], "n_splits": w["n_splits"], "softcap": w["softcap"],
                           "l2": "each step streams the whole cache (larger than the 126 MB L2) before a layer repeats"
                                 if step_bytes > 200e6 else "working set below L2: hot-L2 numbers",
                           "launch": "one CUDA graph replay per token" if job.graph is not None else "stream launches",
                           "dependent_launch_mode": args.pdl, "cluster_merge": args.cluster,
                           "parallelism": f"sequence-sharded x{world}, no collective"},
                "value_stream_launches": ms_stream * 1e3 / denom,
                "tokens_per_s": tokens * args.steps / (ms * 1e-3),
                "achieved_gbs_whole_step": step_bytes * world * args.steps / (ms * 1e-3) / 1e9,
                "roofline": roofline, "kernels": prof, "clocks": clocks, "gpu_launches": launches,
                "e2e": {"value": e2e_ms * 1e3 / denom, "unit": UNIT, "h2d_bytes_per_step": job.h2d_bytes(),
                        "d2h_bytes_per_step": job.d2h_bytes()}}
        if world == 1 and not args.no_extra and args.workload == DEFAULT_WORKLOAD:
            line["roofline_batch64_ctx8192"] = batch64_roofline(job.ctx, args, peak)
            line["next_rows"] = next_rows(job.ctx, args, peak, tensor_peak())
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_sample(w)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_position_sharded(args, w, rank, world, local_rank):
    """One long sequence cut into round-robin pages over the ranks (strong scaling): per step the
    owner of the new position appends, every rank attends over its pages, the (m, l, o) partials are
    all-gathered over NCCL and merged on every rank."""
    import torch
    import torch.distributed as dist
    import vulkanforge_b200 as vf
    from vulkanforge_b200.shard import PositionShards, ShardedSequenceDecoder
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local_rank)
    import datetime
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                            timeout=datetime.timedelta(seconds=90))
    ctx = vf.Context(local_rank)
    sh = PositionShards(world, 256)
    L, hq, hkv, d = w["ctx"], w["hq"], w["hkv"], w["d"]
    cache = vf.KvCache(ctx, vf.KvCacheConfig(w["n_layers"], hkv, d, sh.local_capacity(L)), vf.KvDtype[w["dtype"]])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=w["n_splits"])
    exchange = None
    if args.exchange == "peer":                            # partials by peer stores from the attention kernel
        exchange = vf.PeerExchange(ctx, world, rank, hq, d)
        exchange.connect()
    dec = ShardedSequenceDecoder(fwd, sh, rank, exchange=exchange)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    n_local = sh.local_len(L - 1, rank)
    n_layers = w["n_layers"]
    ctx.check(ctx._lib.vfkv_ctx_set_dependent_launch(ctx.handle, args.pdl))
    for p in range(0, n_local, 4096):                      # this rank's pages of the 131071 earlier tokens
        m = min(4096, n_local - p)
        kv = torch.randn(2, m, hkv * d, device="cuda", generator=g)
        mask = torch.rand(2, m, hkv * d, device="cuda", generator=g) < 0.01
        kv = torch.where(mask, kv * 20.0, kv)
        for layer in range(n_layers):
            fwd.b_step_kv_write(layer, kv[0], kv[1], m, p, 0)
    chunk = torch.randn(2, 512, hkv * d, device="cuda", generator=g)   # a 512-token chunked-prefill append
    q = torch.randn(n_layers, hq, d, device="cuda", generator=g)
    kn = torch.randn(n_layers, 2, 1, hkv * d, device="cuda", generator=g)
    out = torch.zeros(n_layers, hq, d, device="cuda")

    def step():
        for layer in range(n_layers):
            dec.decode(layer, q[layer], kn[layer, 0], kn[layer, 1], out[layer], L - 1)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    fwd.stream = stream.cuda_stream
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
    barrier()
    n0 = ctx.launch_count()
    with torch.cuda.stream(stream):
        step()
    barrier()
    launches = (ctx.launch_count() - n0) * args.steps
    run, launch_kind = step, "stream launches"
    if exchange is not None and not args.no_graph:         # only this library's kernels: always capturable
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        run, launch_kind = graph.replay, "one CUDA graph replay per token"
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            run()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.finish()
    fwd.stream = None
    # the chunked-prefill append of the same config, timed on its own
    base = max(0, L - 1 - 512)
    for _ in range(3):
        dec.prefill(0, chunk[0].view(512, hkv, d), chunk[1].view(512, hkv, d), base, 512)
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(args.steps):
        dec.prefill(0, chunk[0].view(512, hkv, d), chunk[1].view(512, hkv, d), base, 512)
    p1.record()
    barrier()
    prefill_ms = p0.elapsed_time(p1) / args.steps
    t = torch.tensor([ms, prefill_ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tot = torch.tensor([launches], device="cuda", dtype=torch.int64)
    dist.all_reduce(tot)
    ctx.poll()
    if rank == 0:
        ms, prefill_ms = float(t[0]), float(t[1])
        step_bytes = algorithmic_bytes(w, [L], 0) * w["n_layers"]
        line = {"metric": METRIC, "value": ms * 1e3 / args.steps / w["n_layers"], "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32 (fp8/f16 storage)", "data": "synthetic",
                "config": {"workload": args.workload, "n_layers": w["n_layers"], "n_q_heads": hq, "n_kv_heads": hkv,
                           "head_dim": d, "kv_dtype": w["dtype"], "context": L,
                           "parallelism": f"positions sharded x{world} in 256-row pages, " + (
                               "(m, l, o) stored into every GPU's buffer by the attention kernel, flag-waiting merge"
                               if exchange is not None else "NCCL all-gather of (m, l, o)"),
                           "exchange": args.exchange,
                           "collective_bytes_per_rank": (d + 2) * hq * 4, "launch": launch_kind,
                           "l2": "per-GPU share of the cache is %d MiB per step" % (step_bytes // world >> 20)},
                "achieved_gbs_whole_step": step_bytes * args.steps / (ms * 1e-3) / 1e9,
                "prefill_chunk_512_us": prefill_ms * 1e3, "clocks": clocks, "gpu_launches": int(tot[0])}
        print(json.dumps(line), flush=True)
    dist.barrier()
    if exchange is not None:
        exchange.destroy()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline sample")
    ap.add_argument("--no-extra", action="store_true", help="skip the batch-64 roofline measurement")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a CUDA graph replay")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="position-sharded mode: how the per-GPU partials travel (peer stores fused into the "
                         "attention kernel, or an NCCL all-gather)")
    ap.add_argument("--n-splits", type=int, default=None, help="override the workload's split count (0 = choose)")
    ap.add_argument("--pdl", type=int, default=2, choices=[0, 1, 2],
                    help="programmatic dependent launch mode of the attention kernel (vfkv_ctx_set_dependent_launch)")
    ap.add_argument("--probe", default=None, choices=["prefill", "rope"],
                    help="run one kernel of the next rows on its own (for profiling) and exit")
    ap.add_argument("--probe-m", type=int, default=2048)
    ap.add_argument("--probe-ctx", type=int, default=16384)
    ap.add_argument("--cluster", type=int, default=0, choices=[0, 1],
                    help="merge the splits inside a thread-block cluster (vfkv_ctx_set_cluster_merge)")
    ap.add_argument("--tune", default=None, help="tensor-core kernel shape WxS (warps x stages), e.g. 4x3")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = dict(WORKLOADS[args.workload])
    if args.n_splits is not None:
        w["n_splits"] = args.n_splits
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.probe:
        run_probe(args)
        return
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if world > 1 and w.get("shard") == "positions":
        run_position_sharded(args, w, rank, world, local_rank)
        return
    run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
