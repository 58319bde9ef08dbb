#!/usr/bin/env python
"""Headline benchmark: Q4_K decode matvec at the Llama-3-8B FFN-up shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* is one pass of the matvec over a ring of RING distinct device copies
of the 14336 x 4096 Q4_K weight (RING x 33 MB > the 126 MB L2, so every launch
streams its weights from HBM).  `value` is weight-GB/s with everything resident
in HBM (CUDA events on the launching stream); `e2e` is the same metric through
the host-pointer C-ABI call a binding of the reference's `QuantKernel::gemv`
makes (pinned host activations in, host outputs back, copies inside the timed
region).

With N > 1 ranks every rank owns a 14336-row shard of an (N*14336) x 4096 matrix
(weak scaling) and every matvec's output reaches all ranks: the matvec kernel
stores each result, tagged, into a slot array of every rank over NVLink, and a
bounded unpacking wait on every rank polls all N*14336 slots of the call; the
gathered vector is compared with an NCCL all-gather of the single-GPU results
before anything is timed (`gather_checked`).

Beside the headline the line carries the other configurations' figures
(`decode_shapes`, `small_batch`, `layer`, `prefill`, `moe`) and, for N > 1, `moe_layer` and
strong-scaling figures of the large shapes (`strong_scaling`).

`--impl reference` times the CPU restatement of the reference's own fastest
tier (oracle/qk_cpu_simd.c: AVX-512 / AVX2 rows under a row-parallel driver) on
the host cores for the same metric.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from oxillama_b200 import synth as S  # noqa: E402

ROWS, COLS, QTYPE = 14336, 4096, S.Q4_K
RING = 16
METRIC = "q4_k_gemv_weight_bandwidth"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, from the
# ncu capture summarised in profiles/q4k_gemv_14336x4096_m1_ncu.md
DRAM_BYTES_PER_LAUNCH = 33113600
WORKLOAD = "config[1]: Q4_K 14336x4096 matvec, M=1, f32 N(0,1) activations, seed 0"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    """Dense 16-bit tensor-core peak (TFLOP/s) for a kernel timed alone: the measured burst figure."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def big_weight(qtype, rows, cols, seed, stream):
    """A seeded weight matrix; matrices above 64 MB repeat a seeded 1/8-row draw eight times
    (same distribution, an eighth of the host time)."""
    if S.weight_nbytes(qtype, rows, cols) <= 64e6 or rows % 8:
        return S.gen_weight(qtype, rows, cols, seed=seed, stream=stream)
    return np.tile(S.gen_weight(qtype, rows // 8, cols, seed=seed, stream=stream), 8)


def graph_us(torch, stream, fn, calls_per_fn, launches=200, warm=3):
    """fn() enqueues `calls_per_fn` kernels' worth of work on the current stream; it is captured
    once into a CUDA graph and replayed.  Returns microseconds per call (CUDA events)."""
    with torch.cuda.stream(stream):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(warm):
            g.replay()
        torch.cuda.synchronize()
        iters = max(1, launches // calls_per_fn)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * calls_per_fn)


def ring_of(qtype, rows, cols, ctx, seed=0, stream0=97, min_bytes=300e6, row_begin=0, row_end=None, host=None):
    """Enough device copies of one weight (or row shard) that a pass over them exceeds L2."""
    from oxillama_b200.device import DeviceWeights
    row_end = rows if row_end is None else row_end
    nbytes = S.weight_nbytes(qtype, row_end - row_begin, cols)
    ring = max(2, min(16, int(min_bytes / max(nbytes, 1)) + 1))
    base = host if host is not None else big_weight(qtype, rows, cols, seed, stream0)
    return [DeviceWeights(qtype, base, rows, cols, row_begin, row_end, ctx=ctx) for _ in range(ring)]


def matvec_rates(torch, ctx, qtype, rows, cols, ms, stream, bound="hbm", launches=128):
    """One weight shape at each batch size of `ms`: microseconds per call over graph-replayed
    launches that rotate through enough weight copies to exceed L2, and the fraction of the
    roofline that bounds it."""
    from oxillama_b200.device import check_device_status
    dws = ring_of(qtype, rows, cols, ctx)
    nbytes = dws[0].algo_bytes
    outs = []
    for m in ms:
        x = torch.from_numpy(S.gen_acts(m, cols, seed=1)).cuda()
        y = torch.empty(m, rows, device="cuda")

        def fn():
            for d in dws:
                d.gemm(x, y, m)
        us = graph_us(torch, stream, fn, len(dws), launches)
        check_device_status(ctx, stream)
        out = {"workload": f"{S.NAMES[qtype]} {rows}x{cols}, M={m}", "us_per_launch": us, "ring_copies": len(dws)}
        if bound == "hbm":
            peak, which = peaks()
            gbs = nbytes / us / 1e3
            out.update({"weight_gbs": gbs, "frac": gbs / peak, "bound": "hbm", "peak_source": which,
                        "floor_us": nbytes / peak / 1e3})
        else:
            peak, which = tensor_peak()
            tf = 2.0 * m * rows * cols / us / 1e6
            out.update({"tflops": tf, "frac": tf / peak, "bound": "tensor", "peak_tflops": peak, "peak_source": which,
                        "operands": "fp16 (weights dequantised in the kernel), f32 accumulation in TMEM"})
        outs.append(out)
    for d in dws:
        d.free()
    return outs


def matvec_rate(torch, ctx, qtype, rows, cols, m, stream, bound="hbm", launches=128):
    return matvec_rates(torch, ctx, qtype, rows, cols, [m], stream, bound, launches)[0]


LAYER = [("q", S.Q4_K, 4096, 4096), ("k", S.Q4_K, 1024, 4096), ("v", S.Q4_K, 1024, 4096),
         ("o", S.Q4_K, 4096, 4096), ("gate", S.Q4_K, 14336, 4096), ("up", S.Q4_K, 14336, 4096),
         ("down", S.Q6_K, 4096, 14336)]


def layer_rates(torch, ctx, ms, stream, copies=3):
    """The seven linears of one Llama-3-8B-shaped decoder layer (Q4_K_M mix), one call each with
    an independent input, `copies` distinct layers in rotation (3 x 138 MB > L2), at each batch
    size of `ms`."""
    from oxillama_b200.device import DeviceWeights, check_device_status
    hosts = [(t, r, c, S.gen_weight(t, r, c, seed=4, stream=i)) for i, (_, t, r, c) in enumerate(LAYER)]
    layers = [[DeviceWeights(t, w, r, c, ctx=ctx) for (t, r, c, w) in hosts] for _ in range(copies)]
    # q, k and v read the same input and share a format: their rows uploaded as one matrix (GGUF data is
    # row-major, so the bytes simply follow one another) make the three projections one launch
    qkv_rows = sum(r for (_, r, _, _) in hosts[:3])
    qkv_host = np.concatenate([np.asarray(w).reshape(-1) for (_, _, _, w) in hosts[:3]])
    qkvs = [DeviceWeights(hosts[0][0], qkv_host, qkv_rows, hosts[0][2], ctx=ctx) for _ in range(copies)]
    nbytes = sum(d.algo_bytes for d in layers[0])
    outs = []
    for m in ms:
        xs = {c: torch.from_numpy(S.gen_acts(m, c, seed=4)).cuda() for c in (4096, 14336)}
        ys = {r: torch.empty(m, r, device="cuda") for r in (4096, 1024, 14336)}

        def fn():
            for lw in layers:
                for d in lw:
                    d.gemm(xs[d.cols], ys[d.rows], m)
        us = graph_us(torch, stream, fn, copies, launches=60)
        check_device_status(ctx, stream)
        flops = sum(2.0 * m * d.rows * d.cols for d in layers[0])
        out = {"workload": f"config[3]: q,k,v,o,gate,up Q4_K + down Q6_K of one layer, M={m}", "us_per_layer": us,
               "weight_bytes": nbytes}
        if m <= 4:
            # the same layer with its feed-forward block as one call (gate and up in one launch,
            # silu(g) * u formed in its reducer, then down)
            from oxillama_b200.device import ffn

            def fn_fused():
                for lw in layers:
                    for d in lw[:4]:
                        d.gemm(xs[d.cols], ys[d.rows], m)
                    ffn(lw[4], lw[5], lw[6], xs[4096], ys[4096], m)
            us = graph_us(torch, stream, fn_fused, copies, launches=60)
            check_device_status(ctx, stream)
            out["us_per_layer_separate_calls"] = out["us_per_layer"]
            out["us_per_layer"] = us
            out["note"] = "feed-forward block through qk_ffn_dev (5 launches per layer instead of 7)"
            yqkv = torch.empty(m, qkv_rows, device="cuda")

            def fn_qkv():
                for lw, f in zip(layers, qkvs):
                    f.gemm(xs[f.cols], yqkv, m)
                    lw[3].gemm(xs[lw[3].cols], ys[lw[3].rows], m)
                    ffn(lw[4], lw[5], lw[6], xs[4096], ys[4096], m)
            us_qkv = graph_us(torch, stream, fn_qkv, copies, launches=60)
            check_device_status(ctx, stream)
            out["us_per_layer_qkv_rows_as_one_matrix"] = us_qkv
            out["note_qkv"] = ("the same layer with the rows of q, k and v uploaded as one 6144 x 4096 matrix at load "
                               "(3 launches per layer, the same arithmetic per row); not in us_per_layer / frac")
        if m <= 64:
            peak, which = peaks()
            out.update({"weight_gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "bound": "hbm",
                        "floor_us": nbytes / peak / 1e3, "peak_source": which})
            if "us_per_layer_qkv_rows_as_one_matrix" in out:
                out["frac_qkv_rows_as_one_matrix"] = nbytes / out["us_per_layer_qkv_rows_as_one_matrix"] / 1e3 / peak
        else:
            peak, which = tensor_peak()
            out.update({"tflops": flops / us / 1e6, "frac": flops / us / 1e6 / peak, "bound": "tensor",
                        "peak_source": which})
        outs.append(out)
    for lw in layers:
        for d in lw:
            d.free()
    for d in qkvs:
        d.free()
    return outs


def moe_rate(torch, ctx, qtype, stream, n_local=8, expert_begin=0):
    """config[4]: Mixtral-8x7B-shaped MoE FFN, 256 tokens routed top-2 over 8 experts.  The experts
    are device copies of three seeded matrices (gate, up, down): same sizes and traffic as eight
    independent draws, a fraction of the host time."""
    from oxillama_b200 import moe
    hidden, inter, n_exp, tokens, top_k = 4096, 14336, 8, 256, 2
    g = S.gen_weight(qtype, inter, hidden, seed=5, stream=0)
    u = S.gen_weight(qtype, inter, hidden, seed=5, stream=1)
    d = S.gen_weight(qtype, hidden, inter, seed=5, stream=2)
    ex = moe.MoeExperts(qtype, [g] * n_local, [u] * n_local, [d] * n_local, hidden, inter, n_exp,
                        expert_begin=expert_begin, ctx=ctx)
    rng = np.random.default_rng(5)
    logits = torch.from_numpy(rng.standard_normal((tokens, n_exp)).astype(np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((tokens, hidden)).astype(np.float32)).cuda()
    y = torch.empty((tokens, hidden), device="cuda")
    with torch.cuda.stream(stream):
        for _ in range(2):
            ex.forward(logits, x, y, top_k)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 5
        e0.record(stream)
        for _ in range(iters):
            ex.forward(logits, x, y, top_k)
        e1.record(stream)
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    ex.free()
    flops = 2.0 * tokens * top_k * 3 * inter * hidden * (n_local / n_exp)  # expected share of the routed slots
    peak, which = tensor_peak()
    return {"workload": f"config[4]: 8 x {S.NAMES[qtype]} experts (gate, up 14336x4096; down 4096x14336), "
                        f"256 tokens, top-2; {n_local} experts on this GPU",
            "ms": ms, "tflops": flops / ms / 1e9, "frac": flops / ms / 1e9 / peak, "peak_source": which}


def moe_layer_rates(torch, dist, ctx, qtype, stream, world, rank):
    """config[4] as a whole layer on `world` GPUs, collectives included, both ways of sharding it:
    tokens replicated and outputs summed by an all-reduce, and tokens sharded with routed rows
    crossing by two all-to-all exchanges.  Device-timed, max over the ranks."""
    from oxillama_b200 import moe
    hidden, inter, n_exp, tokens, top_k = 4096, 14336, 8, 256, 2
    b, e = moe.expert_range(n_exp, world, rank)
    g = S.gen_weight(qtype, inter, hidden, seed=5, stream=0)
    u = S.gen_weight(qtype, inter, hidden, seed=5, stream=1)
    d = S.gen_weight(qtype, hidden, inter, seed=5, stream=2)
    n_local = e - b
    ex = moe.MoeExperts(qtype, [g] * n_local, [u] * n_local, [d] * n_local, hidden, inter, n_exp,
                        expert_begin=b, ctx=ctx)
    rng = np.random.default_rng(5)
    logits = torch.from_numpy(rng.standard_normal((tokens, n_exp)).astype(np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((tokens, hidden)).astype(np.float32)).cuda()

    def rows_forward(lg, xr, k):
        y = torch.empty((xr.shape[0], hidden), device="cuda")
        ex.forward(lg, xr, y, k)
        return y

    lo, hi = tokens * rank // world, tokens * (rank + 1) // world
    summed = moe.ExpertShardedMoe(n_exp, world, rank, rows_forward)
    exchanged = moe.TokenExchangeMoe(n_exp, world, rank, rows_forward)
    my_logits, my_x = logits[lo:hi].contiguous(), x[lo:hi].contiguous()
    out = {}
    with torch.cuda.stream(stream):
        for name, step in (("all_reduce", lambda: summed.forward(logits, x, top_k)),
                           ("token_exchange", lambda: exchanged.forward(my_logits, my_x, top_k))):
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            iters = 20
            e0.record(stream)
            for _ in range(iters):
                step()
            e1.record(stream)
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[name] = {"ms": float(t), "tflops_aggregate": 180.39e9 / float(t) / 1e9}
    ex.free()
    out["workload"] = (f"config[4]: 8 x {S.NAMES[qtype]} experts over {world} GPUs, 256 tokens, top-2, whole layer "
                       "with its collective: all_reduce = tokens replicated, outputs summed by NCCL; "
                       "token_exchange = 256 / N tokens owned per rank, routed rows by NCCL all-to-all and back "
                       "(the ids are read back to the host for the split sizes)")
    return out


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs (read-only queries).

    NVML through pynvml when it is importable: a background thread samples every 2 ms and
    the timing loop calls sample_now() once while its launches are still executing, so that
    even a region of a few milliseconds has a sample taken under load.  Without pynvml,
    nvidia-smi in a loop (its first line takes longer than a short region)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.nvml, self.handle, self.samples, self.stop_flag, self.t = None, None, [], False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def sample_now(self):
        if not self.nvml:
            return
        n = self.nvml
        try:
            sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
            smax = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
            r = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
                else n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
            self.samples.append((float(sm), float(smax), int(r)))
        except Exception:
            pass

    def _loop(self):
        while not self.stop_flag:
            self.sample_now()
            time.sleep(0.002)

    def start(self):
        if self.nvml:
            self.t = threading.Thread(target=self._loop, daemon=True)
            self.t.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.nvml:
            self.stop_flag = True
            if self.t:
                self.t.join(timeout=2)
            n = self.nvml
            names = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown", "nvmlClocksThrottleReasonHwSlowdown"),
                     ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
                     ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"),
                     ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap", "nvmlClocksThrottleReasonSwPowerCap"))
            reasons = set()
            for name, a, b in names:
                bit = getattr(n, a, None) or getattr(n, b, None)
                if bit and any(r & bit for _, _, r in self.samples):
                    reasons.add(name)
            sm = [v[0] for v in self.samples]
            return {"sm_mhz": statistics.median(sm) if sm else None,
                    "sm_max_mhz": max(v[1] for v in self.samples) if sm else None,
                    "reasons": sorted(reasons), "samples": len(sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# ------------------------------------------------------------------ CPU arm
TIERS = {0: "scalar", 1: "AVX2+FMA", 2: "AVX-512F"}


def _cpu_lib():
    so = os.path.join(ROOT, "oracle", "_build", "libqk_cpu_simd.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    return C.CDLL(so)


def cpu_gemv_rate(seconds: float, threads: int | None = None, tier: int | None = None, qtype=QTYPE, rows=ROWS,
                  cols=COLS, w=None):
    """Times the reference's CPU tiers restated in oracle/qk_cpu_simd.c on this host."""
    lib = _cpu_lib()
    tier = lib.qk_cpu_best_tier() if tier is None else tier
    cores = threads or lib.qk_cpu_max_threads()
    w = S.gen_weight(qtype, rows, cols, seed=0, stream=0) if w is None else w
    x = S.gen_acts(1, cols, seed=0)[0]
    y = np.zeros(rows, np.float32)
    used = C.c_int()

    def once():
        lib.qk_cpu_gemv(qtype, tier, cores, C.c_void_p(w.ctypes.data), C.c_size_t(rows), C.c_size_t(cols),
                        C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data), C.byref(used))

    for _ in range(3):
        once()
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        once()
        n += 1
    dt = time.perf_counter() - t0
    return {"value": w.size * n / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} matvecs of the full {rows}x{cols} {S.NAMES[qtype]} weight in {dt:.1f} s, "
                      f"{TIERS[used.value]} rows, row-parallel over {cores} threads", "ms_per_matvec": dt / n * 1e3}


def cpu_tiers_one_core(seconds_each: float):
    """What the reference actually runs (its call chain is single-threaded): the scalar, AVX2 and
    AVX-512 row kernels on one core, same weight and activations as the headline."""
    lib = _cpu_lib()
    best = lib.qk_cpu_best_tier()
    w = S.gen_weight(QTYPE, ROWS, COLS, seed=0, stream=0)
    out = {}
    for tier in range(best + 1):
        r = cpu_gemv_rate(seconds_each, threads=1, tier=tier, w=w)
        out[TIERS[tier]] = {"value": r["value"], "unit": UNIT, "ms_per_matvec": r["ms_per_matvec"]}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = max(1.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_gemv_rate(min(per_step, 1.0))
    vals = [cpu_gemv_rate(per_step) for _ in range(args.steps)]
    v = statistics.mean(r["value"] for r in vals)
    base = vals[-1]
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": RING * base["ms_per_matvec"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "host cores only; each step is a bounded sample of the workload"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ GPU arm
def sharded_rate(torch, dist, ctx, qtype, rows, cols, stream, world, rank, launches=64):
    """Strong scaling of one large matrix: rows split over the ranks, every matvec's output
    gathered on all ranks (the unpacking wait trails the next matvec by one call; four gather
    objects rotate).  Microseconds per matvec, maximum over the ranks."""
    from oxillama_b200.device import check_device_status
    from oxillama_b200.sharded import PeerGather, shard_rows
    b, e = shard_rows(rows, world, rank)
    host = big_weight(qtype, rows, cols, 0, 55)
    dws = ring_of(qtype, rows, cols, ctx, row_begin=b, row_end=e, host=host)
    n = len(dws)
    n += (-n) % 4
    pgs = [PeerGather(e - b, ctx=ctx) for _ in range(4)]
    x = torch.from_numpy(S.gen_acts(1, cols, seed=1)).cuda()

    def fn():
        for i in range(n):
            pgs[i % 4].gemm(dws[i % len(dws)], x, 1, unpack=pgs[(i - 1) % 4] if i else None)
        pgs[(n - 1) % 4].wait()
    torch.cuda.synchronize()
    dist.barrier()
    us = graph_us(torch, stream, fn, n, launches)
    check_device_status(ctx, stream)
    t = torch.tensor([us], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    nbytes = S.weight_nbytes(qtype, rows, cols)
    for pg in pgs:
        pg.free()
    for d in dws:
        d.free()
    us = float(t)
    peak, which = peaks()
    return {"workload": f"{S.NAMES[qtype]} {rows}x{cols}, M=1, rows split over {world} GPUs, output gathered on all",
            "us_per_matvec": us, "aggregate_weight_gbs": nbytes / us / 1e3, "frac_of_n_gpus_hbm": nbytes / us / 1e3 / (peak * world),
            "peak_source": which}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from oxillama_b200.device import DeviceWeights, check_device_status
    from oxillama_b200.kernels import Context, CudaQuantKernel, QuantTensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for --impl ours")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context(local)

    # ---- synthetic workload: RING distinct shards of this rank's rows
    host_w = [S.gen_weight(QTYPE, ROWS, COLS, seed=0, stream=rank * RING + i) for i in range(RING)]
    dws = [DeviceWeights(QTYPE, w, ROWS, COLS, ctx=ctx) for w in host_w]
    algo_bytes = dws[0].algo_bytes
    x_host = torch.from_numpy(S.gen_acts(1, COLS, seed=0)[0]).pin_memory()
    y_host = torch.empty(world * ROWS, dtype=torch.float32).pin_memory()
    x = x_host.cuda()
    ys = [torch.empty(ROWS, device="cuda") for _ in range(RING)]
    gathered = torch.empty(world * ROWS, device="cuda") if world > 1 else None
    stream = torch.cuda.Stream()
    # N > 1: every matvec's shard output goes to all ranks.  "peer": the matvec kernel stores
    # it, tagged, into every rank's slots over NVLink and a bounded unpacking wait follows;
    # "nccl": an NCCL all-gather after the matvec.
    peer = world > 1 and args.collective == "peer"
    pgs = []
    gather_checked = None
    if peer:
        # every rank must take the same route: agree on whether the IPC setup worked everywhere
        from oxillama_b200.sharded import PeerGather
        ok = torch.ones(1, device="cuda")
        try:
            pgs = [PeerGather(ROWS, m_cap=1, ctx=ctx) for _ in range(4)]
        except Exception as e:  # noqa: BLE001 - any failure means "use the NCCL route"
            print(f"rank {rank}: peer-store gather unavailable ({e!r}); falling back to NCCL", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0.0:
            peer, pgs = False, []
    if peer:
        # correctness before speed: the gathered vector of four matvecs against an NCCL
        # all-gather of the plain single-GPU results, bit for bit, on every rank
        good = torch.ones(1, device="cuda")
        with torch.cuda.stream(stream):
            for i in range(4):
                pgs[i].gemm(dws[i], x, 1)
                pgs[i].wait()
                dws[i].gemv(x, ys[i])
                stream.synchronize()
                dist.all_gather_into_tensor(gathered, ys[i])
                if not torch.equal(pgs[i].buffer[0], gathered):
                    good.zero_()
            torch.cuda.synchronize()
        dist.all_reduce(good, op=dist.ReduceOp.MIN)
        gather_checked = bool(float(good) == 1.0)

    def step(trail=True):
        for i in range(RING):
            if peer:
                # trail: matvec i also unpacks (waits for, with a bound) all ranks' blocks of matvec
                # i - 1, which crossed NVLink meanwhile (four gather objects rotate); else every
                # matvec is followed at once by its own unpacking kernel (one dependent chain, two
                # objects).
                if trail:
                    pgs[i % 4].gemm(dws[i], x, 1, unpack=pgs[(i - 1) % 4] if i else None)
                else:
                    pgs[i % 2].gemm(dws[i], x, 1)
                    pgs[i % 2].wait()
                continue
            dws[i].gemv(x, ys[i])
            if world > 1:
                dist.all_gather_into_tensor(gathered, ys[i])
        if peer and trail:
            pgs[(RING - 1) % 4].wait()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):  # also the first-use setup of every kernel
            step()
        barrier()
        check_device_status(ctx, stream)
        # One step is captured once into a CUDA graph and replayed: at ~10 us per matvec
        # the host would otherwise be the bottleneck of a launch-bound loop.
        graph = None
        if (world == 1 or peer) and not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
        run = graph.replay if graph is not None else step
        for _ in range(3):
            run()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        barrier()
        ev[0].record(stream)
        for _ in range(args.steps):
            run()
        ev[1].record(stream)
        if rank == 0:
            sampler.sample_now()  # the launches above are still executing
        barrier()
        clocks = sampler.stop() if rank == 0 else None  # (its thread must not share the interpreter with the e2e loop)
        ms = ev[0].elapsed_time(ev[1])
        check_device_status(ctx, stream)
        chain_ms = None
        if peer:  # the same work as one dependent chain
            g1 = None
            if graph is not None:
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=stream):
                    step(False)
            run1 = g1.replay if g1 is not None else (lambda: step(False))
            for _ in range(3):
                run1()
            barrier()
            n1 = max(1, args.steps // 4)
            e1 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            e1[0].record(stream)
            for _ in range(n1):
                run1()
            e1[1].record(stream)
            barrier()
            chain_ms = e1[0].elapsed_time(e1[1]) / n1
            check_device_status(ctx, stream)

        # kernel-only launch time for the roofline (no gather in the region), graph-replayed at every N
        if world == 1:
            kernel_ms = ms / (args.steps * RING)
        else:
            def plain():
                for i in range(RING):
                    dws[i].gemv(x, ys[i])
            barrier()
            kernel_ms = graph_us(torch, stream, plain, RING, launches=RING * max(10, args.steps // 4)) * 1e-3

    # ---- end to end: host activations in, host outputs back, every call synchronised
    e2e_note = "qk_gemv host-pointer call per matvec; weights cached on device after first use"
    # Every call is synchronised, so the leg is host-timed; a few hundred calls are too few for a
    # stable mean, so it runs at least 100 steps and is scaled to the K steps of the line.
    e2e_steps = max(args.steps, 100)
    barrier()
    if world == 1:
        kern = CudaQuantKernel(QTYPE, ctx)
        qts = [QuantTensor(w, (ROWS, COLS), QTYPE) for w in host_w]
        xn, yn = x_host.numpy(), y_host.numpy()
        for _ in range(10):  # the first call uploads and caches the weights, as a model load does
            for qt in qts:
                kern.gemv(qt, xn, yn)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for qt in qts:
                kern.gemv(qt, xn, yn)
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) * args.steps / e2e_steps
        e2e_d2h = RING * ROWS * 4
    elif peer:
        # the sharded layer as its user calls it: pinned host x in, the gathered y of all
        # ranks back in pinned host memory, per matvec (two gather objects alternate)
        e2e_note = ("sharded call per matvec: H2D of x, shard matvec with in-kernel fan-out, unpacking wait for all "
                    "ranks' blocks, D2H of the gathered y, stream synchronise")
        xd = torch.empty(COLS, device="cuda")
        with torch.cuda.stream(stream):
            def host_call(i):
                xd.copy_(x_host, non_blocking=True)
                pgs[i % 2].gemm(dws[i], xd, 1)
                pgs[i % 2].wait()
                y_host.copy_(pgs[i % 2].buffer[0], non_blocking=True)
                stream.synchronize()
            for i in range(RING):
                host_call(i)
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                for i in range(RING):
                    host_call(i)
            e2e_s = (time.perf_counter() - t0) * args.steps / e2e_steps
            check_device_status(ctx, stream)
        e2e_d2h = RING * world * ROWS * 4
    else:
        e2e_s, e2e_d2h = None, 0

    # ---- the other configurations, beside the headline metric
    extras = {}
    if world == 1 and not args.quick:
        extras["decode_shapes"] = [
            matvec_rate(torch, ctx, S.Q4_0, 4096, 4096, 1, stream),       # config[0]
            matvec_rate(torch, ctx, S.Q6_K, 128256, 4096, 1, stream, launches=24),  # config[2] LM head
            matvec_rate(torch, ctx, S.Q6_K, 4096, 14336, 1, stream),      # config[3] down
            matvec_rate(torch, ctx, S.Q8_0, 4096, 4096, 1, stream),
            matvec_rate(torch, ctx, S.IQ4_XS, 14336, 4096, 1, stream),    # config[4] expert gate / up
        ]
        for r, (qt, rr, cc) in zip(extras["decode_shapes"], ((S.Q4_0, 4096, 4096), (S.Q6_K, 128256, 4096),
                                                             (S.Q6_K, 4096, 14336), (S.Q8_0, 4096, 4096),
                                                             (S.IQ4_XS, 14336, 4096))):
            # the reference's best CPU tier on the same shape, all host cores, about a second each
            c = cpu_gemv_rate(1.0, qtype=qt, rows=rr, cols=cc, w=big_weight(qt, rr, cc, 0, 97))
            r["cpu_all_cores"] = {"value": c["value"], "unit": UNIT, "cores": c["cores"], "sample": c["sample"]}
        extras["small_batch"] = matvec_rates(torch, ctx, S.Q4_K, 14336, 4096, (2, 4, 8, 32, 64, 128), stream)
        extras["layer"] = layer_rates(torch, ctx, (1, 8, 32, 512), stream)
        extras["prefill"] = [matvec_rate(torch, ctx, S.Q4_K, 14336, 4096, 512, stream, bound="tensor", launches=96),
                             matvec_rate(torch, ctx, S.Q8_0, 4096, 4096, 512, stream, bound="tensor", launches=96),
                             matvec_rate(torch, ctx, S.Q6_K, 4096, 14336, 512, stream, bound="tensor", launches=48),
                             matvec_rate(torch, ctx, S.IQ4_XS, 14336, 4096, 512, stream, bound="tensor", launches=96)]
        extras["moe"] = [moe_rate(torch, ctx, S.IQ4_XS, stream), moe_rate(torch, ctx, S.Q4_K, stream)]
    elif world > 1 and peer and not args.quick:
        extras["strong_scaling"] = [sharded_rate(torch, dist, ctx, S.Q6_K, 128256, 4096, stream, world, rank),
                                    sharded_rate(torch, dist, ctx, S.Q4_K, 14336, 4096, stream, world, rank),
                                    sharded_rate(torch, dist, ctx, S.Q6_K, 4096, 14336, stream, world, rank)]
        if 8 % world == 0:  # expert-sharded MoE: this rank's experts for all tokens (outputs summed over the ranks)
            from oxillama_b200 import moe as _moe
            b, e = _moe.expert_range(8, world, rank)
            r = moe_rate(torch, ctx, S.IQ4_XS, stream, n_local=e - b, expert_begin=b)
            t = torch.tensor([r["ms"]], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            r["ms"] = float(t)
            r["tflops_aggregate"] = 180.39e9 / r["ms"] / 1e9
            r["note"] = "local experts' share only; the all-reduce of the outputs is not in the figure"
            extras["moe"] = [r]
            try:
                extras["moe_layer"] = moe_layer_rates(torch, dist, ctx, S.IQ4_XS, stream, world, rank)
            except Exception as exc:  # an auxiliary figure: report it, keep the line
                extras["moe_layer"] = {"error": repr(exc)}

    t = torch.tensor([ms, (e2e_s or 0.0) * 1e3, kernel_ms, chain_ms or 0.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, kernel_ms, chain_ms = (float(v) for v in t.cpu())
    total_bytes = algo_bytes * RING * args.steps * world
    if rank == 0:
        peak, which = peaks()
        achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
        launches_per_matvec = 1
        line = {
            "metric": METRIC, "value": total_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "ring_copies": RING,
                       "l2": f"{RING} distinct weight copies ({RING * algo_bytes / 1e6:.0f} MB) rotate, larger than L2",
                       "sharding": "none" if world == 1 else
                       f"{world} row shards of ({world}x14336)x4096; y of every matvec " +
                       ("stored, tagged, into every rank's slots by the matvec kernel over NVLink; matvec i + 1 "
                        "waits for and unpacks all ranks' blocks of matvec i while its first weight tiles are in "
                        "flight (see dependent_chain for a separate wait directly behind each matvec)" if peer
                        else "all-gathered by NCCL")},
            "e2e": ({"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                     "h2d_bytes_per_step": RING * COLS * 4, "d2h_bytes_per_step": e2e_d2h, "steps_timed": e2e_steps, "note": e2e_note}
                    if e2e_s is not None else None),
            "gpu_launches": RING * args.steps * launches_per_matvec,
            "cuda_graph": graph is not None,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": which, "traffic": DRAM_BYTES_PER_LAUNCH, "algorithmic_bytes_per_launch": algo_bytes,
                         "us_per_launch": kernel_ms * 1e3},
            "clocks": clocks,
        }
        if gather_checked is not None:
            line["gather_checked"] = gather_checked
        if peer and chain_ms:
            line["dependent_chain"] = {
                "value": algo_bytes * RING * world / (chain_ms * 1e-3) / 1e9, "unit": UNIT,
                "ms_per_step": chain_ms,
                "note": "same work, every matvec followed at once by the wait for all ranks' blocks"}
        if world == 1:
            line["cpu_baseline"] = cpu_gemv_rate(args.cpu_seconds)
            if not args.quick:
                line["cpu_baseline"]["one_core"] = cpu_tiers_one_core(2.0)
        line.update(extras)
        print(json.dumps(line))
    for pg in pgs:
        pg.free()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-graph", action="store_true", help="launch every matvec from the host")
    ap.add_argument("--quick", action="store_true", help="the headline metric only (no other configurations)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="N = 1: only the batched-matmul measurements (a short run, e.g. for a profiler)")
    ap.add_argument("--small-batch-only", action="store_true",
                    help="N = 1: only Q4_K 14336x4096 at 8 and 16 activation rows (a short run, e.g. for a profiler)")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the shard outputs reach all ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.small_batch_only:
        import torch
        from oxillama_b200.kernels import Context
        torch.cuda.set_device(0)
        ctx, stream = Context(0), torch.cuda.Stream()
        print(json.dumps({"small_batch": matvec_rates(torch, ctx, S.Q4_K, 14336, 4096, (8, 16), stream)}))
    elif args.prefill_only:
        import torch
        from oxillama_b200.kernels import Context
        torch.cuda.set_device(0)
        ctx, stream = Context(0), torch.cuda.Stream()
        print(json.dumps({"prefill": [
            matvec_rate(torch, ctx, S.Q4_K, 14336, 4096, 512, stream, bound="tensor", launches=30),
            matvec_rate(torch, ctx, S.Q8_0, 4096, 4096, 512, stream, bound="tensor", launches=32)]}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
