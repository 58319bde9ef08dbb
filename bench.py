#!/usr/bin/env python
"""Headline benchmark: Q4_K decode matvec at the Llama-3-8B FFN-up shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* is one pass of the matvec over a ring of RING distinct device copies
of the 14336 x 4096 Q4_K weight (RING x 33 MB > the 126 MB L2, so every launch
streams its weights from HBM).  `value` is weight-GB/s with everything resident
in HBM (CUDA events on the launching stream); `e2e` is the same metric through
the host-pointer C-ABI call a binding of the reference's `QuantKernel::gemv`
makes (pinned host activations in, host outputs back, copies inside the timed
region).  With N > 1 ranks every rank owns a 14336-row shard of an
(N*14336) x 4096 matrix and the shard outputs are all-gathered over NCCL after
every matvec (weak scaling).

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
NOWAIT = bool(os.environ.get("QK_BENCH_NOWAIT"))  # developer knob: fan out but never wait for the peers
METRIC = "q4_k_gemv_weight_bandwidth"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, from the
# ncu capture summarised in profiles/q4k_gemv_14336x4096_m1_ncu.md
DRAM_BYTES_PER_LAUNCH = 33082112
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


def prefill_rate(torch, ctx, qtype, rows, cols, m, stream, launches=96):
    """Batched matmul (prefill) of one weight shape: TFLOP/s over graph-replayed launches that
    rotate through enough weight copies to exceed L2; everything resident in HBM."""
    from oxillama_b200.device import DeviceWeights, check_device_status
    nbytes = S.weight_nbytes(qtype, rows, cols)
    ring = max(2, min(16, int(300e6 / nbytes) + 1))
    base = S.gen_weight(qtype, rows, cols, seed=0, stream=97)
    dws = [DeviceWeights(qtype, base, rows, cols, ctx=ctx) for _ in range(ring)]
    x = torch.from_numpy(S.gen_acts(m, cols, seed=1)).cuda()
    y = torch.empty(m, rows, device="cuda")
    with torch.cuda.stream(stream):
        for d in dws:
            d.gemm(x, y, m)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for d in dws:
                d.gemm(x, y, m)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        iters = max(1, launches // ring)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        check_device_status(ctx, stream)
    us = e0.elapsed_time(e1) * 1e3 / (iters * ring)
    for d in dws:
        d.free()
    peak, which = tensor_peak()
    tf = 2.0 * m * rows * cols / us / 1e6
    return {"workload": f"{S.NAMES[qtype]} {rows}x{cols} weight x {m} tokens (f32 in, f32 out)", "tflops": tf,
            "us_per_launch": us, "peak_tflops": peak, "peak_source": which, "frac": tf / peak,
            "operands": "fp16 (weights dequantised in the kernel), f32 accumulation in TMEM",
            "launches": iters * ring, "ring_copies": ring}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
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
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU arm
def cpu_gemv_rate(seconds: float, threads: int | None = None):
    """Times the reference's CPU tier restated in oracle/qk_cpu_simd.c on this host."""
    so = os.path.join(ROOT, "oracle", "_build", "libqk_cpu_simd.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = C.CDLL(so)
    tier = lib.qk_cpu_best_tier()
    cores = threads or lib.qk_cpu_max_threads()
    w = S.gen_weight(QTYPE, ROWS, COLS, seed=0, stream=0)
    x = S.gen_acts(1, COLS, seed=0)[0]
    y = np.zeros(ROWS, np.float32)
    used = C.c_int()

    def once():
        lib.qk_cpu_gemv(QTYPE, tier, cores, C.c_void_p(w.ctypes.data), C.c_size_t(ROWS), C.c_size_t(COLS),
                        C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data), C.byref(used))

    for _ in range(3):
        once()
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        once()
        n += 1
    dt = time.perf_counter() - t0
    tiers = {0: "scalar", 1: "AVX2+FMA", 2: "AVX-512F"}
    return {"value": w.size * n / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} matvecs of the full 14336x4096 Q4_K weight in {dt:.1f} s, {tiers[used.value]} rows, "
                      f"row-parallel over {cores} threads", "ms_per_matvec": dt / n * 1e3}


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
    y_host = torch.empty(ROWS, dtype=torch.float32).pin_memory()
    x = x_host.cuda()
    ys = [torch.empty(ROWS, device="cuda") for _ in range(RING)]
    gathered = torch.empty(world * ROWS, device="cuda") if world > 1 else None
    stream = torch.cuda.Stream()
    # N > 1: every matvec's shard output goes to all ranks.  "peer": the matvec kernel stores
    # it into every rank's buffer over NVLink and publishes a flag, a bounded wait follows
    # (two buffers alternate); "nccl": an NCCL all-gather after the matvec.
    peer = (world > 1 or bool(os.environ.get("QK_BENCH_PEER1"))) and args.collective == "peer"
    pgs = []
    if peer:
        # every rank must take the same route: agree on whether the IPC setup worked everywhere
        from oxillama_b200.sharded import PeerGather
        ok = torch.ones(1, device="cuda")
        try:  # (world == 1 with QK_BENCH_PEER1: the protocol's own cost without NVLink)
            pgs = [PeerGather(ROWS, m_cap=1, ctx=ctx) for _ in range(2)]
        except Exception as e:  # noqa: BLE001 - any failure means "use the NCCL route"
            print(f"rank {rank}: peer-store gather unavailable ({e!r}); falling back to NCCL", file=sys.stderr)
            ok.zero_()
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0.0:
            peer, pgs = False, []

    def step(distance=2):
        for i in range(RING):
            if peer:
                # Every matvec fans its block out to all ranks and, before it starts, waits
                # in-kernel (under its prologue) for an earlier matvec's blocks from all ranks:
                # distance 2 = the matvec before the previous one, whose buffer it is about to
                # overwrite (two interleaved dependency chains, the cross-GPU hand-off hidden
                # behind one matvec); distance 1 = the previous one (one decode chain, the
                # hand-off exposed).  Either way every gather is waited for.
                after = pgs[i & 1] if distance == 2 else pgs[(i + 1) & 1]
                pgs[i & 1].gemm(dws[i], x, 1, after=None if NOWAIT else after)
                if i >= RING - 2:
                    pgs[i & 1].wait()
                continue
            dws[i].gemv(x, ys[i])
            if world > 1:
                dist.all_gather_into_tensor(gathered, ys[i])

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
        barrier()
        ms = ev[0].elapsed_time(ev[1])
        check_device_status(ctx, stream)
        chain_ms = None
        if peer:  # the same work as one dependent chain
            g1 = None
            if graph is not None:
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=stream):
                    step(1)
            run1 = g1.replay if g1 is not None else (lambda: step(1))
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

        # kernel-only launch time for the roofline (no collective in the region)
        if world == 1:
            kernel_ms = ms / (args.steps * RING)
        else:
            barrier()
            e2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            e2[0].record(stream)
            for _ in range(args.steps):
                for i in range(RING):
                    dws[i].gemv(x, ys[i])
            e2[1].record(stream)
            torch.cuda.synchronize()
            kernel_ms = e2[0].elapsed_time(e2[1]) / (args.steps * RING)

    # ---- end to end through the reference-facing host-pointer call
    kern = CudaQuantKernel(QTYPE, ctx)
    qts = [QuantTensor(w, (ROWS, COLS), QTYPE) for w in host_w]
    xn, yn = x_host.numpy(), y_host.numpy()
    for qt in qts:  # first call uploads and caches the weights, as a model load does
        kern.gemv(qt, xn, yn)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for qt in qts:
            kern.gemv(qt, xn, yn)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    # ---- prefill (batched matmul) on the tensor cores: reported beside the headline metric
    prefill = None
    if rank == 0 and not args.no_prefill:
        prefill = [prefill_rate(torch, ctx, S.Q4_K, 14336, 4096, 512, stream),
                   prefill_rate(torch, ctx, S.Q8_0, 4096, 4096, 512, stream)]
    t = torch.tensor([ms, e2e_s * 1e3, kernel_ms, chain_ms or 0.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, kernel_ms, chain_ms = (float(v) for v in t.cpu())
    total_bytes = algo_bytes * RING * args.steps * world
    if rank == 0:
        peak, which = peaks()
        achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": total_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "ring_copies": RING,
                       "l2": f"{RING} distinct weight copies ({RING * algo_bytes / 1e6:.0f} MB) rotate, larger than L2",
                       "sharding": "none" if world == 1 else
                       f"{world} row shards of ({world}x14336)x4096; y of every matvec " +
                       ("stored into every rank by the matvec kernel over NVLink; each matvec first waits "
                        "in-kernel for the blocks, from all ranks, of the matvec before the previous one "
                        "(see dependent_chain for distance 1)" if peer else "all-gathered by NCCL")},
            "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": RING * COLS * 4, "d2h_bytes_per_step": RING * ROWS * 4,
                    "note": "qk_gemv host-pointer call per matvec; weights cached on device after first use"},
            "gpu_launches": RING * args.steps,
            "cuda_graph": graph is not None,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": which, "traffic": DRAM_BYTES_PER_LAUNCH, "algorithmic_bytes_per_launch": algo_bytes,
                         "us_per_launch": kernel_ms * 1e3},
            "clocks": clocks,
        }
        if peer and chain_ms:
            line["dependent_chain"] = {
                "value": algo_bytes * RING * world / (chain_ms * 1e-3) / 1e9, "unit": UNIT,
                "ms_per_step": chain_ms,
                "note": "same work, every matvec waiting for the previous one's blocks from all ranks"}
        if world == 1:
            line["cpu_baseline"] = cpu_gemv_rate(args.cpu_seconds)
        line["prefill"] = prefill
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
    ap.add_argument("--no-prefill", action="store_true", help="skip the batched-matmul measurements")
    ap.add_argument("--prefill-only", action="store_true",
                    help="N = 1: only the batched-matmul measurements (a short run, e.g. for a profiler)")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the shard outputs reach all ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.prefill_only:
        import torch
        from oxillama_b200.kernels import Context
        torch.cuda.set_device(0)
        ctx, stream = Context(0), torch.cuda.Stream()
        print(json.dumps({"prefill": [prefill_rate(torch, ctx, S.Q4_K, 14336, 4096, 512, stream, launches=30),
                                      prefill_rate(torch, ctx, S.Q8_0, 4096, 4096, 512, stream, launches=32)]}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
