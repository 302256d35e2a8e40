#!/usr/bin/env python
"""Benchmark of the Q4_K_M dequant-matvec hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the Llama-3-8B up/gate shape, 14336 x 4096 Q4_K_M weights (16 superblocks of 144 B per
row), fp32 activations, batch 1, synthetic seeded data.  One *pass* visits 16 distinct weight
matrices (16 matvec calls, 528 MB of weights, > 4x the 126 MB L2), so every call streams its
weights from HBM; one *step* is PASSES_PER_STEP passes (2048 calls, about 12 ms on one GPU), so
that the timed region is long enough for the clock samples taken inside it whatever --steps is.
The metric is effective bandwidth: algorithmic bytes (q + x + y = 33 103 872 B per call) / time.

  value   weights, x and y resident in HBM; a pass is replayed from a CUDA graph; CUDA events.
  e2e     the same calls through the reference-facing runtime call (``dispatch_handle`` over the
          C ABI) with HOST buffers: per call x goes host->device and y device->host inside the
          timed region (weights resident via the empty-input rule); wall clock.
  N > 1   one process per GPU.  The headline is the split the workload states: the 14336 rows of
          every matrix sharded over the N GPUs (strong scaling), the y slices assembled on every
          GPU by the all-gather fused into the matvec's epilogue.  The weak-scaling figure (every
          GPU holds a whole 14336-row shard of an N x 14336-row matrix) is carried beside it as
          ``weak_scaling``.  Before timing every rank checks rows of EVERY rank's slice of the
          assembled vector against the CPU oracle.
  N = 1   also reports the other configurations as ``sub_records`` (Q4_0 4096 x 4096, the down
          projection 4096 x 14336, the M = 512 prefill, a decode-sweep sample, and the reference's
          own published one-shot dispatch sizes).

``--impl reference`` times the reference's CPU implementation of the same path (the C
restatement in oracle/, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import struct
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, N_SB = 14336, 16                      # 14336 x 4096
K_COLS = N_SB * 256
ROW_BYTES = N_SB * 144
N_MATRICES = 16
PASSES_PER_STEP = 128
# Passes captured in one CUDA graph.  A graph launch starts only after the one before it has
# completed, so with independent calls (which overlap each other on every SM) a one-pass graph
# drains and refills the GPU every 16 calls: 5.65 us per call against 5.16 with 16 passes per graph.
PASSES_PER_GRAPH = 16
Q_BYTES = ROWS * ROW_BYTES
ALGO_BYTES_PER_CALL = Q_BYTES + K_COLS * 4 + ROWS * 4   # 33 103 872
METRIC = "q4k_matvec_14336x4096_effective_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
WORKLOAD = "q4k_matvec up/gate 14336x4096 (Llama-3-8B FFN), batch 1"
ARITH = ("x: 22-bit block fixed point per 64 columns (power-of-two scale from the chunk maximum), exact int32 "
         "dp4a against the 4-bit weights, fp32 scales and row sum")

# The reference's published one-shot dispatch medians (BENCHMARKS.md "NVIDIA RTX PRO 6000 Blackwell
# Workstation": Vulkan, pipeline rebuilt per call, one output per call), in milliseconds.
PUBLISHED_MS = {"dispatch_gpu_q4km_128": 3.38, "dispatch_gpu_q4km_512": 8.84,
                "dispatch_gpu_q4_0_128": 2.56, "dispatch_gpu_q4_0_1024": 3.26}

# DRAM traffic of one streaming-kernel launch from an ncu capture of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum; the 57 KB of y stay in L2).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 33088512


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return {"hbm": float(d["hbm_gbs"]), "hbm_src": "measured (MEASURED_PEAKS.json hbm_gbs)",
                "bf16": float(d["bf16_tflops"]), "bf16_src": "measured (MEASURED_PEAKS.json bf16_tflops, burst)"}
    except Exception:
        return {"hbm": FALLBACK_HBM_GBS, "hbm_src": "fallback (6.65 TB/s copy bandwidth, an earlier B200 measurement)",
                "bf16": FALLBACK_BF16_TFLOPS,
                "bf16_src": "fallback (1.59 PFLOP/s cuBLAS bf16, an earlier B200 measurement)"}


def bench_config(world: int, strong: bool) -> dict:
    """The workload description both arms print (identical keys and values for a given N)."""
    return {"workload": WORKLOAD, "format": "Q4_K_M", "rows": ROWS if strong or world == 1 else ROWS * world,
            "cols": K_COLS, "batch": 1, "matrices_per_pass": N_MATRICES,
            "l2": f"inputs larger than L2: {N_MATRICES} distinct weight matrices "
                  f"({N_MATRICES * Q_BYTES / 1e6:.0f} MB) visited round-robin",
            "split": "single GPU" if world == 1 else f"rows sharded over {world} GPUs, y assembled on every GPU"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self.power_w, self.power_limit_w = [], None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            try:   # read only: the limit in force, for the power figures beside the clocks
                self.power_limit_w = round(pynvml.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0, 1)
            except Exception:
                self.power_limit_w = None
            self.ok = True
        except Exception:
            self.ok = False

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.ok:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()

    def summary(self, elapsed_ms=None):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        med = int(statistics.median(self.samples))
        out = {"sm_mhz": med, "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples),
               "sampled": "inside the timed region only"}
        if elapsed_ms is not None:
            out["ms_times_mhz"] = round(elapsed_ms * med, 1)
        if self.power_w:
            out["power_w"] = {"median": round(statistics.median(self.power_w), 1), "max": round(max(self.power_w), 1),
                              "limit": self.power_limit_w,
                              "note": "NVML board power: a moving average that lags a sub-second run"}
        return out


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------------
# Synthetic weights: one seeded base matrix; matrix m of rank r is the base with its rows rotated
# and one byte lane flipped, so any row of any matrix on any rank can be rebuilt for checking.

def base_matrix():
    synth = importlib.import_module("axiom-compute_b200.synth")
    return synth.q4k_weights(ROWS, N_SB, synth.config_seed(2, 0)).reshape(ROWS, ROW_BYTES)


def matrix_rows(base: np.ndarray, m: int, shard: int, row_begin: int, count: int) -> np.ndarray:
    """Rows [row_begin, row_begin + count) of matrix `m` of weak-scaling shard `shard` (0 for the
    one global matrix of the strong split): the same bytes ``build_matrix`` puts on the device."""
    shift = 97 * m + 1009 * shard
    idx = (np.arange(row_begin, row_begin + count) - shift) % ROWS
    w = base[idx].copy()
    if m or shard:
        w[:, 16 + ((m + 5 * shard) % 128)] ^= np.uint8((m + 16 * shard) & 0xFF)
    return w


def build_matrix(base: np.ndarray, m: int, shard: int) -> np.ndarray:
    return matrix_rows(base, m, shard, 0, ROWS)


# ------------------------------------------------------------------------------------------------
# CPU arm

def cpu_matvec_run(seconds_budget: float, threads: int, steps: int | None = None, warmup: int = 1):
    """Times the CPU oracle (reference order, rows split over `threads`) on the benchmark's matrices,
    visited round-robin like the GPU arm.  A step is `calls` whole-matrix calls, sized from a probe
    so that warmup + steps fit the budget.  Returns a dict."""
    import oracle
    synth = importlib.import_module("axiom-compute_b200.synth")
    base = base_matrix()
    mats = [np.ascontiguousarray(build_matrix(base, m, 0)).reshape(-1) for m in range(N_MATRICES)]
    x = synth.activations(K_COLS, synth.config_seed(2, 1))
    t0 = time.perf_counter()
    oracle.matvec_rows("q4k", mats[0], x, ROWS, N_SB, threads=threads)
    per_call = time.perf_counter() - t0
    n_steps = steps if steps else 5
    calls = int(seconds_budget / max(per_call * (n_steps + warmup), 1e-9))
    calls = max(1, min(N_MATRICES * PASSES_PER_STEP, calls))
    nxt = [1]

    def step():
        for _ in range(calls):
            oracle.matvec_rows("q4k", mats[nxt[0] % N_MATRICES], x, ROWS, N_SB, threads=threads)
            nxt[0] += 1

    for _ in range(max(warmup, 1)):
        step()
    times = []
    for _ in range(n_steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return {"gbs": calls * ALGO_BYTES_PER_CALL / mean / 1e9, "ms_per_step": mean * 1e3, "calls_per_step": calls,
            "us_per_call": mean / calls * 1e6,
            "sample": (f"{calls} whole-matrix calls (14336 x 4096 each, {N_MATRICES} matrices round-robin) per step "
                       f"of the workload's {N_MATRICES * PASSES_PER_STEP}, {n_steps} steps, reference operation "
                       f"order, {threads} thread(s); value from the mean step")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    cores = host_cores()
    r = cpu_matvec_run(60.0, cores, steps=max(args.steps, 1), warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(r["gbs"], 4), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(world, True),
        "calls_per_step": r["calls_per_step"], "us_per_call": round(r["us_per_call"], 2),
        "note": "reference CPU path (scalar fp32, reference operation order) on the host cores; no GPU is used",
        "cpu_baseline": {"value": round(r["gbs"], 4), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": round(r["gbs"], 4), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm

def error_figures(y_gpu, y_ref, y64, mag):
    """The three error figures of a row sample: (i) strict per-row relative error against the
    fp32-sequential CPU result under the reference's own denominator rule, (ii) norm-wise error
    |dy| / sum|w_i x_i| (the gate), (iii) distance to the fp64 result, GPU beside CPU."""
    y_gpu = y_gpu.astype(np.float64)
    y_ref64 = y_ref.astype(np.float64)
    d = np.abs(y_gpu - y_ref64)
    strict = np.where(np.abs(y_ref64) > 1e-10, d / np.maximum(np.abs(y_ref64), 1e-300), d)
    normwise = d / mag
    gpu64 = np.abs(y_gpu - y64) / mag
    cpu64 = np.abs(y_ref64 - y64) / mag
    f = lambda v: float(f"{v:.3e}")
    return {"rows": int(y_ref.size),
            "strict_rel_vs_cpu_f32": {"median": f(np.median(strict)), "p99": f(np.quantile(strict, 0.99)),
                                      "max": f(strict.max()), "frac_within_1e-5": round(float((strict <= 1e-5).mean()), 4)},
            "normwise_vs_cpu_f32": {"max": f(normwise.max()), "median": f(np.median(normwise)), "gate": 1e-5},
            "normwise_vs_f64": {"gpu_max": f(gpu64.max()), "gpu_median": f(np.median(gpu64)),
                                "cpu_f32_max": f(cpu64.max()), "cpu_f32_median": f(np.median(cpu64))}}


def time_graph(torch, dist, world, dev, run_pass, passes_per_step, steps, warmup, sampler=None):
    """W warm-up steps, then exactly `steps` steps between barriers; CUDA events; max over ranks."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        for _ in range(passes_per_step):
            run_pass()
    barrier()
    if sampler is not None:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(steps):
        for _ in range(passes_per_step):
            run_pass()
    ev1.record()
    barrier()
    if sampler is not None:
        sampler.stop()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class MatvecLeg:
    """The 16-matrix pass on this rank's GPU for one way of splitting the rows."""

    def __init__(self, torch, dist, pkg, world, rank, dev, base, x_host, strong, collective):
        self.torch, self.dist, self.world, self.rank, self.dev = torch, dist, world, rank, dev
        self.ops = importlib.import_module("axiom-compute_b200.ops")
        self.sharding = importlib.import_module("axiom-compute_b200.sharding")
        self.strong = strong and world > 1
        self.rows_local = ROWS // world if self.strong else ROWS
        self.rows_global = ROWS if self.strong or world == 1 else ROWS * world
        self.base, self.x_host = base, x_host
        self.x_dev = torch.from_numpy(x_host).to(dev)
        self.weights = []
        for m in range(N_MATRICES):
            if self.strong:
                w = matrix_rows(base, m, 0, rank * self.rows_local, self.rows_local)
            else:
                w = build_matrix(base, m, rank if world > 1 else 0)
            self.weights.append(torch.from_numpy(np.ascontiguousarray(w).reshape(-1)).to(dev))
        self.gather, self.collective = None, "none"
        self.finish_early = True
        if world > 1:
            self.collective = collective
            if collective == "fused":
                coll = importlib.import_module("axiom-compute_b200.collective")
                self.gather = coll.PeerGather(self.rows_global, N_MATRICES, dev)
        self.y_local = [torch.empty(self.rows_local, dtype=torch.float32, device=dev) for _ in range(N_MATRICES)]
        self.y_full = [torch.empty(self.rows_global, dtype=torch.float32, device=dev) for _ in range(N_MATRICES)] \
            if world > 1 and self.gather is None else None
        self.status = self.ops.new_status(dev)
        self.bytes_per_call_local = self.rows_local * ROW_BYTES + K_COLS * 4 + self.rows_local * 4
        self.graphs = {}

    def one_pass(self, tn):
        if self.gather is not None:
            for m in range(N_MATRICES):
                self.gather.matvec(self.weights[m], self.x_dev, N_SB, m, status=self.status, tuning=tn)
            # every all-gather of the pass is complete inside the timed region; with calls declared
            # independent the next pass's matvecs may start while this launch still waits for the words
            self.gather.finish(self.status, let_next_start=self.finish_early and tn.pdl == 3)
            return
        for m in range(N_MATRICES):
            self.ops.q4k_matvec(self.weights[m], self.x_dev, self.rows_local, N_SB, y=self.y_local[m],
                                status=self.status, tuning=tn)
            if self.world > 1:
                self.sharding.all_gather_rows(self.y_local[m], self.rows_global, out=self.y_full[m])

    def assembled(self, m):
        if self.gather is not None:
            return self.gather.vector(m)
        return self.y_full[m] if self.world > 1 else self.y_local[m]

    def check(self, rows_per_slice=64, matrices=(0, 7)):
        """Rows of EVERY rank's slice of the assembled vectors against the CPU oracle (checker only).
        Returns the largest norm-wise error; raises SystemExit on a miss or a kernel status bit."""
        import oracle
        torch = self.torch
        self.one_pass(self.ops.make_tuning(pdl=2))
        torch.cuda.synchronize()
        if int(self.status.item()) != 0:
            raise SystemExit(f"rank {self.rank}: kernel status {int(self.status.item())}")
        worst = 0.0
        for m in matrices:
            got_all = self.assembled(m).cpu().numpy()
            for r in range(self.world):
                if self.strong:
                    begin, shard, mrow = r * self.rows_local, 0, r * self.rows_local
                else:
                    begin, shard, mrow = r * ROWS if self.world > 1 else 0, r if self.world > 1 else 0, 0
                # first and last rows of the slice
                for off in (0, self.rows_local - rows_per_slice):
                    w = matrix_rows(self.base, m, shard, mrow + off, rows_per_slice).reshape(-1)
                    y_ref = oracle.matvec_rows("q4k", w, self.x_host, rows_per_slice, N_SB)
                    _y64, mag = oracle.matvec_rows_f64("q4k", w, self.x_host, rows_per_slice, N_SB)
                    got = got_all[begin + off:begin + off + rows_per_slice]
                    err = float((np.abs(got - y_ref) / mag).max())
                    worst = max(worst, err)
                    if not err <= 1e-5:
                        raise SystemExit(f"rank {self.rank}: parity check failed before timing: matrix {m}, slice of "
                                         f"rank {r}, rows {begin + off}..: norm-wise error {err:.3e}")
        return worst

    def graph_for(self, tn_key, tn, use_graph, passes=1):
        """A callable that runs `passes` passes: a CUDA graph of them, replayed, or plain launches."""
        torch = self.torch

        def run_passes():
            for _ in range(passes):
                self.one_pass(tn)

        if not use_graph:
            return run_passes
        tn_key = (tn_key, passes)
        if tn_key not in self.graphs:
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.one_pass(tn)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                run_passes()
            self.graphs[tn_key] = g
        return self.graphs[tn_key].replay

    def launches_per_pass(self):
        return N_MATRICES + (1 if self.gather is not None else 0)


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    pkg = importlib.import_module("axiom-compute_b200")
    ops = importlib.import_module("axiom-compute_b200.ops")
    synth = pkg.synth
    peaks = measured_peaks()

    strong = world > 1 and args.scaling != "weak"
    base = base_matrix()
    x_host = synth.activations(K_COLS, synth.config_seed(2, 1))
    collective = args.collective
    leg = MatvecLeg(torch, dist, pkg, world, rank, dev, base, x_host, strong, collective)

    # The 16 calls of a pass read the same x and write 16 different y: no call depends on the
    # one before it, which the caller states with pdl = 3 (only the final store of y waits for
    # the previous launch).  The strict figure (pdl = 2: x is read only after the previous
    # launch has completed, as a dependent decode chain needs) is measured beside it.
    pdl_mode = args.pdl if args.pdl >= 0 else 3
    extra = {}
    for item in filter(None, args.tune.split(",")):      # launch tunables for experiments: "threads=256,resident=2"
        k, v = item.split("=")
        extra[k.strip()] = int(v)
    tuning = ops.make_tuning(pdl=pdl_mode, **extra)
    tuning_strict = ops.make_tuning(pdl=2, **extra)

    # ---- parity before timing (checker only): every rank, every rank's slice ----
    peer_err = leg.check()
    # the benchmark's own launch geometry too
    leg.one_pass(tuning)
    torch.cuda.synchronize()
    errors = None
    if world == 1:
        import oracle
        rs = 2048
        w = matrix_rows(base, 0, 0, 0, rs).reshape(-1)
        y_ref = oracle.matvec_rows("q4k", w, x_host, rs, N_SB)
        y64, mag = oracle.matvec_rows_f64("q4k", w, x_host, rs, N_SB)
        errors = error_figures(leg.y_local[0][:rs].cpu().numpy(), y_ref, y64, mag)
        if not errors["normwise_vs_cpu_f32"]["max"] <= 1e-5:
            raise SystemExit(f"parity check failed before timing (benchmark geometry): {errors}")
    if int(leg.status.item()) != 0:
        raise SystemExit(f"kernel status {int(leg.status.item())}")

    # With NCCL collectives in the pass the default is plain stream launches: capturing the NCCL
    # all-gather together with programmatic-dependent-launch kernels hung on this stack.
    use_graph = not args.no_graph and (world == 1 or leg.gather is not None or args.force_graph)
    pps = max(1, args.passes_per_step)
    ppg = math.gcd(pps, max(1, args.passes_per_graph))   # whole graphs per step
    run_pass = leg.graph_for("main", tuning, use_graph, ppg)
    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    elapsed_ms = time_graph(torch, dist, world, dev, run_pass, pps // ppg, args.steps, warm, sampler)
    if int(leg.status.item()) != 0:
        raise SystemExit(f"kernel status {int(leg.status.item())} after the timed region")

    calls = args.steps * pps * N_MATRICES
    us_per_call = elapsed_ms * 1e3 / calls
    value = calls * leg.bytes_per_call_local * world / (elapsed_ms * 1e-3) / 1e9

    strict = None
    if world == 1 and pdl_mode == 3:
        run2 = leg.graph_for("strict", tuning_strict, use_graph, ppg)
        n2 = max(2, min(args.steps, 8))
        ms2 = time_graph(torch, dist, world, dev, run2, pps // ppg, n2, 1)
        us2 = ms2 * 1e3 / (n2 * pps * N_MATRICES)
        strict = {"us_per_call": round(us2, 4), "value": round(leg.bytes_per_call_local / us2 / 1e3, 2), "unit": UNIT,
                  "frac_of_measured_peak": round(leg.bytes_per_call_local / us2 / 1e3 / peaks["hbm"], 4),
                  "steps": n2, "timed_ms": round(ms2, 2),
                  "note": "same step with every call ordered after the previous one (pdl = 2)"}

    # ---- N > 1: the weak-scaling figure beside the strong headline ----
    weak = None
    if world > 1 and strong and not args.skip_weak:
        wleg = MatvecLeg(torch, dist, pkg, world, rank, dev, base, x_host, False, collective)
        werr = wleg.check(matrices=(0,))
        wrun = wleg.graph_for("main", tuning, use_graph, ppg)
        wsteps = max(2, min(args.steps, 6))
        wms = time_graph(torch, dist, world, dev, wrun, pps // ppg, wsteps, 1)
        wcalls = wsteps * pps * N_MATRICES
        weak = {"metric": "q4k_matvec_weak_scaling_14336_rows_per_gpu_effective_bandwidth",
                "value": round(wcalls * wleg.bytes_per_call_local * world / (wms * 1e-3) / 1e9, 2), "unit": UNIT,
                "scaling": "weak", "rows_per_gpu": ROWS, "global_rows": ROWS * world,
                "us_per_call": round(wms * 1e3 / wcalls, 4), "steps": wsteps, "timed_ms": round(wms, 2),
                "peer_slice_check_max_normwise_err": float(f"{werr:.3e}")}
        del wleg

    # ---- end to end through the runtime layer (host buffers, dispatch_handle) ----
    e2e = None
    if not args.skip_e2e:
        e2e = run_e2e(pkg, local_rank, leg, args, world, dist if world > 1 else None, dev)

    sub = None
    if world == 1 and not args.skip_sub:
        sub = run_sub_records(torch, pkg, ops, dev, peaks, args)

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = leg.bytes_per_call_local / (us_per_call * 1e-6) / 1e9   # per GPU
    roofline = {"bound": "hbm", "achieved": round(achieved, 2), "peak": peaks["hbm"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm"], 4),
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if leg.rows_local == ROWS else
                int(NCU_TRAFFIC_BYTES_PER_LAUNCH * leg.bytes_per_call_local / ALGO_BYTES_PER_CALL),
                "kernel": "q4_matvec_stream_kernel<Q4_K_M>", "algorithmic_bytes_per_launch": leg.bytes_per_call_local,
                "peak_source": peaks["hbm_src"],
                "note": "achieved = algorithmic bytes per launch / mean launch-to-launch time over the timed "
                        "region (includes inter-kernel gaps" + (" and the all-gather" if world > 1 else "") + ")"
                        + ("; traffic scaled from the 14336-row capture by the rows per launch" if leg.rows_local != ROWS else "")}

    cores = host_cores()
    cpu = None
    if world == 1 and not args.skip_cpu:
        r = cpu_matvec_run(12.0, cores)
        r1 = cpu_matvec_run(6.0, 1)
        cpu = {"value": round(r["gbs"], 4), "unit": UNIT, "cores": cores, "kind": "port",
               "sample": r["sample"], "single_thread_value": round(r1["gbs"], 4)}

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": warm,
        "ms_per_step": round(elapsed_ms / args.steps, 6), "higher_is_better": True,
        "scaling": "weak" if world > 1 and not strong else "strong", "vs_baseline": None, "dtype": "f32",
        "arith": ARITH,
        "data": "synthetic",
        "config": bench_config(world, strong or world == 1),
        "calls_per_step": pps * N_MATRICES, "passes_per_step": pps, "timed_region_ms": round(elapsed_ms, 3),
        "launch": {"mode": f"cuda_graph of {ppg} pass(es), replayed" if use_graph else "stream", "tune": args.tune or "default",
                   "dependency": {3: "independent calls (shared x, distinct y): pdl=3", 2: "strict stream order: pdl=2",
                                  1: "strict stream order: pdl=1", 0: "no programmatic dependent launch"}[pdl_mode],
                   "rows_per_gpu": leg.rows_local, "global_rows": leg.rows_global,
                   "exchange": "none" if world == 1 else f"all-gather of y per call ({leg.collective})"},
        "us_per_call": round(us_per_call, 4),
        "pct_of_8TBs": round(100.0 * (leg.bytes_per_call_local / (us_per_call * 1e-6)) / 8e12, 2),
        "peer_slice_check": {"ranks_checked": world, "rows_per_slice": 128, "matrices": [0, 7],
                             "max_normwise_err": float(f"{peer_err:.3e}"), "gate": 1e-5},
        "errors": errors,
        "strict_stream_order": strict, "weak_scaling": weak,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "sub_records": sub,
        "gpu_launches": args.steps * pps * leg.launches_per_pass(), "clocks": sampler.summary(elapsed_ms),
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(pkg, device_index, leg, args, world, dist, dev):
    """The same calls through CudaContext.dispatch_handle with host buffers (wall clock)."""
    import torch
    rows_local, x_host = leg.rows_local, leg.x_host
    ctx = pkg.CudaContext.new_with_options(pkg.CudaContextOptions(None, device_index, None))
    plan = pkg.q4_matvec_binding_plan("q4km_dequant_matvec")
    handles = []
    pc = struct.pack("<I", N_SB)
    for m in range(N_MATRICES):
        h = ctx.prepare_kernel([0x07230203, m], plan, 4, "q4km_dequant_matvec", spirv_hash=0xE2E0 + m)
        # upload this matrix once (not timed): the empty-input rule keeps it resident afterwards
        ctx.dispatch_handle(h, (rows_local, 1, 1), [leg.weights[m].cpu().numpy(), x_host, b""],
                            [0, 0, rows_local * 4], pc)
        handles.append(h)
    x_buf = bytearray(x_host.tobytes())   # the caller's host buffer: read again on every dispatch
    bound = [ctx.bind(handles[m], (rows_local, 1, 1), [b"", x_buf, b""], [0, 0, rows_local * 4], pc)
             for m in range(N_MATRICES)]
    if world > 1:
        # every rank's host ends a pass with all 16 assembled vectors: the 16 slices of a pass go to the
        # device in one copy and are exchanged by one NCCL all-gather (the runtime call itself is
        # single-GPU, as in the reference; assembling is the caller's step)
        stage = torch.empty(N_MATRICES * rows_local, dtype=torch.float32).pin_memory()
        stage_np = stage.numpy()
        y_loc = torch.empty(N_MATRICES * rows_local, dtype=torch.float32, device=dev)
        y_all = torch.empty(world * N_MATRICES * rows_local, dtype=torch.float32, device=dev)
        y_all_host = torch.empty(world * N_MATRICES * rows_local, dtype=torch.float32).pin_memory()

    def one_pass():
        out = None
        for m in range(N_MATRICES):
            out = bound[m].run()
            if world > 1:
                stage_np[m * rows_local:(m + 1) * rows_local] = np.frombuffer(out[2], np.float32)
        if world > 1:
            y_loc.copy_(stage, non_blocking=True)
            dist.all_gather_into_tensor(y_all, y_loc)
            y_all_host.copy_(y_all, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return out

    # result check (checker only): the last call's y against the device-resident path
    out = one_pass()
    torch.cuda.synchronize()
    got = np.frombuffer(bytes(out[2]), np.float32)
    want = leg.ops.q4k_matvec(leg.weights[N_MATRICES - 1], leg.x_dev, rows_local, N_SB).cpu().numpy()
    if not np.array_equal(got, want):
        raise SystemExit("e2e: dispatch_handle result differs from the device-resident call")

    passes = max(8, min(args.steps * args.passes_per_step, 256))
    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(passes):
        one_pass()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    val = passes * N_MATRICES * leg.bytes_per_call_local * world / dt / 1e9

    # Beside it (N = 1): the same calls issued from several host threads.  Dispatches on different
    # handles may run concurrently (crates/axc-runtime/src/context.rs:494-497); each call is still a
    # complete host-to-host round trip, the threads only overlap their launch and completion latencies.
    concurrent = None
    if world == 1 and args.e2e_threads > 1:
        from concurrent.futures import ThreadPoolExecutor
        nt = args.e2e_threads
        per = [bound[i::nt] for i in range(nt)]

        def worker(mine, n_pass):
            for _ in range(n_pass):
                for b in mine:
                    b.run()

        with ThreadPoolExecutor(nt) as pool:
            list(pool.map(lambda mine: worker(mine, 8), per))
            t0 = time.perf_counter()
            list(pool.map(lambda mine: worker(mine, passes), per))
            dtc = time.perf_counter() - t0
        ok = all(np.array_equal(np.frombuffer(bytes(bound[m].outputs[2]), np.float32),
                                leg.ops.q4k_matvec(leg.weights[m], leg.x_dev, rows_local, N_SB).cpu().numpy())
                 for m in range(N_MATRICES))
        if not ok:
            raise SystemExit("e2e: concurrent dispatches returned a wrong result")
        concurrent = {"threads": nt, "value": round(passes * N_MATRICES * leg.bytes_per_call_local / dtc / 1e9, 3),
                      "unit": UNIT, "us_per_call": round(dtc / (passes * N_MATRICES) * 1e6, 3),
                      "note": "same calls, different handles dispatched concurrently from host threads; results checked"}
    for h in handles:
        h.drop()
    ctx.drop()
    cps = args.passes_per_step * N_MATRICES
    extra = cps * rows_local * 4 if world > 1 else 0             # the slices going back up for the exchange
    back = cps * rows_local * 4 * world if world > 1 else 0       # the assembled vectors coming down
    return {"value": round(val, 3), "unit": UNIT, "h2d_bytes_per_step": cps * K_COLS * 4 + extra,
            "d2h_bytes_per_step": cps * rows_local * 4 + back, "us_per_call": round(dt / (passes * N_MATRICES) * 1e6, 3),
            "calls_timed": passes * N_MATRICES, "concurrent": concurrent,
            "api": "CudaContext.dispatch_handle (axc_cuda_dispatch), one handle per matrix, weights resident via "
                   "the empty-input rule, x from and y to host buffers on every call, sequential calls on one thread"
                   + ("; per pass the 16 slices are exchanged by one NCCL all-gather and the assembled vectors "
                      "copied back to the host" if world > 1 else "")}


# ------------------------------------------------------------------------------------------------
# Sub-records: the other configurations, single GPU

def _timed_loop(torch, fn, min_ms=60.0, chunk=64):
    """Runs fn() back to back for at least `min_ms` of device time (after a warm-up); ms per call."""
    for _ in range(chunk):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, total = 0, 0.0
    while total < min_ms and n < 1 << 20:
        e0.record()
        for _ in range(chunk):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
        n += chunk
    return total / n, n, total


def _matvec_sub(torch, ops, synth, dev, peaks, fmt, rows, n, seed_cfg, label):
    """One matvec shape: 16 distinct matrices round-robin from a CUDA graph, independent and strict."""
    import oracle
    blk_b, blk_e = (144, 256) if fmt == "q4k" else (18, 32)
    gen = synth.q4k_weights if fmt == "q4k" else synth.q4_0_weights
    fn = ops.q4k_matvec if fmt == "q4k" else ops.q4_0_matvec
    n_mat = max(4, int(np.ceil(4 * 126e6 / (rows * n * blk_b))))
    n_mat = min(n_mat, 64)
    base = gen(rows, n, synth.config_seed(seed_cfg, 0)).reshape(rows, n * blk_b)
    x_host = synth.activations(n * blk_e, synth.config_seed(seed_cfg, 1))
    x = torch.from_numpy(x_host).to(dev)
    ws = [torch.from_numpy(np.ascontiguousarray(np.roll(base, 31 * m, axis=0)).reshape(-1)).to(dev) for m in range(n_mat)]
    ys = [torch.empty(rows, dtype=torch.float32, device=dev) for _ in range(n_mat)]
    st = ops.new_status(dev)
    bytes_call = rows * n * blk_b + n * blk_e * 4 + rows * 4
    out = {"workload": label, "rows": rows, "cols": n * blk_e, "format": "Q4_K_M" if fmt == "q4k" else "Q4_0",
           "algorithmic_bytes_per_call": bytes_call, "matrices_round_robin": n_mat}
    # parity (checker only): 256 rows against the oracle
    rs = min(rows, 256)
    fn(ws[0], x, rows, n, y=ys[0], status=st, tuning=ops.make_tuning(pdl=3))
    torch.cuda.synchronize()
    y_ref = oracle.matvec_rows(fmt, base[:rs].reshape(-1), x_host, rs, n)
    _y64, mag = oracle.matvec_rows_f64(fmt, base[:rs].reshape(-1), x_host, rs, n)
    err = float((np.abs(ys[0][:rs].cpu().numpy() - y_ref) / mag).max())
    if not err <= 1e-5 or int(st.item()) != 0:
        raise SystemExit(f"sub-record {label}: parity check failed ({err:.3e}, status {int(st.item())})")
    out["max_normwise_err_256_rows"] = float(f"{err:.3e}")
    for key, pdl in (("independent_calls", 3), ("strict_stream_order", 2)):
        tn = ops.make_tuning(pdl=pdl)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for m in range(n_mat):
                fn(ws[m], x, rows, n, y=ys[m], status=st, tuning=tn)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        # several rounds over the matrices per graph: a graph launch starts only after the one before
        # it has completed, so a short graph of independent calls would drain the GPU at every replay
        reps = max(1, -(-128 // n_mat))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for m in range(n_mat):
                    fn(ws[m], x, rows, n, y=ys[m], status=st, tuning=tn)
        ms_pass, n_pass, total = _timed_loop(torch, g.replay, chunk=16)
        us = ms_pass * 1e3 / (n_mat * reps)
        gbs = bytes_call / us / 1e3
        out[key] = {"us_per_call": round(us, 3), "value": round(gbs, 1), "unit": UNIT, "timed_ms": round(total, 1),
                    "calls_per_graph": n_mat * reps,
                    "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm"],
                                 "frac": round(gbs / peaks["hbm"], 4), "peak_source": peaks["hbm_src"]}}
    if int(st.item()) != 0:
        raise SystemExit(f"sub-record {label}: kernel status {int(st.item())}")
    return out


def _prefill_sub(torch, ops, synth, dev, peaks):
    import oracle
    m, n, n_sb, n_mat = 512, ROWS, N_SB, 8
    base = synth.q4k_weights(n, n_sb, synth.config_seed(3, 0))
    rng = np.random.default_rng(synth.config_seed(3, 1))
    a_bf = torch.from_numpy(rng.standard_normal((m, n_sb * 256)).astype(np.float32)).to(torch.bfloat16)
    a_dev = a_bf.to(dev)
    weights = [torch.from_numpy(np.ascontiguousarray(np.roll(base.reshape(n, -1), 131 * j, axis=0)).reshape(-1)).to(dev)
               for j in range(n_mat)]
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for _ in range(n_mat)]
    st = ops.new_status(dev)

    def one_pass(ind):
        for j in range(n_mat):
            ops.q4k_prefill(weights[j], a_dev, m, n, n_sb, c=outs[j], status=st, independent=ind)

    one_pass(False)
    torch.cuda.synchronize()
    rows = np.array([0, 127, 128, 9999, n - 1])
    ref = oracle.q4km_prefill(np.ascontiguousarray(base.reshape(n, -1)[rows]).reshape(-1),
                              a_bf.to(torch.float32).numpy(), m, len(rows), n_sb)
    got = outs[0][:, torch.from_numpy(rows).to(dev)].cpu().numpy()
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    if int(st.item()) != 0 or not (np.abs(got - ref) <= 1e-2 * np.maximum(np.abs(ref), rms)).all():
        raise SystemExit("sub-record prefill: parity check failed")
    flops = 2.0 * m * n * n_sb * 256
    out = {"workload": "Q4_K_M batched prefill, M=512 tokens, K=4096, N=14336, bf16 operands, fp32 accumulate",
           "flops_per_call": flops, "matrices_round_robin": n_mat, "dtype": "bf16", "tolerance": "1e-2 relative"}
    for key, ind in (("strict_stream_order", False), ("independent_calls", True)):
        ms_pass, _n, total = _timed_loop(torch, lambda: one_pass(ind), chunk=8)
        tf = flops * n_mat / (ms_pass * 1e-3) / 1e12
        out[key] = {"us_per_call": round(ms_pass * 1e3 / n_mat, 3), "value": round(tf, 1), "unit": "TFLOP/s",
                    "timed_ms": round(total, 1),
                    "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peaks["bf16"],
                                 "frac": round(tf / peaks["bf16"], 4), "peak_source": peaks["bf16_src"]}}
    if int(st.item()) != 0:
        raise SystemExit("sub-record prefill: kernel status")
    return out


def _decode_sub(torch, ops, dev, peaks, layers):
    decode = importlib.import_module("axiom-compute_b200.decode")
    full = decode.LLAMA_70B
    shape = decode.SweepShape(full.hidden, full.kv, full.ffn, layers)
    sweep = decode.DecodeSweep(shape, dev, tuning=ops.make_tuning(pdl=2))
    g = torch.Generator(device=dev)
    g.manual_seed(0xA0C0 + 4 * 16 + 15)
    sweep.h.copy_(torch.randn(shape.hidden, device=dev, generator=g))

    def step():
        sweep.token()
        sweep.advance()

    step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    ms_tok, n_tok, total = _timed_loop(torch, graph.replay, chunk=8)
    if int(sweep.status.item()) != 0:
        raise SystemExit("sub-record decode: kernel status")
    wbytes = shape.bytes_per_layer * shape.layers
    gbs = wbytes / (ms_tok * 1e-3) / 1e9
    return {"workload": f"decode-sweep SAMPLE: {layers} of the 80 layers of the 70B-shaped stack (qkv 10240x8192, o "
                        "8192x8192, gate+up 57344x8192, down 8192x28672, Q4_K_M), one token, every launch ordered",
            "layers": layers, "weight_bytes": wbytes, "ms_per_token_sample": round(ms_tok, 4),
            "us_per_layer": round(ms_tok * 1e3 / layers, 2),
            "tokens_per_s_extrapolated_to_80_layers": round(1e3 / (ms_tok * 80 / layers), 2),
            "value": round(gbs, 1), "unit": UNIT, "timed_ms": round(total, 1), "mode": sweep.mode,
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm"],
                         "frac": round(gbs / peaks["hbm"], 4), "peak_source": peaks["hbm_src"]}}


def _published_sub(pkg, device_index):
    """The reference's own published cases: one-shot ``dispatch`` (prepare + dispatch + release per
    call) of ONE output at 128 / 512 superblocks and 128 / 1024 Q4_0 blocks, all three buffers
    uploaded and y read back (crates/axc-driver/benches/dispatch_q4km.rs:195-298,
    benches/dispatch.rs:513-687), checked against the CPU oracle first."""
    import oracle
    synth = pkg.synth
    ctx = pkg.CudaContext.new_with_options(pkg.CudaContextOptions(None, device_index, None))
    out = {}
    cases = [("dispatch_gpu_q4km_128", "q4k", 128), ("dispatch_gpu_q4km_512", "q4k", 512),
             ("dispatch_gpu_q4_0_128", "q4_0", 128), ("dispatch_gpu_q4_0_1024", "q4_0", 1024)]
    for name, fmt, n in cases:
        if fmt == "q4k":
            q, x = oracle.generate_q4km_test_data(n, 0xCAFEBABE)
            entry, cpu = "q4km_dequant_matvec", float(oracle.q4km_dequant_matvec_cpu(q, x, n))
        else:
            q = synth.q4_0_weights(1, n, 42)
            x = np.random.default_rng(42).uniform(-1.0, 1.0, n * 32).astype(np.float32)
            entry, cpu = "q4_0_dequant_matvec", float(oracle.q4_0_dequant_matvec_cpu(q, x, n))
        plan = pkg.q4_matvec_binding_plan(entry)
        req = pkg.DispatchRequest([0x07230203, n], plan, [1, 1, 1], [q, x, bytes(4)], [0, 0, 4],
                                  struct.pack("<I", n), entry)
        got = float(np.frombuffer(bytes(ctx.dispatch(req)[2]), np.float32)[0])
        if not abs(got - cpu) <= 1e-3 * max(abs(cpu), 1e-10):
            raise SystemExit(f"sub-record {name}: pre-flight parity failed ({got} vs {cpu})")
        for _ in range(20):
            ctx.dispatch(req)
        samples = []
        t_end = time.perf_counter() + 0.06
        while time.perf_counter() < t_end or len(samples) < 50:
            t0 = time.perf_counter()
            ctx.dispatch(req)
            samples.append(time.perf_counter() - t0)
        med = sorted(samples)[len(samples) // 2] * 1e3
        out[name] = {"median_ms": round(med, 5), "samples": len(samples), "published_ms": PUBLISHED_MS[name],
                     "vs_baseline": round(PUBLISHED_MS[name] / med, 1),
                     "pre_flight_rel_err": float(f"{abs(got - cpu) / max(abs(cpu), 1e-30):.2e}")}
    ctx.drop()
    out["note"] = ("vs_baseline = published median / this median (time-like: above 1 is faster here).  The published "
                   "figures are Vulkan on an RTX PRO 6000 Blackwell with the pipeline rebuilt per call; hardware and "
                   "API differ, so this compares dispatch paths, not kernels.")
    return out


def run_sub_records(torch, pkg, ops, dev, peaks, args):
    synth = pkg.synth
    sub = {}
    sub["q4_0_4096x4096"] = _matvec_sub(torch, ops, synth, dev, peaks, "q4_0", 4096, 128, 1,
                                        "Q4_0 dequant matvec 4096x4096, batch 1")
    sub["q4k_down_4096x14336"] = _matvec_sub(torch, ops, synth, dev, peaks, "q4k", 4096, 56, 2,
                                             "q4k_matvec down 4096x14336 (Llama-3-8B FFN), batch 1")
    sub["q4k_prefill_512x4096x14336"] = _prefill_sub(torch, ops, synth, dev, peaks)
    torch.cuda.empty_cache()
    sub["decode70b_sample"] = _decode_sub(torch, ops, dev, peaks, args.sub_decode_layers)
    torch.cuda.empty_cache()
    sub["published_one_shot_dispatch"] = _published_sub(pkg, dev.index)
    return sub


# ------------------------------------------------------------------------------------------------
# Other workloads (not the headline): the decode sweep and the prefill contraction

def run_decode(args):
    """`--workload decode70b`: tokens/s of the 70B-shaped decode sweep (80 layers x 7 linears,
    38.5 GB of Q4_K_M weights, rows of every linear sharded over the ranks, strong scaling).
    One step = one token.  Not the headline metric: reported beside it."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    decode = importlib.import_module("axiom-compute_b200.decode")
    ops = importlib.import_module("axiom-compute_b200.ops")
    full = decode.LLAMA_70B
    shape = decode.SweepShape(full.hidden, full.kv, full.ffn, args.layers)
    sweep = decode.DecodeSweep(shape, dev, tuning=ops.make_tuning(pdl=args.pdl if args.pdl >= 0 else 2),
                               mode=args.decode_mode)
    g = torch.Generator(device=dev)
    g.manual_seed(0xA0C0 + 4 * 16 + 15)
    sweep.h.copy_(torch.randn(shape.hidden, device=dev, generator=g))

    def step():
        sweep.token()
        sweep.advance()

    sweep.token(normalise_input=False)
    torch.cuda.synchronize()
    if int(sweep.status.item()) != 0:
        raise SystemExit(f"rank {rank}: kernel status {int(sweep.status.item())}")
    # checker only, on every rank: rows of EVERY rank's slice of the first linear's assembled
    # vector against the oracle (any rank's weights can be rebuilt from the seed)
    import oracle
    rs, n_sb = 32, shape.hidden // 256
    rows0 = shape.linears[0][1]
    h0 = sweep.h.cpu().numpy()
    worst = 0.0
    if sweep.mode == "paired":
        # the first exchanged vector: o before its input's scale = sum over ranks of (columns of Wo) x (slice of q).
        # q on the CPU from the whole first matrix, then sampled rows of Wo against it: a wrong or missing
        # part of ANY rank shows in every row.
        hid = shape.hidden
        wq_full = decode.full_matrix(shape, sweep.seed, 0, 0, dev)[:hid * n_sb * 144].cpu().numpy()
        q_full = oracle.matvec_rows("q4k", wq_full, h0, hid, n_sb)
        wo_full = decode.full_matrix(shape, sweep.seed, 0, 1, dev).view(hid, -1)
        got_o = sweep.local_output(0, 1).cpu().numpy()
        for b in (0, hid // 2, hid - rs):
            wo = wo_full[b:b + rs].contiguous().view(-1).cpu().numpy()
            y_ref = oracle.matvec_rows("q4k", wo, q_full, rs, n_sb)
            _y64, mag = oracle.matvec_rows_f64("q4k", wo, q_full, rs, n_sb)
            err = float((np.abs(got_o[b:b + rs] - y_ref) / mag).max())
            worst = max(worst, err)
            if not err <= 2e-5:
                raise SystemExit(f"rank {rank}: parity check failed before timing: summed o, rows {b}..: {err:.3e}")
        del wo_full
    got_all = sweep.output(0, 0).cpu().numpy() if sweep.mode != "paired" else None
    for c in range(decode.CHUNKS if sweep.mode != "paired" else 0):
        wq = decode.synth_chunk(rows0 // decode.CHUNKS, n_sb, sweep.seed + c, dev)[:rs * n_sb * 144].cpu().numpy()
        y_ref = oracle.matvec_rows("q4k", wq, h0, rs, n_sb)
        _y64, mag = oracle.matvec_rows_f64("q4k", wq, h0, rs, n_sb)
        b = c * (rows0 // decode.CHUNKS)
        err = float((np.abs(got_all[b:b + rs] - y_ref) / mag).max())
        worst = max(worst, err)
        if not err <= 1e-5:
            raise SystemExit(f"rank {rank}: parity check failed before timing: first linear, row chunk {c}: "
                             f"norm-wise error {err:.3e}")
    sweep.advance()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            step()
    run = graph.replay if graph is not None else step
    steps, warmup = max(1, min(args.steps, 200)), max(3, min(args.warmup, 10))
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = int(sweep.status.item())
    ms_tok = float(ms.item()) / steps
    if status != 0:
        raise SystemExit(f"rank {rank}: kernel status {status}")
    kv_checksum = float(sweep.kv_checksum().item())   # every rank: may reduce over the ranks
    if world > 1:
        dist.barrier()
    if rank != 0:
        dist.destroy_process_group()
        return
    weight_bytes = shape.bytes_per_layer * shape.layers
    peaks = measured_peaks()
    agg = weight_bytes / (ms_tok * 1e-3) / 1e9
    line = {
        "metric": "decode_sweep_tokens_per_s", "value": round(1e3 / ms_tok, 3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_tok, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "arith": ARITH,
        "data": "synthetic",
        "config": {"workload": f"70B-shaped decode sweep, {shape.layers} layers x (qkv 10240x8192, o 8192x8192, "
                               "gate+up 57344x8192, down 8192x28672) Q4_K_M, batch 1",
                   "weight_bytes": weight_bytes, "exchange": sweep.mode, "launch": "cuda_graph" if graph is not None else "stream",
                   "l2": "inputs larger than L2: every token streams all weights once",
                   "parallelism": "single GPU" if world == 1 else sweep.parallelism},
        "aggregate_gbs": round(agg, 1), "kv_checksum": kv_checksum,
        "us_per_layer": round(ms_tok * 1e3 / shape.layers, 2),
        "peer_slice_check": {"what": "summed partial products of every rank (o of layer 0), 3 x 32 rows" if sweep.mode == "paired"
                             else f"first linear, {rs} rows of each of the {decode.CHUNKS} row chunks (every rank's slice)",
                             "max_normwise_err": float(f"{worst:.3e}"), "gate": 2e-5 if sweep.mode == "paired" else 1e-5},
        "roofline": {"bound": "hbm", "achieved": round(agg / world, 1), "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": round(agg / world / peaks["hbm"], 4), "traffic": None, "peak_source": peaks["hbm_src"],
                     "note": "per-GPU weight bytes per token / token time (all launches, gaps and exchanges included)"},
        "cpu_baseline": None, "e2e": None,
        "gpu_launches": steps * sweep.launches_per_token, "clocks": sampler.summary(float(ms.item())),
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_allgather_share(args):
    """`--workload allgather_share` (N > 1): one pass of the row-sharded matvec as the headline times it
    (16 calls with the all-gather epilogue + the finish launch) against the 16 calls alone, for the
    strong and the weak split: the share of the exchange step's finish launch and the NVLink bytes."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("allgather_share needs more than one rank (launch with torch.distributed.run)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    pkg = importlib.import_module("axiom-compute_b200")
    ops = importlib.import_module("axiom-compute_b200.ops")
    base = base_matrix()
    x_host = pkg.synth.activations(K_COLS, pkg.synth.config_seed(2, 1))
    tn = ops.make_tuning(pdl=3)
    out = {}
    for strong in (True, False):
        leg = MatvecLeg(torch, dist, pkg, world, rank, dev, base, x_host, strong, "fused")
        leg.check(matrices=(0,))

        def matvecs_only():
            for m in range(N_MATRICES):
                leg.gather.matvec(leg.weights[m], leg.x_dev, N_SB, m, status=leg.status, tuning=tn)

        res = {}
        for name, fn in (("pass_with_finish_us", lambda: leg.one_pass(tn)), ("matvec_launches_only_us", matvecs_only)):
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            ppg = max(1, args.passes_per_graph)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for _ in range(ppg):
                    fn()
            ms = time_graph(torch, dist, world, dev, g.replay, max(1, args.passes_per_step // ppg), max(2, min(args.steps, 8)), 1)
            res[name] = round(ms * 1e3 / (max(2, min(args.steps, 8)) * args.passes_per_step), 3)
            if name == "matvec_launches_only_us":
                leg.gather.finish(leg.status)     # end the step the replays left open
                torch.cuda.synchronize()
        res["finish_launch_us"] = round(res["pass_with_finish_us"] - res["matvec_launches_only_us"], 3)
        res["nvlink_bytes_out_per_gpu_per_pass"] = N_MATRICES * leg.rows_local * 8 * (world - 1)
        res["rows_per_gpu"] = leg.rows_local
        if int(leg.status.item()) != 0:
            raise SystemExit(f"rank {rank}: kernel status {int(leg.status.item())}")
        out["strong" if strong else "weak"] = res
        del leg
    dist.barrier()
    if rank == 0:
        print(json.dumps({"metric": "allgather_finish_share", "n_gpus": world, "calls_per_pass": N_MATRICES, **out}), flush=True)
    dist.destroy_process_group()


def run_prefill(args):
    """`--workload prefill`: the batched-prefill contraction (M = 512 tokens, K = 4096, N = 14336;
    tensor-pipe bound), 8 distinct weight matrices round-robin.  Single GPU."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this backend has no CPU path")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pkg = importlib.import_module("axiom-compute_b200")
    ops = importlib.import_module("axiom-compute_b200.ops")
    peaks = measured_peaks()
    sampler = ClockSampler(dev.index)
    sampler.start()
    rec = _prefill_sub(torch, ops, pkg.synth, dev, peaks)
    sampler.stop()
    main = rec["strict_stream_order" if args.prefill_strict else "independent_calls"]
    line = {
        "metric": "q4k_prefill_512x4096x14336_tflops", "value": main["value"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main["us_per_call"] * 8 / 1e3, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": rec["workload"], "calls_per_step": 8, "launch": "stream",
                   "launch_dependency": "strict stream order" if args.prefill_strict else
                   "independent calls (shared A, distinct C)",
                   "l2": "8 distinct weight matrices and outputs per step (0.5 GB) visited round-robin"},
        "us_per_call": main["us_per_call"], "strict_stream_order": rec["strict_stream_order"],
        "independent_calls": rec["independent_calls"],
        "roofline": dict(main["roofline"], unit="TFLOP/s", traffic=None, kernel="q4k_prefill_kernel",
                         flops_per_launch=rec["flops_per_call"]),
        "cpu_baseline": None, "e2e": None, "gpu_launches": None, "clocks": sampler.summary(),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["matvec", "decode70b", "prefill", "allgather_share"], default="matvec",
                    help="matvec: the headline 14336 x 4096 metric; decode70b: the 70B-shaped decode sweep")
    ap.add_argument("--layers", type=int, default=80, help="decode70b: layers in the stack")
    ap.add_argument("--prefill-strict", action="store_true",
                    help="prefill: headline the figure with every call ordered after the one before")
    ap.add_argument("--decode-mode", choices=["auto", "prepared", "fused", "poll", "mixed", "paired"], default="auto",
                    help="decode70b: how a linear's output reaches the next linear (see decode.py)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--passes-per-graph", type=int, default=PASSES_PER_GRAPH,
                    help="passes captured in one CUDA graph (a graph launch starts only after the one before it has completed)")
    ap.add_argument("--passes-per-step", type=int, default=PASSES_PER_STEP,
                    help="16-matrix passes per step (a step is this many graph replays)")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["auto", "weak", "strong"], default="auto",
                    help="N > 1: strong (default: the 14336 rows sharded) or weak (14336 rows per GPU) as the headline")
    ap.add_argument("--no-graph", action="store_true", help="launch from the stream, no CUDA graph")
    ap.add_argument("--collective", choices=["fused", "nccl"], default="fused",
                    help="N > 1: all-gather fused into the matvec epilogue, or NCCL after each call")
    ap.add_argument("--force-graph", action="store_true", help="CUDA graph even with NCCL collectives in the pass")
    ap.add_argument("--pdl", type=int, default=-1, help="programmatic dependent launch mode (0 off, 1, 2, 3; -1 default)")
    ap.add_argument("--tune", default="", help="matvec launch tunables, e.g. threads=256,ctas_per_sm=1,resident=2 "
                                               "(fields of axc_tuning; default: the library's choice)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--e2e-threads", type=int, default=4, help="host threads of the concurrent e2e sub-figure (N = 1)")
    ap.add_argument("--skip-sub", action="store_true", help="skip the sub-records of the other configurations")
    ap.add_argument("--skip-weak", action="store_true", help="N > 1: skip the weak-scaling sub-record")
    ap.add_argument("--sub-decode-layers", type=int, default=8, help="layers in the decode-sweep sample sub-record")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode70b":
        run_decode(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "allgather_share":
        run_allgather_share(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
