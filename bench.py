#!/usr/bin/env python
"""Benchmark of the Q4_K_M dequant-matvec hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Llama-3-8B up/gate shape, 14336 x 4096 Q4_K_M weights (16 superblocks of
144 B per row), fp32 activations, batch 1, synthetic seeded data.  One *step* is one pass over
a batch of 16 distinct weight matrices (16 matvec calls, 528 MB of weights, > 4x the 126 MB L2),
so every call streams its weights from HBM.  The metric is effective bandwidth: algorithmic
bytes (q + x + y = 33 103 872 B per call) / time.

  value   weights, x and y resident in HBM; the step is replayed from a CUDA graph; CUDA events.
  e2e     the same step through the reference-facing runtime call (``dispatch_handle`` over the
          C ABI) with HOST buffers: per call x is copied host->device and y device->host inside
          the timed region (weights resident via the empty-input rule); wall clock.
  N > 1   one process per GPU; every rank holds its own 14336-row shard (global matrix
          N x 14336 rows, weak scaling) and the y slices are assembled with an NCCL all-gather
          after every call.  ``--scaling strong`` shards the fixed 14336 rows instead.

``--impl reference`` times the reference's CPU implementation of the same path (the C
restatement in oracle/, all host threads) on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, N_SB = 14336, 16                      # 14336 x 4096
K_COLS = N_SB * 256
N_MATRICES = 16
Q_BYTES = ROWS * N_SB * 144
ALGO_BYTES_PER_CALL = Q_BYTES + K_COLS * 4 + ROWS * 4   # 33 103 872
METRIC = "q4k_matvec_14336x4096_effective_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


# DRAM traffic of one streaming-kernel launch from an ncu capture of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum); see profiles/.  None until captured.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 33088512   # ncu: dram__bytes_read.sum 33 088 512 B + dram__bytes_write.sum 0 B (y stays in L2)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
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
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.ok:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline_run(seconds_budget: float, threads: int, steps: int | None = None,
                     warmup: int = 1):
    """Times the CPU oracle (reference order, rows split over `threads`) on a row sample of the
    benchmark matrix.  Returns (GB/s, sample description, ms per step, rows in the sample)."""
    import oracle
    synth = importlib.import_module("axiom-compute_b200.synth")
    q = synth.q4k_weights(ROWS, N_SB, synth.config_seed(2, 0))
    x = synth.activations(K_COLS, synth.config_seed(2, 1))
    probe_rows = 1024
    t0 = time.perf_counter()
    oracle.matvec_rows("q4k", q, x, probe_rows, N_SB, threads=threads)
    per_row = (time.perf_counter() - t0) / probe_rows
    n_steps = steps if steps else 5
    rows = int(seconds_budget / max(per_row * (n_steps + warmup), 1e-9))
    rows = max(1024, min(ROWS, rows))
    for _ in range(max(warmup, 1)):
        oracle.matvec_rows("q4k", q, x, rows, N_SB, threads=threads)
    times = []
    for _ in range(n_steps):
        t0 = time.perf_counter()
        oracle.matvec_rows("q4k", q, x, rows, N_SB, threads=threads)
        times.append(time.perf_counter() - t0)
    bytes_step = rows * N_SB * 144 + K_COLS * 4 + rows * 4
    best, mean = min(times), sum(times) / len(times)
    sample = (f"{rows} of {ROWS} rows x {K_COLS} cols of the benchmark matrix per step, {n_steps} "
              f"steps, reference operation order, {threads} thread(s); value from the mean step")
    return bytes_step / mean / 1e9, sample, mean * 1e3, rows, bytes_step / best / 1e9


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_cores()
    budget = 90.0
    gbs, sample, ms, rows, _best = cpu_baseline_run(budget, cores, steps=max(args.steps, 1),
                                                    warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "q4k_matvec up/gate 14336x4096 (Llama-3-8B FFN), batch 1",
                   "note": "reference CPU path (scalar fp32, reference operation order) on host cores"},
        "cpu_baseline": {"value": round(gbs, 4), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
    sharding = importlib.import_module("axiom-compute_b200.sharding")
    synth = pkg.synth

    strong = args.scaling == "strong" and world > 1
    rows_local = ROWS // world if strong else ROWS
    rows_global = ROWS if strong else ROWS * world

    # ---- resident inputs: N_MATRICES distinct weight shards per rank ----
    x_host = synth.activations(K_COLS, synth.config_seed(2, 1))
    x_dev = torch.from_numpy(x_host).to(dev)
    weights = []
    base = synth.q4k_weights(ROWS, N_SB, synth.config_seed(2, 0) + 1000 * rank)
    row_bytes = N_SB * 144
    for m in range(N_MATRICES):
        if m == 0:
            w = base
        else:
            # distinct bytes per matrix without 16 full RNG passes: rotate rows and flip a byte lane
            w = np.roll(base.reshape(ROWS, row_bytes), 97 * m, axis=0).copy()
            w[:, 16 + (m % 128)] ^= np.uint8(m)
            w = w.reshape(-1)
        if strong:
            w = w[rank * rows_local * row_bytes:(rank + 1) * rows_local * row_bytes]
        weights.append(torch.from_numpy(np.ascontiguousarray(w)).to(dev))
    # N > 1: the all-gather is fused into the matvec epilogue (peer stores over NVLink, value and
    # epoch in one word); `--collective nccl` keeps the plain NCCL all-gather after each call instead.
    gather = None
    collective = "none"
    if world > 1:
        collective = args.collective
        if collective == "fused":
            try:
                coll = importlib.import_module("axiom-compute_b200.collective")
                gather = coll.PeerGather(rows_global, N_MATRICES, dev)
            except Exception as exc:   # symmetric memory not available on this box
                sys.stderr.write(f"bench.py: fused all-gather unavailable ({exc!r}); using NCCL\n")
                collective = "nccl"
    y_local = [torch.empty(rows_local, dtype=torch.float32, device=dev) for _ in range(N_MATRICES)]
    y_full = [torch.empty(rows_global, dtype=torch.float32, device=dev) for _ in range(N_MATRICES)] \
        if world > 1 else None
    status = ops.new_status(dev)

    # The 16 calls of a step read the same x and write 16 different y: no call depends on the
    # one before it, which the caller states with pdl = 3 (only the final store of y waits for
    # the previous launch).  The strict figure (pdl = 2: x is read only after the previous
    # launch has completed, as a dependent decode chain needs) is measured beside it.
    pdl_mode = args.pdl if args.pdl >= 0 else 3
    tuning = ops.make_tuning(pdl=pdl_mode)
    tuning_strict = ops.make_tuning(pdl=2)

    def step(tn=None):
        tn = tuning if tn is None else tn
        if gather is not None:
            gather.begin_step()
        for m in range(N_MATRICES):
            if gather is not None:
                gather.matvec(weights[m], x_dev, N_SB, m, status=status, tuning=tn)
            else:
                ops.q4k_matvec(weights[m], x_dev, rows_local, N_SB, y=y_local[m], status=status, tuning=tn)
                if world > 1:
                    sharding.all_gather_rows(y_local[m], rows_global, out=y_full[m])
        if gather is not None:
            gather.finish(status)   # every all-gather of the step is complete inside the timed region

    # ---- parity spot check against the oracle before timing (checker only) ----
    step()
    torch.cuda.synchronize()
    if int(status.item()) != 0:
        raise SystemExit(f"kernel status {int(status.item())}")
    if rank == 0:
        import oracle
        rs = 64
        y_ref = oracle.matvec_rows("q4k", weights[0][:rs * row_bytes].cpu().numpy(), x_host, rs, N_SB)
        _y64, mag = oracle.matvec_rows_f64("q4k", weights[0][:rs * row_bytes].cpu().numpy(), x_host, rs, N_SB)
        got = gather.vector(0)[gather.row_offset:gather.row_offset + rs] if gather is not None else y_local[0][:rs]
        err = float((np.abs(got.cpu().numpy() - y_ref) / mag).max())
        if not err <= 1e-5:
            raise SystemExit(f"parity check failed before timing: norm-wise error {err:.3e}")

    # ---- capture one step in a CUDA graph (launch overhead would otherwise dominate) ----
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = None
    # With collectives in the step the default is plain stream launches: capturing the NCCL
    # all-gather together with programmatic-dependent-launch kernels hung on this stack.
    use_graph = not args.no_graph and (world == 1 or gather is not None or args.force_graph)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            step()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()

    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        run_step()
    ev1.record()
    barrier()
    elapsed_ms = ev0.elapsed_time(ev1)
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    # Keep the GPU under the same load a little longer so the clock sampler sees it.  The number
    # of extra steps is derived from the rank-agreed time, so every rank runs the same count
    # (the steps contain collectives).
    hold_steps = max(20, min(5000, int(400.0 / max(elapsed_ms / args.steps, 1e-3))))
    for _ in range(hold_steps):
        run_step()
    torch.cuda.synchronize()
    sampler.stop()

    strict = None
    if world == 1 and graph is not None and pdl_mode == 3:
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            step(tuning_strict)
        for _ in range(5):
            g2.replay()
        torch.cuda.synchronize()
        n2 = max(50, args.steps // 4)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n2):
            g2.replay()
        e1.record()
        torch.cuda.synchronize()
        us2 = e0.elapsed_time(e1) * 1e3 / (n2 * N_MATRICES)
        strict = {"us_per_call": round(us2, 4),
                  "value": round((rows_local * row_bytes + K_COLS * 4 + rows_local * 4) / us2 / 1e3, 2),
                  "unit": UNIT, "steps": n2,
                  "note": "same step with every call ordered after the previous one (pdl = 2)"}

    calls = args.steps * N_MATRICES
    bytes_per_call_local = rows_local * row_bytes + K_COLS * 4 + rows_local * 4
    total_bytes = float(calls) * bytes_per_call_local * world
    value = total_bytes / (elapsed_ms * 1e-3) / 1e9
    us_per_call = elapsed_ms * 1e3 / calls

    # ---- end to end through the runtime layer (host buffers, dispatch_handle) ----
    e2e = None
    if (rank == 0 or world > 1) and not args.skip_e2e:
        e2e_val, h2d, d2h = run_e2e(pkg, local_rank, weights, x_host, rows_local, args, world,
                                    dist if world > 1 else None, dev)
        e2e = {"value": round(e2e_val, 3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h}

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    achieved = bytes_per_call_local / (us_per_call * 1e-6) / 1e9   # per GPU
    roofline = {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                "kernel": "q4_matvec_stream_kernel<Q4_K_M>", "algorithmic_bytes_per_launch": bytes_per_call_local,
                "peak_source": peak_src,
                "note": "achieved = algorithmic bytes per launch / mean launch-to-launch time over "
                        "the timed region (includes inter-kernel gaps"
                        + (" and the all-gather" if world > 1 else "") + ")"}

    cores = host_cores()
    cpu = None
    if world == 1 and not args.skip_cpu:
        gbs, sample, _ms, _rows, _best = cpu_baseline_run(12.0, cores)
        gbs1, _s1, _m1, _r1, _b1 = cpu_baseline_run(6.0, 1)
        cpu = {"value": round(gbs, 4), "unit": UNIT, "cores": cores, "kind": "port",
               "sample": sample, "single_thread_value": round(gbs1, 4)}

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(elapsed_ms / args.steps, 6), "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": "q4k_matvec up/gate 14336x4096 (Llama-3-8B FFN), batch 1",
            "rows_per_gpu": rows_local, "global_rows": rows_global, "cols": K_COLS,
            "calls_per_step": N_MATRICES,
            "l2": f"inputs larger than L2: {N_MATRICES} distinct weight matrices per GPU "
                  f"({N_MATRICES * rows_local * row_bytes / 1e6:.0f} MB) visited round-robin",
            "launch": "cuda_graph" if graph is not None else "stream",
            "launch_dependency": {3: "independent calls (shared x, distinct y): pdl=3", 2: "strict stream order: pdl=2",
                                  1: "strict stream order: pdl=1", 0: "no programmatic dependent launch"}[pdl_mode],
            "parallelism": "single GPU" if world == 1 else
                           f"rows sharded over {world} GPUs + all-gather of y per call ({collective})",
        },
        "us_per_call": round(us_per_call, 4),
        "pct_of_8TBs": round(100.0 * (bytes_per_call_local / (us_per_call * 1e-6)) / 8e12, 2),
        "strict_stream_order": strict,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": calls + (2 * args.steps if gather is not None else 0), "clocks": sampler.summary(),
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(pkg, device_index, weights, x_host, rows_local, args, world, dist, dev):
    """Same step through CudaContext.dispatch_handle with host buffers (wall clock)."""
    import struct
    import torch
    ctx = pkg.CudaContext.new_with_options(pkg.CudaContextOptions(None, device_index, None))
    plan = pkg.q4_matvec_binding_plan("q4km_dequant_matvec")
    handles = []
    pc = struct.pack("<I", N_SB)
    for m in range(N_MATRICES):
        h = ctx.prepare_kernel([0x07230203, m], plan, 4, "q4km_dequant_matvec", spirv_hash=0xE2E0 + m)
        # upload this matrix once (not timed): the empty-input rule keeps it resident afterwards
        ctx.dispatch_handle(h, (rows_local, 1, 1), [weights[m].cpu().numpy(), x_host, b""],
                            [0, 0, rows_local * 4], pc)
        handles.append(h)
    x_buf = bytearray(x_host.tobytes())   # the caller's host buffer: read again on every dispatch
    y_full = torch.empty(rows_local * world, dtype=torch.float32, device=dev) if world > 1 else None
    bound = [ctx.bind(handles[m], (rows_local, 1, 1), [b"", x_buf, b""], [0, 0, rows_local * 4], pc)
             for m in range(N_MATRICES)]

    def step():
        for m in range(N_MATRICES):
            out = bound[m].run()
            if world > 1:
                y_loc = torch.frombuffer(out[2], dtype=torch.float32).to(dev, non_blocking=True)
                dist.all_gather_into_tensor(y_full, y_loc)
        return out

    steps = max(1, min(args.steps, 200))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    bytes_per_call = rows_local * N_SB * 144 + K_COLS * 4 + rows_local * 4
    val = steps * N_MATRICES * bytes_per_call * world / dt / 1e9
    for h in handles:
        h.drop()
    ctx.drop()
    return val, N_MATRICES * K_COLS * 4, N_MATRICES * rows_local * 4


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
        raise SystemExit(f"kernel status {int(sweep.status.item())}")
    if rank == 0:   # checker only: first rows of the first linear against the oracle
        import oracle
        rs, n_sb = 32, shape.hidden // 256
        wq = sweep.weights[0][0][:rs * n_sb * 144].cpu().numpy()
        h0 = sweep.h.cpu().numpy()
        y_ref = oracle.matvec_rows("q4k", wq, h0, rs, n_sb)
        _y64, mag = oracle.matvec_rows_f64("q4k", wq, h0, rs, n_sb)
        err = float((np.abs(sweep.output(0, 0)[:rs].cpu().numpy() - y_ref) / mag).max())
        if not err <= 1e-5:
            raise SystemExit(f"parity check failed before timing: norm-wise error {err:.3e}")
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
    if rank != 0:
        return
    if status != 0:
        raise SystemExit(f"kernel status {status}")
    weight_bytes = shape.bytes_per_layer * shape.layers
    peak, peak_src = measured_peak()
    agg = weight_bytes / (ms_tok * 1e-3) / 1e9
    line = {
        "metric": "decode_sweep_tokens_per_s", "value": round(1e3 / ms_tok, 3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_tok, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"70B-shaped decode sweep, {shape.layers} layers x (qkv 10240x8192, o 8192x8192, "
                               "gate+up 57344x8192, down 8192x28672) Q4_K_M, batch 1",
                   "weight_bytes": weight_bytes, "exchange": sweep.mode, "launch": "cuda_graph" if graph is not None else "stream",
                   "l2": "inputs larger than L2: every token streams all weights once",
                   "parallelism": "single GPU" if world == 1 else
                                  f"rows of every linear sharded over {world} GPUs, all-gather fused into the "
                                  "producer's epilogue, consumer polls the epoch words"},
        "aggregate_gbs": round(agg, 1), "kv_checksum": float(sweep.kv_checksum().item()),
        "roofline": {"bound": "hbm", "achieved": round(agg / world, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(agg / world / peak, 4), "traffic": None, "peak_source": peak_src,
                     "note": "per-GPU weight bytes per token / token time (all launches, gaps and exchanges included)"},
        "cpu_baseline": None, "e2e": None,
        "gpu_launches": steps * sweep.launches_per_token, "clocks": sampler.summary(),
    }
    print(json.dumps(line), flush=True)


def run_prefill(args):
    """`--workload prefill`: the batched-prefill contraction (M = 512 tokens, K = 4096, N = 14336;
    tensor-pipe bound).  One step = one pass over 8 distinct weight matrices.  Single GPU."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this backend has no CPU path")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pkg = importlib.import_module("axiom-compute_b200")
    ops = importlib.import_module("axiom-compute_b200.ops")
    synth = pkg.synth
    m, n, n_sb, n_mat = 512, ROWS, N_SB, 8
    base = synth.q4k_weights(n, n_sb, synth.config_seed(3, 0))
    rng = np.random.default_rng(synth.config_seed(3, 1))
    a32 = rng.standard_normal((m, n_sb * 256)).astype(np.float32)
    a_bf = torch.from_numpy(a32).to(torch.bfloat16)
    a_dev = a_bf.to(dev)
    weights = []
    for j in range(n_mat):
        w = np.roll(base.reshape(n, -1), 131 * j, axis=0).copy() if j else base
        weights.append(torch.from_numpy(np.ascontiguousarray(w).reshape(-1)).to(dev))
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for _ in range(n_mat)]
    status = ops.new_status(dev)

    indep = not args.prefill_strict   # the 8 calls of a step share A and write 8 different C

    def step(independent=None):
        ind = indep if independent is None else independent
        for j in range(n_mat):
            ops.q4k_prefill(weights[j], a_dev, m, n, n_sb, c=outs[j], status=status, form=args.prefill_form,
                            independent=ind)

    step()
    torch.cuda.synchronize()
    if int(status.item()) != 0:
        raise SystemExit(f"kernel status {int(status.item())}")
    import oracle   # checker only: a few weight rows against dequant-then-GEMM on the CPU
    rows = np.array([0, 127, 128, 9999, n - 1])
    ref = oracle.q4km_prefill(np.ascontiguousarray(base.reshape(n, -1)[rows]).reshape(-1),
                              a_bf.to(torch.float32).numpy(), m, len(rows), n_sb)
    got = outs[0][:, torch.from_numpy(rows).to(dev)].cpu().numpy()
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    if not (np.abs(got - ref) <= 1e-2 * np.maximum(np.abs(ref), rms)).all():
        raise SystemExit("parity check failed before timing")
    steps, warmup = max(1, min(args.steps, 500)), max(3, min(args.warmup, 20))
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    strict = None
    if indep:   # the same step with every call ordered after the one before, for reference
        for _ in range(3):
            step(False)
        torch.cuda.synchronize()
        s_steps = max(1, min(steps, 100))
        e0.record()
        for _ in range(s_steps):
            step(False)
        e1.record()
        torch.cuda.synchronize()
        ms_strict = e0.elapsed_time(e1) / s_steps
        strict = {"us_per_call": round(ms_strict * 1e3 / n_mat, 3),
                  "value": round(2.0 * m * n * n_sb * 256 * n_mat / (ms_strict * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                  "steps": s_steps}
    flops = 2.0 * m * n * n_sb * 256
    tf = flops * n_mat / (ms * 1e-3) / 1e12
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        peak, peak_src = float(pk["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        peak, peak_src = 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"
    line = {
        "metric": "q4k_prefill_512x4096x14336_tflops", "value": round(tf, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Q4_K_M batched prefill, M=512 tokens, K=4096, N=14336, bf16 operands, fp32 accumulate",
                   "calls_per_step": n_mat, "launch": "stream", "form": args.prefill_form,
                   "launch_dependency": "independent calls (shared A, distinct C)" if indep else "strict stream order",
                   "l2": f"{n_mat} distinct weight matrices and outputs per step (0.5 GB) visited round-robin"},
        "us_per_call": round(ms * 1e3 / n_mat, 3), "strict_stream_order": strict,
        "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tf / peak, 4), "traffic": None, "kernel": "q4k_prefill_kernel",
                     "flops_per_launch": flops, "peak_source": peak_src},
        "cpu_baseline": None, "e2e": None, "gpu_launches": steps * n_mat, "clocks": sampler.summary(),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["matvec", "decode70b", "prefill"], default="matvec",
                    help="matvec: the headline 14336 x 4096 metric; decode70b: the 70B-shaped decode sweep")
    ap.add_argument("--layers", type=int, default=80, help="decode70b: layers in the stack")
    ap.add_argument("--prefill-form", type=int, default=0, choices=[0, 1, 2],
                    help="prefill: 0 = library's choice, 1 = one CTA per tile, 2 = CTA pair (cta_group::2)")
    ap.add_argument("--prefill-strict", action="store_true",
                    help="prefill: every call ordered after the one before (no overlap onto idle SMs)")
    ap.add_argument("--decode-mode", choices=["auto", "prepared", "fused", "poll", "mixed"], default="auto",
                    help="decode70b: how a linear's output reaches the next linear (see decode.py)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--no-graph", action="store_true", help="launch from the stream, no CUDA graph")
    ap.add_argument("--collective", choices=["fused", "nccl"], default="fused",
                    help="N > 1: all-gather fused into the matvec epilogue, or NCCL after each call")
    ap.add_argument("--force-graph", action="store_true", help="CUDA graph even with collectives in the step")
    ap.add_argument("--pdl", type=int, default=-1, help="programmatic dependent launch mode (0 off, 1, 2; -1 default)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode70b":
        run_decode(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
