#!/usr/bin/env python
"""Benchmark of the population-scoring hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("Secant-SR population scoring"): P = 65,536 seeded
random postfix programs of at most 32 tokens over {+, -, *, protected /, sin, cos, exp,
protected log}, 16 coefficient slots, 64 coefficient sets per program (per-program bank
tables), N = 1,048,576 rows of F = 8 float32 features ~U[-3, 3], target = a hidden seeded
depth-6 expression plus N(0, 0.05) noise, fused squared-error score per (program, set).
One step scores the whole population once.  With N GPUs every rank scores its own
65,536-program shard of an N x 65,536 population against the replicated dataset (weak
scaling); per-program best scores are combined with one all-gather and every rank takes the
same top-1024.

The line printed by rank 0:
  value       scored program-rows per second (programs x rows / time; each program-row
              covers all 64 coefficient sets) over the device time of each step: the library's
              CUDA events on its launch streams plus the combine kernels, max over ranks
  e2e         the same metric over the wall clock of the same steps, each a call of the
              reference-facing secant_cubin_runner_run with host programs, including
              host->device copies of data and banks, program encoding and upload and the
              device->host copy of all scores
  roofline    FP32-pipe roofline of the evaluator kernel: algorithmic
              lane-operations per second over the probed FFMA rate of this device
  cpu_baseline the CPU evaluator timed on this box's cores on a bounded sample
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "gpu-program-specialization_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

from secant_b200 import abi, programs as P  # noqa: E402

WORKLOAD = dict(name="configs[1] Secant-SR population scoring", programs=65536, max_tokens=32, slots=16, banks=64,
                rows=1 << 20, features=8, seed=2)
METRIC = "scored program·rows/sec"


def hidden_target(x, seed, depth=6):
    """Seeded random expression of the given depth over the feature columns, in float32."""
    words = iter(P._stream(seed, 777, 4096).tolist())

    def nxt(n):
        return int(next(words) % n)

    def build(d):
        if d == 0 or (d < depth - 2 and nxt(5) == 0):
            return x[nxt(x.shape[0])] if nxt(4) else np.float32((nxt(2001) - 1000) / 500.0)
        k = nxt(7)
        a = build(d - 1)
        if k == 4:
            return np.sin(a)
        if k == 5:
            return np.cos(a)
        if k == 6:
            return np.tanh(a)
        b = build(d - 1)
        return (a + b, a - b, a * b, a * b / (b * b + np.float32(0.01)))[k]
    with np.errstate(all="ignore"):
        y = np.asarray(build(depth), dtype=np.float32) * np.ones(x.shape[1], dtype=np.float32)
    return np.nan_to_num(y, nan=0.0, posinf=0.0, neginf=0.0).astype(np.float32)


def make_workload(w, rank):
    """Programs and banks of this rank's shard, and the (replicated) dataset."""
    pop = P.random_population(w["seed"], w["programs"], w["max_tokens"], w["features"], w["slots"], 3.0,
                              first_index=rank * w["programs"])
    x = np.stack([P.uniform(w["seed"] + 100, c, w["rows"], -3.0, 3.0) for c in range(w["features"])])
    y = (hidden_target(x, w["seed"]) + P.normal(w["seed"] + 200, 0, w["rows"], 0.05))[None, :].astype(np.float32)
    rng = np.random.Generator(np.random.Philox(key=w["seed"] * 1000 + rank))
    banks = rng.standard_normal((w["programs"], w["banks"], w["slots"]), dtype=np.float32)
    return pop, x, y, banks


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        busy = [v for v in sm if v > 0.5 * max(sm)]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------ CPU evaluator legs ----

def cpu_evaluator():
    """(callable, kind): the reference's own host evaluator when its library was built on
    a machine with the reference checkout (oracle/_ref), else this repository's CPU port."""
    import support as S
    ref = S.reference_lib()
    if ref is not None:
        def run(pop, x, y, banks_shared):
            code, _ = S.reference_toggle_sse(ref, pop, x, y, banks_shared, banks_shared.shape[1], 0)
            assert code == 0
        return run, "reference"

    def run(pop, x, y, banks_shared):
        code, _, _ = S.oracle_toggle_sse(pop, x, y, banks_shared, banks_shared.shape[1], 0)
        assert code == 0
    return run, "port"


def cpu_throughput(w, programs_per_thread, rows, threads, repeats=1):
    """Scored program-rows/s of the CPU evaluator on `threads` host threads, each scoring its
    own slice of a seeded sample of the workload (all 64 coefficient sets, `rows` rows)."""
    run, kind = cpu_evaluator()
    total = programs_per_thread * threads
    pop = P.random_population(w["seed"], total, w["max_tokens"], w["features"], w["slots"], 3.0)
    x = np.stack([P.uniform(w["seed"] + 100, c, rows, -3.0, 3.0) for c in range(w["features"])])
    y = (hidden_target(x, w["seed"]) + P.normal(w["seed"] + 200, 0, rows, 0.05))[None, :].astype(np.float32)
    banks = np.random.Generator(np.random.Philox(key=w["seed"])).standard_normal((w["banks"], w["slots"]), dtype=np.float32)
    parts = [pop.subset(range(t * programs_per_thread, (t + 1) * programs_per_thread)) for t in range(threads)]
    best = None
    for _ in range(repeats):
        workers = [threading.Thread(target=run, args=(parts[t], x, y, banks)) for t in range(threads)]
        t0 = time.perf_counter()
        for th in workers:
            th.start()
        for th in workers:
            th.join()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return total * rows / best, kind, best, f"{total} programs x {w['banks']} sets x {rows} rows"


def reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows, per_thread = 4096, 8
    # size one step to a few seconds from a quick calibration
    rate, kind, dt, _ = cpu_throughput(w, 1, 1024, threads)
    per_thread = max(1, int(rate * 4.0 / (rows * threads)))
    samples = []
    for _ in range(args.warmup):
        cpu_throughput(w, per_thread, rows, threads)
    t_all = time.perf_counter()
    for _ in range(args.steps):
        rate, kind, dt, sample = cpu_throughput(w, per_thread, rows, threads)
        samples.append(dt)
    ms = 1e3 * (time.perf_counter() - t_all) / args.steps
    value = per_thread * threads * rows / (sum(samples) / len(samples))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "program-rows/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "programs": w["programs"], "rows": w["rows"], "features": w["features"],
                       "coefficient_sets": w["banks"], "max_tokens": w["max_tokens"]},
            "cpu_baseline": {"value": value, "unit": "program-rows/s", "cores": threads, "kind": kind,
                             "sample": f"each step: {sample}, {threads} host threads"},
            "e2e": {"value": value, "unit": "program-rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# What the evaluator kernel executes, from one multi-pass profiler capture of a reduced case of this
# workload (4,096 programs x 131,072 rows, the summary is profiles/eval_kernel_configs1_reduced_ncu_full.md).
# Not measured in this run: counters of that kind need a profiler and the full size is too large for it.
EXECUTED_ON_REDUCED_CASE = {
    "source": "profiler capture of a reduced case (4,096 programs x 131,072 rows), not this run",
    "pipe_fma_pct": 32.8, "pipe_alu_pct": 36.6, "pipe_xu_pct": 13.8, "issue_active_pct": 69.0,
    "instruction_cache_hit_pct": 97.6, "fp32_share_of_executed_instructions": 0.335,
}


# ------------------------------------------------------------------------ RK4 arm ----

# The same kind of figures for the rollout kernel: one launch of 2,048 systems of the configs[3]
# population under a profiler (profiles/rk4_kernel_configs3.md), not this run.
RK4_EXECUTED_ON_REDUCED_CASE = {
    "source": "profiler capture of one launch of 2,048 systems, not this run",
    "warp_instructions_per_interpreted_instruction": 50, "fp32_share_of_executed_instructions": 0.138,
    "issue_active_pct_at_2_warps_per_scheduler": 35.7,
}

def rk4_arm(args, w):
    """`--impl rk4`: the rollout-scoring variant (16,384 candidate systems of
    3 right-hand sides with at most 24 tokens over 3 states and 8 coefficients, 64 initial
    conditions, 1,000 fixed RK4 steps scored at every step).  Reference trajectories come from
    the same integrator run on the Lorenz system; programs are seeded random stand-ins."""
    import torch
    from secant_b200.runner import rk4_score
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    systems, S, ics, steps, K = (args.programs or 16384), 3, 64, 1000, 8
    banks = max(1, args.banks)                      # development only: several coefficient sets per system
    pop = P.random_population(4, systems * S, 24, S, K, 1.0)
    ops = P.count_ops(pop).reshape(systems, S).sum(axis=1)
    rng = np.random.Generator(np.random.Philox(key=4))
    coeffs = rng.standard_normal((systems, banks, K), dtype=np.float32)
    h = np.float32(0.01)
    state = rng.uniform(-10, 10, size=(3, ics)).astype(np.float32)
    ref = np.empty((3, ics, steps + 1), dtype=np.float32)
    ref[:, :, 0] = state

    def rhs(v):
        return np.stack([(v[1] - v[0]) * np.float32(10.0), v[0] * (np.float32(28.0) - v[2]) - v[1],
                         v[0] * v[1] - np.float32(8.0 / 3.0) * v[2]]).astype(np.float32)
    for k in range(1, steps + 1):
        k1 = rhs(state); k2 = rhs(state + h / 2 * k1); k3 = rhs(state + h / 2 * k2); k4 = rhs(state + h * k3)
        state = (state + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4)).astype(np.float32)
        ref[:, :, k] = state
    times = (np.arange(steps + 1, dtype=np.float32) * h).astype(np.float32)
    ref_d = torch.from_numpy(ref.reshape(3, ics * (steps + 1))).to(dev)
    times_d, coeffs_d = torch.from_numpy(times).to(dev), torch.from_numpy(coeffs).to(dev)
    lib = abi.load()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    integrated = torch.zeros(1, dtype=torch.int64, device=dev)
    seconds = []
    for it in range(args.warmup + args.steps):
        launches0 = lib.secant_b200_kernel_launch_count()
        integrated.zero_()
        start.record()
        scores = rk4_score(pop, S, ref_d, times_d, coeffs_d, K, banks, integrated=integrated)   # encodes, uploads, integrates, blocks
        stop.record()
        stop.synchronize()
        if it >= args.warmup:
            seconds.append(start.elapsed_time(stop) * 1e-3)
    dt = float(np.median(seconds))           # host threads encode inside the call: the mean follows their stragglers
    # A candidate is integrated until one of its states stops being finite (its score is FLT_MAX from
    # then on), so the work done is what the device counted, not systems x conditions x steps.
    done = float(integrated.item())                                   # (trajectory, step) pairs integrated
    share = done / (float(systems) * banks * ics * steps)
    stage_evals = done * 4
    per_system_step = (4 * ops + 4 * 2 * S + S + 2 * S).astype(np.float64)          # lane operations per (system, IC, step)
    lane_ops = float(per_system_step.mean()) * done                   # weighted by the mean: the counter is not per system
    peak = C.c_double()
    abi.check(lib.secant_b200_fp32_peak_probe(0.5, C.byref(peak)), "fp32 peak probe")
    valid = float((scores < 3.0e38).float().mean().item())
    print(json.dumps({"impl": "rk4", "metric": "candidate systems scored/sec", "value": systems * banks / dt, "unit": "systems/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "configs[3] RK4 rollout scoring", "systems": systems, "coefficient_sets": banks, "states": S, "coefficients": K,
                                 "initial_conditions": ics, "rk4_steps": steps, "max_tokens_per_state": 24,
                                 "mean_ops_per_system": float(ops.mean()), "valid_fraction": valid,
                                 "integrated_share": share, "ms_per_call": [round(x * 1e3, 1) for x in seconds],
                                 "timed": "secant_b200_rk4_score with host programs: encoding, upload and kernels; candidates "
                                          "are integrated until a state stops being finite"},
                      "system_stage_evals_per_s": stage_evals / dt,
                      "gpu_launches": int(lib.secant_b200_kernel_launch_count() - launches0),
                      "roofline": {"bound": "fp32", "achieved": lane_ops / dt / 1e12, "peak": peak.value / 1e12, "unit": "TFLOP/s",
                                   "frac": lane_ops / dt / peak.value, "traffic": None,
                                   "note": "operations of the integrations that were carried out (device counter), mean operation "
                                           "count per system",
                                   "executed": RK4_EXECUTED_ON_REDUCED_CASE}}))


# ------------------------------------------------------ the other benchmark shapes ----

def _device_peak(lib):
    probe = C.c_double()
    abi.check(lib.secant_b200_fp32_peak_probe(0.5, C.byref(probe)), "fp32 peak probe")
    return probe.value


def toggles_arm(args, w):
    """`--impl toggles`: the toggle-heavy shape (16,384 programs of at most 48 tokens whose sub-trees
    are gated by 8 toggle bits, 256 variants x 4 coefficient sets = 1,024 configurations per program,
    262,144 rows of 6 N(0,1) features), fused losses plus the best variant per program."""
    import torch
    from secant_b200 import runner as R
    from secant_b200.runner import Runner
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    lib = abi.load()
    Pn, bits, NB, F, K, N = (args.programs or 16384), 8, 4, 6, 8, (args.rows or 262144)
    pop = P.gated_population(3, Pn, 48, F, K, bits)
    ops = P.count_ops(pop)
    x = torch.from_numpy(np.stack([P.normal(3, c, N) for c in range(F)])).to(dev)
    y = torch.from_numpy(np.stack([P.normal(3, 100, N)])).to(dev)
    banks = torch.from_numpy(np.stack([P.normal(3, 200 + b, K) for b in range(NB)])).to(dev)
    configs = NB << bits
    out = torch.empty((Pn, 1, configs), dtype=torch.float32, device=dev)
    best = torch.empty(Pn * R.SCORE_BYTES, dtype=torch.uint8, device=dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    peak = _device_peak(lib)
    seconds = []
    with Runner(abi.SHAPE_TOGGLE_SSE, F, 1, K, workers=min(8, os.cpu_count() or 2), streams=2) as runner:
        req = runner.toggle_request(pop, x, y, banks, NB, bits, out)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.secant_b200_kernel_launch_count()
        for it in range(args.warmup + args.steps):
            flush.fill_(1)
            torch.cuda.synchronize()
            if it == args.warmup:
                launches0 = lib.secant_b200_kernel_launch_count()
            runner.run(req)
            ev0.record()
            R.best_config(out.view(Pn, configs), out=best)
            ev1.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                seconds.append(runner.stats.runtime_seconds + ev0.elapsed_time(ev1) * 1e-3)
        launches = lib.secant_b200_kernel_launch_count() - launches0
    dt = sum(seconds) / len(seconds)
    lane_ops = float((ops + 2).sum()) * configs * N
    sse, cfg, valid = R.score_fields(best)
    print(json.dumps({"impl": "toggles", "metric": METRIC, "value": float(Pn) * N / dt, "unit": "program-rows/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "toggle-heavy specialization", "programs": Pn, "max_tokens": 48, "toggle_bits": bits,
                                 "coefficient_sets": NB, "configurations_per_program": configs, "rows": N, "features": F,
                                 "mean_ops_per_program": float(ops.mean()), "timed": "secant_cubin_runner_run with host "
                                 "programs (CUDA events of the library's streams) plus the best-variant kernel"},
                      "row_evals_per_s": float(Pn) * configs * N / dt, "gpu_launches": int(launches),
                      "valid_fraction": float((valid > 0).float().mean().item()),
                      "roofline": {"bound": "fp32", "achieved": lane_ops / dt / 1e12, "peak": peak / 1e12, "unit": "TFLOP/s",
                                   "frac": lane_ops / dt / peak, "traffic": None}}))


def box_arm(args, w):
    """`--impl box`: the box-scale shape on one GPU (16 features, 2^22 rows, 16 coefficient sets per
    program, programs of at most 32 tokens) with a program sample sized to seconds.  The 272 MiB
    dataset does not fit the L2 cache, so every group of thread blocks streams its row range from
    HBM: the line reports that stream in GB/s beside the arithmetic fraction."""
    import torch
    from secant_b200.runner import Runner
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    lib = abi.load()
    Pn, NB, F, K, N = (args.programs or 49152), 16, 16, 16, (args.rows or 1 << 22)
    pop = P.random_population(5, Pn, 32, F, K, 1.0)
    ops = P.count_ops(pop)
    x = torch.from_numpy(np.stack([P.uniform(5, c, N, -1.0, 1.0) for c in range(F)])).to(dev)
    y = torch.from_numpy(hidden_target(x.cpu().numpy(), 5, depth=8)[None, :]).to(dev)
    banks = torch.from_numpy(np.random.Generator(np.random.Philox(key=5)).standard_normal((Pn, NB, K), dtype=np.float32)).to(dev)
    out = torch.empty((Pn, 1, NB), dtype=torch.float32, device=dev)
    peak = _device_peak(lib)
    seconds = []
    with Runner(abi.SHAPE_TOGGLE_SSE, F, 1, K, workers=min(8, os.cpu_count() or 2), streams=2) as runner:
        req = runner.toggle_request(pop, x, y, banks, NB, 0, out, bank_stride=K, program_bank_stride=NB * K)
        launches0, stream0 = lib.secant_b200_kernel_launch_count(), lib.secant_b200_row_stream_bytes()
        for it in range(args.warmup + args.steps):
            if it == args.warmup:
                launches0, stream0 = lib.secant_b200_kernel_launch_count(), lib.secant_b200_row_stream_bytes()
            runner.run(req)                      # the dataset is larger than L2: nothing to flush
            if it >= args.warmup:
                seconds.append(runner.stats.runtime_seconds)
        launches = lib.secant_b200_kernel_launch_count() - launches0
        stream = (lib.secant_b200_row_stream_bytes() - stream0) / float(args.steps)
    dt = sum(seconds) / len(seconds)
    lane_ops = float((ops + 2).sum()) * NB * N
    line = {"impl": "box", "metric": METRIC, "value": float(Pn) * N / dt, "unit": "program-rows/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "box-scale population, one GPU's share sampled", "programs": Pn, "rows": N, "features": F,
                       "coefficient_sets": NB, "max_tokens": 32, "dataset_bytes": (F + 1) * 4 * N,
                       "mean_ops_per_program": float(ops.mean())},
            "row_evals_per_s": float(Pn) * NB * N / dt, "gpu_launches": int(launches),
            "roofline": {"bound": "fp32", "achieved": lane_ops / dt / 1e12, "peak": peak / 1e12, "unit": "TFLOP/s",
                         "frac": lane_ops / dt / peak, "traffic": None}}
    line["row_stream"] = {"passes_over_the_dataset": stream / ((F + 1) * 4.0 * N), "bytes_per_step": stream,
                          "GB_per_s": stream / dt / 1e9, "hbm_peak_GB_per_s": 6560.3,
                          "note": "every program group of every launch reads each row once; measured copy peak of this pool's B200s"}
    print(json.dumps(line))


# ------------------------------------------------------------------ comparator arm ----

def comparator_arm(args, w):
    """`--impl comparator`: the reference's kernel design with compiler-written program bodies
    (tests/comparator.py) against this library's evaluator, on the same sample of the
    workload with one shared coefficient table (the reference's bank semantics).  Compile time
    is reported beside the kernel time; it is what the reference's machine-code patching and
    this library's record interpreter both exist to avoid."""
    import torch
    import comparator as K
    from secant_b200.runner import Runner
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    dev = torch.device("cuda", 0)
    count = min(w["programs"], 512)
    NB, Kc, F, N = w["banks"], w["slots"], w["features"], w["rows"]
    w = dict(w, programs=count)
    pop, x_h, y_h, banks_h = make_workload(w, 0)
    x, y, banks = (torch.from_numpy(a).to(dev) for a in (x_h, y_h, np.ascontiguousarray(banks_h[0])))
    row_evals = float(count) * NB * N
    out = torch.empty((count, 1, NB), device=dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    result = {"impl": "comparator", "metric": "row-evals/s", "unit": "row-evals/s", "n_gpus": 1, "data": "synthetic",
              "config": {"workload": w["name"] + f" (sample: {count} programs, shared coefficient table)", "rows": N,
                         "coefficient_sets": NB, "recipe": "8 kernels x 8 programs per module, tile 128 rows, 128 threads"}}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for mode, fast in (("fast_math", True), ("accurate", False)):
        compiled = K.CompiledPopulation(pop, F, Kc, 1, fast_math=fast)
        times = []
        for it in range(args.warmup + args.steps):
            out.zero_()
            flush.fill_(1)
            start.record()
            launches = compiled.score(x, y, banks, NB, 0, out)
            stop.record()
            stop.synchronize()
            if it >= args.warmup:
                times.append(start.elapsed_time(stop) * 1e-3)
        seconds = sum(times) / len(times)
        result[mode] = {"row_evals_per_s": row_evals / seconds, "kernel_ms": seconds * 1e3, "launches": launches,
                        "compile_s": compiled.compile_seconds, "module_load_s": compiled.load_seconds,
                        "compile_ms_per_program": compiled.compile_seconds * 1e3 / count,
                        "finite_fraction": float(torch.isfinite(out).float().mean().item())}
        compiled.close()
    with Runner(abi.SHAPE_TOGGLE_SSE, F, 1, Kc, workers=4, streams=2) as runner:
        req = runner.toggle_request(pop, x, y, banks, NB, 0, out)
        times = []
        for it in range(args.warmup + args.steps):
            flush.fill_(1)
            runner.run(req)                      # encodes and uploads the programs every time
            if it >= args.warmup:
                times.append((runner.stats.runtime_seconds, runner.stats.compile_work_seconds, runner.stats.total_seconds))
        kernel = sum(t[0] for t in times) / len(times)
        result["this_library"] = {"row_evals_per_s": row_evals / kernel, "kernel_ms": kernel * 1e3,
                                  "encode_ms_per_program": 1e3 * sum(t[1] for t in times) / len(times) / count,
                                  "call_ms": 1e3 * sum(t[2] for t in times) / len(times),
                                  "finite_fraction": float(torch.isfinite(out).float().mean().item())}
        runner.set_math(True)                    # the reference GPU kernels' approximations, opt-in
        times = []
        for it in range(args.warmup + args.steps):
            flush.fill_(1)
            runner.run(req)
            if it >= args.warmup:
                times.append(runner.stats.runtime_seconds)
        kernel = sum(times) / len(times)
        result["this_library_fast_math"] = {"row_evals_per_s": row_evals / kernel, "kernel_ms": kernel * 1e3,
                                            "finite_fraction": float(torch.isfinite(out).float().mean().item())}
    result["value"] = result["fast_math"]["row_evals_per_s"]
    print(json.dumps(result))


# ------------------------------------------------------------------------- GPU arm ----

def parity_spot(w, pop, x_h, y_h, banks_h, runner, dev, programs=32, rows=65536):
    """Scores `programs` seeded programs of the timed population on a row prefix with the library and
    with the CPU checker (float64-accumulated sums, widened by the 2-ulp sensitivity of the math
    functions as in tests/parity.py) and counts the bins that disagree."""
    import torch
    from concurrent.futures import ThreadPoolExecutor
    import parity
    import support as S
    NB, K = w["banks"], w["slots"]
    rows = min(rows, x_h.shape[1])
    pick = np.random.Generator(np.random.Philox(key=w["seed"] + 17)).choice(len(pop.asts), size=min(programs, len(pop.asts)),
                                                                           replace=False)
    pick.sort()
    sub = pop.subset(pick.tolist())
    xs, ys = np.ascontiguousarray(x_h[:, :rows]), np.ascontiguousarray(y_h[:, :rows])
    bs = np.ascontiguousarray(banks_h[pick])
    out = torch.empty((len(pick), 1, NB), dtype=torch.float32, device=dev)
    req = runner.toggle_request(sub, torch.from_numpy(xs).to(dev), torch.from_numpy(ys).to(dev), torch.from_numpy(bs).to(dev),
                                NB, 0, out, bank_stride=K, program_bank_stride=NB * K)
    runner.run(req)
    got = out.cpu().numpy()

    def check(i):
        one = sub.subset([i])
        code, _, want64 = S.oracle_toggle_sse(one, xs, ys, bs[i:i + 1], K, 0, bank_stride=K, program_bank_stride=NB * K)
        assert code == 0
        slack = S.sse_slack(one, xs, ys, bs[i:i + 1], K, 0, program_bank_stride=NB * K)
        bad = parity.sse_mismatches(got[i:i + 1], want64, slack)
        return int(bad.sum()), int((~np.isfinite(slack)).sum()), int(bad.size)
    with ThreadPoolExecutor(max_workers=min(len(pick), os.cpu_count() or 1)) as pool:
        results = list(pool.map(check, range(len(pick))))
    return {"programs": int(len(pick)), "rows": int(rows), "bins": sum(r[2] for r in results), "bad": sum(r[0] for r in results),
            "skipped": sum(r[1] for r in results), "rule": "1e-4 relative to the float64-accumulated checker sum, widened by 2-ulp sensitivity"}


def gpu_arm(args, w):
    import torch
    import torch.distributed as dist
    from secant_b200 import sharding
    from secant_b200.runner import Runner

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the evaluator has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lib = abi.load()

    # roofline denominator and (single-GPU runs only) the CPU baseline, before any rank waits on another
    peak, cpu = None, None
    if rank == 0:
        probe = C.c_double()
        abi.check(lib.secant_b200_fp32_peak_probe(0.5, C.byref(probe)), "fp32 peak probe")
        peak = probe.value
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            rate, kind, dt, sample = cpu_throughput(w, 1, 1024, threads)
            per_thread = max(1, int(rate * 5.0 / (4096 * threads)))
            rate, kind, dt, sample = cpu_throughput(w, per_thread, 4096, threads)
            cpu = {"value": rate, "unit": "program-rows/s", "cores": threads, "kind": kind,
                   "sample": f"{sample}, {dt:.1f} s on {threads} host threads"}
            one, _, dt1, sample1 = cpu_throughput(w, max(1, per_thread // 4), 4096, 1)  # the evaluator as shipped is single-threaded
            cpu["one_thread"] = {"value": one, "sample": f"{sample1}, {dt1:.1f} s"}
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    Pn, NB, K, F, N = w["programs"], w["banks"], w["slots"], w["features"], w["rows"]
    pop, x_h, y_h, banks_h = make_workload(w, rank)
    ops = P.count_ops(pop)
    lane_ops_per_step = float((ops + 2).sum()) * NB * N          # W = n_ops + 2 per (program, set, row)
    pin = lambda a: torch.from_numpy(a).pin_memory()
    x_pin, y_pin, banks_pin = pin(x_h), pin(y_h), pin(banks_h)
    scores_pin = torch.empty((Pn, 1, NB), dtype=torch.float32).pin_memory()
    top_pin = torch.empty(1024, dtype=torch.int64).pin_memory()
    x_d, y_d, banks_d = torch.empty_like(x_pin, device=dev), torch.empty_like(y_pin, device=dev), torch.empty_like(banks_pin, device=dev)
    out = torch.empty((Pn, 1, NB), dtype=torch.float32, device=dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)   # larger than the 126 MB L2

    # best set per program (device kernel writing straight into the all-gather send buffer), one
    # all-gather of the 24-byte records, the same top-1024 kernel on every rank
    combine_step = sharding.Combine(world * Pn, world, rank, 1024, dev)
    k_top = combine_step.k

    def combine(scores):
        return combine_step(scores.view(Pn, NB))[0]

    runner = Runner(abi.SHAPE_TOGGLE_SSE, F, 1, K, workers=min(8, max(2, (os.cpu_count() or 2) // max(1, world))), streams=2)
    req = runner.toggle_request(pop, x_d, y_d, banks_d, NB, 0, out, bank_stride=K, program_bank_stride=NB * K)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def step():
        """One pass of the hot path through the reference-facing call: host buffers in, scores out.
        Returns (wall seconds, device seconds of the evaluation and of the combine step)."""
        t0 = time.perf_counter()
        flush.fill_(1)
        x_d.copy_(x_pin, non_blocking=True)
        y_d.copy_(y_pin, non_blocking=True)
        banks_d.copy_(banks_pin, non_blocking=True)
        torch.cuda.current_stream().synchronize()          # the library's streams do not wait on torch's
        runner.run(req)                                      # encodes and uploads the programs, evaluates, blocks
        device_s = runner.stats.runtime_seconds              # CUDA events on the library's launch streams
        ev0.record()
        top = combine(out)
        ev1.record()
        scores_pin.copy_(out, non_blocking=True)
        top_pin[:k_top].copy_(top, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return time.perf_counter() - t0, device_s + ev0.elapsed_time(ev1) * 1e-3

    steps, warmup = args.steps, args.warmup
    budget = float(os.environ.get("SECANT_BENCH_BUDGET_S", "700"))
    t_first = time.perf_counter()
    done_warm = 0
    if warmup:
        step()
        done_warm = 1
        first = time.perf_counter() - t_first
        plan = torch.tensor([first], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(plan, op=dist.ReduceOp.MAX)
        first = float(plan.item())
        if first * (steps + warmup) > budget:                # keep the whole run inside the time the caller allows
            room = max(2, int(budget / first))
            warmup = min(warmup, max(1, min(3, room - 1)))
            steps = max(1, min(steps, room - warmup))
    for _ in range(done_warm, warmup):
        step()
    barrier()
    launches_before = lib.secant_b200_kernel_launch_count()
    walls, devices = [], []
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        for _ in range(steps):
            wall, device_s = step()
            walls.append(wall)
            devices.append(device_s)
        barrier()
        total_wall = time.perf_counter() - t0
    launches = lib.secant_b200_kernel_launch_count() - launches_before
    clock_summary = clocks.summary()
    encode_s, upload_s = runner.stats.compile_work_seconds, runner.stats.module_load_seconds
    per_rank = torch.tensor([total_wall / steps, sum(devices) / len(devices)], dtype=torch.float64, device=dev)
    all_ranks = [torch.empty_like(per_rank) for _ in range(world)]
    if world > 1:
        dist.all_gather(all_ranks, per_rank)
    else:
        all_ranks = [per_rank]
    step_wall = max(float(t[0]) for t in all_ranks)
    step_device = max(float(t[1]) for t in all_ranks)
    h2d = x_h.nbytes + y_h.nbytes + banks_h.nbytes + len(pop.ast_blob)
    d2h = scores_pin.numel() * 4 + k_top * 8

    line = None
    if rank == 0:
        spot = None
        if not args.no_cpu:
            try:
                spot = parity_spot(w, pop, x_h, y_h, banks_h, runner, dev)
            except Exception as exc:  # the line is still printed
                spot = {"error": repr(exc)}
        achieved = lane_ops_per_step / step_device
        total_program_rows = float(Pn) * N * world
        line = {
            "metric": METRIC, "value": total_program_rows / step_device, "unit": "program-rows/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": step_device * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "programs_per_gpu": Pn, "rows": N, "features": F, "coefficient_slots": K,
                       "coefficient_sets": NB, "banks": "per-program", "max_tokens": w["max_tokens"],
                       "row_evals_per_step_per_gpu": float(Pn) * NB * N, "mean_ops_per_program": float(ops.mean()),
                       "l2": "192 MiB flush between steps", "combine": "best-set kernel, all-gather of 24-byte records, top-1024 kernel",
                       "timed": "value: CUDA events of the library's launch streams plus the combine kernels, inputs resident; "
                                "e2e: wall clock of the same steps including host-to-device copies of data and banks, program "
                                "encoding and upload, and the device-to-host copy of all scores",
                       "steps_requested": args.steps, "warmup_requested": args.warmup,
                       "per_rank_device_ms": [float(t[1]) * 1e3 for t in all_ranks]},
            "row_evals_per_s": float(Pn) * NB * N * world / step_device,
            "node_evals_per_s": lane_ops_per_step * world / step_device,
            "e2e": {"value": total_program_rows / step_wall, "unit": "program-rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": step_wall * 1e3, "encode_ms": encode_s * 1e3,
                    "program_upload_ms": upload_s * 1e3},
            "gpu_launches": int(launches),
            "clocks": clock_summary,
            "roofline": {"bound": "fp32", "achieved": achieved / 1e12, "peak": peak / 1e12, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None,
                         "note": "achieved = sum over programs of (ops + 2) x sets x rows / device time, one per "
                                 "algorithmic operation; peak = FFMA lane-instructions/s probed on this device in this "
                                 "run; DRAM traffic needs a multi-pass capture: measured on a reduced case only and not "
                                 "proportional to the unit count",
                         "executed": EXECUTED_ON_REDUCED_CASE},
            "cpu_baseline": cpu,
            "parity_spot": spot,
            "top1024_head": [int(i) for i in top_pin[:4].tolist()],
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    runner.destroy()
    if line is not None:
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "comparator", "rk4", "toggles", "box"])
    ap.add_argument("--programs", type=int, default=None, help="development only: shrink the population")
    ap.add_argument("--rows", type=int, default=None, help="development only: shrink the dataset")
    ap.add_argument("--banks", type=int, default=1, help="development only (--impl rk4): coefficient sets per system")
    ap.add_argument("--no-cpu", action="store_true", help="development only: skip the CPU baseline and the parity spot check")
    args = ap.parse_args()
    w = dict(WORKLOAD)
    if args.programs:
        w["programs"] = args.programs
        w["name"] += f" (reduced: {args.programs} programs)"
    if args.rows:
        w["rows"] = args.rows
        w["name"] += f" (reduced: {args.rows} rows)"
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        reference_arm(args, w)
    elif args.impl == "comparator":
        comparator_arm(args, w)
    elif args.impl == "rk4":
        rk4_arm(args, w)
    elif args.impl == "toggles":
        toggles_arm(args, w)
    elif args.impl == "box":
        box_arm(args, w)
    else:
        gpu_arm(args, w)


if __name__ == "__main__":
    main()
