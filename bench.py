#!/usr/bin/env python
"""Headline benchmark: BF16 GEMM 8192^3, C = alpha*A*B + beta*C, TFLOP/s on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the GEMM hot path over the whole problem: at N GPUs the 8192^3
problem is split by N-column blocks (B and C sharded, A replicated, no collective in the
timed step), each rank launching its shard through the C ABI of libckl_gemm.so.  Prints ONE
JSON line on rank 0.  For N > 1 run under torchrun (one rank per GPU); a bare
`python bench.py --gpus N` re-launches itself that way.

`value`      device-resident inputs, CUDA events on the launching stream, max over ranks.
`e2e`        the same problem with pinned HOST buffers, copies inside the timed region:
             ckl_gemm_host at N = 1; ckl_gemm_host_sharded at N > 1 (each rank uploads its own
             rows of A and its blocks of B and C, A is all-gathered over NVLink), so the bytes
             crossing the host links do not grow with N.  `e2e.parity` compares the result with
             the device-resident kernel on the same inputs.
`roofline`   tensor-bound: 2*M*N*K FLOP per launch / mean launch duration, against the
             measured cuBLAS BF16 burst rate in MEASURED_PEAKS.json; `sustained_tflops` is the
             same launch back to back for a second, against the sustained cuBLAS figure.
`gathered`   (N > 1) the step that leaves the whole C on every rank (ckl_gemm_gathered), its
             parity on every rank, and the NCCL all-gather form beside it.
`mlp_sharded` (N > 1) BASELINE config 5, weights N-sharded: no-gather and gathered.
`configs`    (N = 1) the other BASELINE configurations, a few launches each, cuBLAS beside.
`cpu_baseline` (N = 1) the reference's own CPU GEMM (oracle/_ref when built, else the
             plain-C port) timed on a bounded row sample of the same problem.

`--impl reference` times only that CPU GEMM, on every host core, as the reference arm.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import socket
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "cuda-kernel-library_b200")

M = N = K = 8192
ALPHA, BETA = 1.0, 0.5
INPUT_SCALE = 0.02
METRIC = "BF16 GEMM TFLOP/s at 8192^3 (C = A*B + 0.5*C, FP32 accumulate, BF16 C)"
DATASHEET_DENSE_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}



def ncu_dram_traffic(algo_name: str, m: int, n: int, k: int):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures
    summarised under profiles/ (profiles/dram_traffic.json, keyed by kernel and shape).  None
    when no capture of the kernel the run launched on this shape is on file: a figure from
    another kernel or shape would be stale."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            table = json.load(f)
        entry = table.get(f"{algo_name}:{m}x{n}x{k}:bf16:beta0.5")
        return int(entry["dram_bytes_read"]) + int(entry["dram_bytes_written"]) if entry else None
    except (OSError, ValueError, KeyError):
        return None


def load_module(name: str, path: str, search=None):
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=search)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_ckl():
    return load_module("ckl_b200", os.path.join(PKG_DIR, "__init__.py"), [PKG_DIR])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured (MEASURED_PEAKS.json, cuBLAS BF16 8192^3 burst)"
    return dict(FALLBACK_PEAKS), "fallback (earlier measurement on this pool)"


# --------------------------------------------------------------------------------------
# clocks: NVML samples while the GPU is under load
# --------------------------------------------------------------------------------------

REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}


class ClockSampler:
    """Reads SM clock, power and clock-event reasons every 10 ms (reads only, sets nothing)."""

    def __init__(self, nv, handle):
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        self.nv, self.handle = nv, handle
        try:
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
        except Exception:  # NVML missing: the JSON line says so
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                util = nv.nvmlDeviceGetUtilizationRates(self.handle).gpu
                watts = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((mhz, int(reasons), util, watts))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [],
                    "note": "NVML unavailable"}
        loaded = [s for s in self.samples if not (s[1] & 0x1)] or self.samples  # drop idle samples
        clocks = sorted(s[0] for s in loaded)
        mask = 0
        for s in loaded:
            mask |= s[1]
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [name for bit, name in REASON_BITS.items() if mask & bit],
                "power_w_max": round(max(s[3] for s in loaded), 1), "samples": len(loaded),
                "window": "warm-up, timed region, a 1 s back-to-back loop of the same launch, the "
                          "gathered and end-to-end steps"}


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU GEMM on a row sample of the problem
# --------------------------------------------------------------------------------------

def cpu_sample_inputs(rows: int):
    import numpy as np
    rng = np.random.default_rng(0x1111 + M)
    a = (rng.standard_normal((rows, K)) * INPUT_SCALE).astype(np.float32)
    b = (rng.standard_normal((K, N)) * INPUT_SCALE).astype(np.float32)
    c = (rng.standard_normal((rows, N)) * INPUT_SCALE).astype(np.float32)
    return a, b, c


def time_cpu_reference(rows_per_thread: int, threads: int, steps: int, warmup: int):
    """Each thread runs the reference's CPU GEMM (ckl::gemm_reference from oracle/_ref when it was
    built, else the plain-C port) on its own block of rows of the 8192^3 problem.  The function
    is single-threaded; ctypes releases the GIL.  Returns (seconds per step, kind, rows)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle  # the checker; only this CPU-baseline leg executes it
    rows = rows_per_thread * threads
    a, b, c = cpu_sample_inputs(rows)
    timer = oracle.RowBlockTimer(b)
    blocks = []
    for t in range(threads):
        sl = slice(t * rows_per_thread, (t + 1) * rows_per_thread)
        blocks.append((np.ascontiguousarray(a[sl]), np.ascontiguousarray(c[sl]),
                       np.empty((rows_per_thread, N), dtype=np.float64)))

    def one_step():
        if threads == 1:
            timer.run(blocks[0][0], blocks[0][1], ALPHA, BETA, blocks[0][2])
            return
        workers = [threading.Thread(target=timer.run, args=(ab, cb, ALPHA, BETA, ob))
                   for ab, cb, ob in blocks]
        for wk in workers:
            wk.start()
        for wk in workers:
            wk.join()

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    sec = (time.perf_counter() - t0) / max(steps, 1)
    timer.close()
    return sec, timer.kind, rows


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows_per_thread = 1
    sec, kind, rows = time_cpu_reference(rows_per_thread, threads, args.steps, args.warmup)
    tflops = 2.0 * rows * N * K / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate over f32 inputs (CPU)", "data": "synthetic",
        "config": workload_config(args.gpus, "cpu"),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": f"{rows} rows of the 8192x8192x8192 problem per step "
                                   f"({rows_per_thread} row per thread, {threads} threads), "
                                   "ckl::gemm_reference of the reference on each row block"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(gpus: int, algo: str) -> dict:
    return {"workload": "bf16_8192_cubed", "m": M, "n": N, "k": K, "alpha": ALPHA, "beta": BETA,
            "a_b_dtype": "bf16", "c_dtype": "bf16", "inputs": "N(0,1)*0.02, seeded, host-generated",
            "layout": "row-major A (MxK), B (KxN), C (MxN)",
            "parallelism": f"N-column blocks over {gpus} GPU(s): B, C sharded, A replicated, "
                           "no collective in the timed step",
            "l2": "inputs larger than L2 (A+B+C per rank >= 160 MB vs 126 MB L2); no flush",
            "algo": algo}


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------

def nvml_handle(torch, local_rank: int):
    """NVML handle of the CUDA device `local_rank` (matched by PCI address, so that a
    CUDA_VISIBLE_DEVICES remapping cannot pair the wrong GPU), or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(local_rank)
        bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
    except Exception:
        return None, None


def bind_near_gpu(nv, handle) -> str:
    """Runs this process on the CPUs next to its GPU, so that the pinned host buffers it
    allocates afterwards (first touch) sit in the memory of the GPU's own socket.  Changes only
    this process's CPU affinity; nothing of the GPU."""
    try:
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(handle, words)
        near = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus = sorted(near & os.sched_getaffinity(0))
        if not cpus:
            return "unchanged (no CPU of the GPU's node is available to this process)"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} CPUs of the GPU's NUMA node"
    except Exception as exc:  # affinity is an optimisation only
        return f"unchanged ({type(exc).__name__})"


def time_launches(torch, fn, launches: int, warm: int = 3) -> float:
    """Mean milliseconds per call of fn over `launches` back-to-back calls (CUDA events on the
    current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches


def sustained_rate(torch, fn, flop: float, seconds: float = 1.0) -> dict:
    """fn back to back for about `seconds` (the power cap engages after roughly 50 launches of
    this size): TFLOP/s over the whole loop, timed with CUDA events."""
    ms, launches = _timed_window(torch, fn, seconds)
    return {"tflops": flop * launches / (ms * 1e-3) / 1e12, "launches": launches, "seconds": ms * 1e-3}


def _timed_window(torch, fn, seconds: float):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    t_end = time.perf_counter() + seconds
    e0.record()
    while time.perf_counter() < t_end:
        for _ in range(20):
            fn()
        launches += 20
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), launches


def sustained_side_by_side(torch, fn_ours, fn_lib, flop: float, windows: int = 4,
                           seconds: float = 0.3) -> dict:
    """The power-capped regime compared fairly: the GPU is first brought under its cap with one
    second of the library's own launches, then windows of `seconds` alternate between the two
    callables, so both are measured in the same thermal and clock state.  TFLOP/s of each over
    its windows."""
    _timed_window(torch, fn_ours, 1.0)
    total = {"ours": [0.0, 0], "lib": [0.0, 0]}
    for _ in range(windows):
        for key, fn in (("ours", fn_ours), ("lib", fn_lib)):
            ms, launches = _timed_window(torch, fn, seconds)
            total[key][0] += ms
            total[key][1] += launches
    rate = {k: flop * v[1] / (v[0] * 1e-3) / 1e12 for k, v in total.items()}
    return {"ours_tflops": rate["ours"], "cublas_tflops": rate["lib"],
            "ratio": rate["ours"] / rate["lib"],
            "protocol": f"1 s of load, then {windows} alternating windows of {seconds} s each"}


BASELINE_CONFIGS = [
    # name, m, n, k, in dtype, alpha, beta (C has the input type): BASELINE.json configs 2, 4, 5
    ("fp16_4096_cubed", 4096, 4096, 4096, "f16", 1.0, 0.0),
    ("fp16_4000x3000x5000", 4000, 3000, 5000, "f16", 1.0, 0.0),
    ("fp16_1024x1024x32768", 1024, 1024, 32768, "f16", 1.0, 0.0),
    ("bf16_mlp_shard_16384x1792x4096", 16384, 1792, 4096, "bf16", 1.0, 0.0),
    ("bf16_mlp_whole_16384x14336x4096", 16384, 14336, 4096, "bf16", 1.0, 0.0),
]


def other_configs(torch, ckl, peak_tflops: float) -> list:
    """The other BASELINE configurations on one GPU: 10 launches each through the C ABI (what
    every caller gets, CKL_ALGO_AUTO) and the same shape through cuBLAS (torch.matmul)."""
    rows = []
    for name, m, n, k, dt, alpha, beta in BASELINE_CONFIGS:
        tdt = torch.float16 if dt == "f16" else torch.bfloat16
        cdt = ckl.F16 if dt == "f16" else ckl.BF16
        g = torch.Generator(device="cuda").manual_seed(0x1111 + m)
        a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(tdt)
        b = (torch.rand(k, n, device="cuda", generator=g) * 2 - 1).to(tdt)
        c = torch.zeros(m, n, device="cuda", dtype=tdt)
        ms = time_launches(torch, lambda: ckl.gemm_ex(cdt, a, b, c, cdt, m, n, k, k, n, n, alpha, beta), 10)
        plan = ckl.last_plan()
        ms_lib = time_launches(torch, lambda: torch.matmul(a, b, out=c), 10)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        rows.append({"name": name, "m": m, "n": n, "k": k, "dtype": dt, "alpha": alpha, "beta": beta,
                     "algo": ckl.algo_name(plan.algo), "ms": ms, "tflops": tf,
                     "frac_of_measured_peak": tf / peak_tflops,
                     "cublas_same_box_tflops": 2.0 * m * n * k / (ms_lib * 1e-3) / 1e12,
                     "launches": 10})
        del a, b, c
    return rows


def compare(torch, got, want) -> dict:
    """How far two device matrices of one type are apart (max abs and relative Frobenius)."""
    g, w = got.float(), want.float()
    diff = (g - w)
    return {"bit_equal": bool(torch.equal(got, want)),
            "max_abs_diff": float(diff.abs().max()),
            "rel_frobenius": float(diff.norm() / w.norm().clamp_min(1e-30)),
            "max_abs_value": float(w.abs().max())}


def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for the product")
    torch.cuda.set_device(local_rank)
    nv, nv_handle = nvml_handle(torch, local_rank)
    affinity = bind_near_gpu(nv, nv_handle) if nv is not None else "unchanged (NVML unavailable)"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    ckl = load_ckl()
    sharded = load_module("ckl_b200_sharded", os.path.join(PKG_DIR, "sharded.py"))
    op = sharded.ShardedGemm(ckl, M, N, K, ckl.BF16, ckl.BF16, world, rank)
    w, col0 = op.shard.width, op.shard.col0
    comm = sharded.make_comm(ckl, world, rank, device="cuda") if world > 1 else None

    def all_max(x: float) -> float:
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- synthetic inputs: generated on the host, rounded to BF16, kept in pinned memory ----
    rng = np.random.default_rng(0x1111 + M)
    def draw(rows, cols):
        return torch.from_numpy((rng.standard_normal((rows, cols)) * INPUT_SCALE)
                                .astype(np.float32)).to(torch.bfloat16)
    a_full = draw(M, K)
    b_full = draw(K, N)
    c_full = draw(M, N)
    hplan = ckl.plan_host_sharded(M, world, rank)
    # end to end, every rank holds only ITS rows of A on the host (all of them at N = 1)
    a_host = a_full[hplan.row0:hplan.row0 + hplan.rows].contiguous().pin_memory()
    b_host = b_full[:, col0:col0 + w].contiguous().pin_memory()
    c_host = c_full[:, col0:col0 + w].contiguous().pin_memory()
    c_in_host = c_host.clone()
    a = a_full.cuda()
    b = b_host.cuda()
    c = c_host.cuda()
    c_in = c.clone()
    stream = torch.cuda.current_stream()

    algos = {ckl.algo_name(i): i for i in range(ckl.NUM_ALGOS)}
    if args.algo not in algos:
        raise SystemExit(f"--algo must be one of {sorted(algos)}")
    algo = algos[args.algo]

    def step():
        op.run(a, b, c, ALPHA, BETA, algo=algo, stream=stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(nv, nv_handle) if rank == 0 else None
    if sampler:
        sampler.start()

    for _ in range(max(args.warmup, 3)):
        step()
    plan = ckl.last_plan()          # what the library really launched for this shape and C type
    # a split schedule is one launch when fused (whole tiles remain for every unit), else two
    launches_per_step = 1 + (1 if plan.sk_tiles > 0 and plan.dp_tiles < plan.units else 0)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_per_step = all_max(e0.elapsed_time(e1)) / args.steps
    ckl.device_status()

    # ---- the same launch back to back for a second: the power-capped regime ------------------
    flop_local = 2.0 * M * w * K
    sustained = sustained_rate(torch, step, flop_local)
    barrier()

    # ---- what this rank's block must hold after ONE step from the seeded C_in ----------------
    c.copy_(c_in)
    step()
    want_block = c.clone()
    torch.cuda.synchronize()

    # ---- gathered variant (N > 1): every rank ends with the whole row-major C ----------------
    gathered = None
    if world > 1 and sharded.even_shards(N, world):
        try:
            gathered = run_gathered(torch, ckl, op, comm, world, a, b, c, c_in, b_full, c_full, col0, w,
                                    step, barrier, all_max, stream, args.steps)
        except Exception as exc:      # keep the headline line; say what went wrong
            gathered = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- end to end through the host-buffer entry point --------------------------------------
    e2e_steps = max(3, min(args.steps, 10))
    if world == 1:
        def host_step():
            ckl.gemm_host(ckl.BF16, a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr(), ckl.BF16,
                          M, w, K, ALPHA, BETA)
        e2e_api = "ckl_gemm_host (pinned host A, B, C; copies inside the timed region)"
    else:
        def host_step():
            op.run_host(comm, a_host, b_host, c_host, ALPHA, BETA)
        e2e_api = ("ckl_gemm_host_sharded (pinned host buffers; each rank uploads its own rows of A "
                   "and its blocks of B and C, A is all-gathered over NVLink; copies and the "
                   "all-gather inside the timed region)")
    for _ in range(2):
        host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_step()
    torch.cuda.synchronize()
    e2e_sec = all_max(time.perf_counter() - t0) / e2e_steps
    h2d = M * K * 2 + K * N * 2 + M * N * 2      # A, B and C each cross the host links once
    d2h = M * N * 2
    # parity, outside the timed region: one call from the seeded C_in against the device path
    c_host.copy_(c_in_host)
    host_step()
    cmp = compare(torch, c_host.cuda(), want_block)
    tol = 2e-2 * math.sqrt(K / 4096.0) * cmp["max_abs_value"]
    e2e_ok = cmp["rel_frobenius"] <= 1e-3 and cmp["max_abs_diff"] <= tol
    e2e_parity = {"ok_on_every_rank": all_max(0.0 if e2e_ok else 1.0) == 0.0,
                  "max_abs_diff": all_max(cmp["max_abs_diff"]),
                  "rel_frobenius": all_max(cmp["rel_frobenius"]),
                  "checked": "the rank's block of C from the host entry point against the "
                             "device-resident kernel on the same inputs"}

    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()

    # ---- BASELINE config 5 (MLP-shaped, weights N-sharded) on N > 1 GPUs ----------------------
    mlp = None
    if world > 1:
        try:
            mlp = run_mlp_sharded(torch, dist, ckl, sharded, comm, world, rank, all_max, barrier)
        except Exception as exc:
            mlp = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- comparator on the same box: cuBLAS through torch.matmul (not the product) ------------
    cublas_tflops = cublas_beta_tflops = cublas_sustained = None
    configs = None
    peaks, peak_src = measured_peaks()
    if rank == 0:
        ref_b = b if world == 1 else b_full.cuda()
        ms = time_launches(torch, lambda: torch.matmul(a, ref_b), args.steps)
        cublas_tflops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        # the same workload (beta 0.5, C read and written in place) through cuBLAS
        c_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda").normal_(std=0.02)
        addmm = lambda: torch.addmm(c_ref, a, ref_b, beta=BETA, alpha=ALPHA, out=c_ref)
        ms = time_launches(torch, addmm, args.steps)
        cublas_beta_tflops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        time.sleep(1.0)
        if world == 1:
            cublas_sustained = sustained_side_by_side(torch, step, addmm, 2.0 * M * N * K)
        del c_ref, ref_b
        if world == 1:
            time.sleep(1.0)
            try:
                configs = other_configs(torch, ckl, float(peaks["bf16_tflops"]))
            except Exception as exc:
                configs = [{"error": f"{type(exc).__name__}: {exc}"}]

    if rank == 0:
        tflops = 2.0 * M * N * K / (ms_per_step * 1e-3) / 1e12
        per_gpu = tflops / world
        peak = float(peaks["bf16_tflops"])
        peak_sustained = float(peaks.get("bf16_tflops_sustained", peak))
        algo_name = ckl.algo_name(plan.algo)
        line = {
            "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, algo_name),
            "roofline": {
                "bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                "frac": per_gpu / peak,
                "traffic": ncu_dram_traffic(algo_name, M, w, K),
                "peak_source": peak_src,
                "flop_per_launch": flop_local,
                "frac_of_datasheet_dense_bf16": per_gpu / DATASHEET_DENSE_BF16_TFLOPS,
                "algorithmic_bytes_per_launch": 2 * (M * K + K * w) + 2 * 2 * M * w,
                "achieved_hbm_gbs": (2 * (M * K + K * w) + 4 * M * w) / (ms_per_step * 1e-3) / 1e9,
                "sustained_tflops": sustained["tflops"],
                "frac_sustained": sustained["tflops"] / peak_sustained,
                "peak_sustained": peak_sustained,
                "sustained_window": f"{sustained['launches']} launches back to back in "
                                    f"{sustained['seconds']:.2f} s on rank 0's GPU",
            },
            "e2e": {"value": 2.0 * M * N * K / e2e_sec / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps, "api": e2e_api,
                    "parity": e2e_parity, "host_affinity": affinity},
            "gpu_launches": args.steps * launches_per_step * world,
            "clocks": clocks,
            "cublas_same_box_tflops": cublas_tflops,
            "cublas_same_box_same_workload_tflops": cublas_beta_tflops,
            "sustained_vs_cublas_same_workload": cublas_sustained,
        }
        if gathered is not None:
            line["gathered"] = gathered
        if mlp is not None:
            line["mlp_sharded"] = mlp
        if configs is not None:
            line["configs"] = configs
        if world == 1:
            sec, kind, rows = time_cpu_reference(16, 1, 1, 0)
            line["cpu_baseline"] = {
                "value": 2.0 * rows * N * K / sec / 1e12, "unit": "TFLOP/s", "cores": 1,
                "kind": kind,
                "sample": f"{rows} of the 8192 rows of C (all 8192 columns, K = 8192), one pass of "
                          "the reference's single-threaded ckl::gemm_reference"}
        emit(line)

    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def run_gathered(torch, ckl, op, comm, world, a, b, c, c_in, b_full, c_full, col0, w, step, barrier,
                 all_max, stream, steps) -> dict:
    """The step that leaves the whole row-major C on every rank: ckl_gemm_gathered timed over
    `steps` steps, its parity on every rank, and the NCCL all-gather form beside it."""
    full_ptr = comm.alloc_shared(M * N * 2)
    def gstep():
        op.gathered(comm, a, b, c, full_ptr, ALPHA, BETA, stream=stream)
    for _ in range(3):
        gstep()
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for _ in range(steps):
        gstep()
    g1.record(stream)
    barrier()
    gms = all_max(g0.elapsed_time(g1)) / steps
    # parity, outside the timed region: one step from the seeded C_in; every rank checks the
    # WHOLE assembled C against the unsharded kernel run here on the full B and C_in
    c.copy_(c_in)
    gstep()
    got_full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ckl.stream_copy(got_full, full_ptr, M * N * 2, stream)
    ref_full = c_full.cuda()
    b_dev_full = b_full.cuda()
    ckl.gemm_ex(ckl.BF16, a, b_dev_full, ref_full, ckl.BF16, M, N, K, K, N, N, ALPHA, BETA, 0, stream)
    torch.cuda.synchronize()
    cmp = compare(torch, got_full, ref_full)
    own_ok = torch.equal(got_full[:, col0:col0 + w], c)
    tol = 2e-2 * math.sqrt(K / 4096.0) * cmp["max_abs_value"]
    ok = own_ok and cmp["rel_frobenius"] <= 1e-3 and cmp["max_abs_diff"] <= tol
    parity = {"ok_on_every_rank": all_max(0.0 if ok else 1.0) == 0.0,
              "max_abs_diff": all_max(cmp["max_abs_diff"]),
              "rel_frobenius": all_max(cmp["rel_frobenius"]),
              "bit_equal_on_every_rank": all_max(0.0 if cmp["bit_equal"] else 1.0) == 0.0,
              "checked": "whole C on every rank against the unsharded kernel on the same inputs "
                         "(rel. Frobenius <= 1e-3, max error <= 2e-2*sqrt(K/4096)*max|C|); the "
                         "rank's own block bit for bit against its local c_shard"}
    del got_full, ref_full, b_dev_full
    gathered = {"value": 2.0 * M * N * K / (gms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": gms, "parity": parity,
                "note": "ckl_gemm_gathered: GEMM in row panels, each panel's column block "
                        "written into every rank's C by this library's copy kernel (plain "
                        "peer stores over NVLink) while the next panel multiplies"}
    comm.free_shared(full_ptr)
    # the same through NCCL: GEMM, all_gather_into_tensor, interleave kernel, one after another
    staging = torch.empty(world, M, w, dtype=torch.bfloat16, device="cuda")
    full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    def nstep():
        step()
        op.gather(c, staging, full, stream=stream)
    for _ in range(3):
        nstep()
    barrier()
    g0.record(stream)
    for _ in range(steps):
        nstep()
    g1.record(stream)
    barrier()
    nms = all_max(g0.elapsed_time(g1)) / steps
    gathered["nccl_all_gather_variant"] = {
        "value": 2.0 * M * N * K / (nms * 1e-3) / 1e12, "ms_per_step": nms,
        "note": "GEMM + NCCL all-gather of the C column blocks + interleave kernel"}
    return gathered


def run_mlp_sharded(torch, dist, ckl, sharded, comm, world, rank, all_max, barrier) -> dict:
    """BASELINE config 5 on `world` GPUs: M = 16384 tokens, K = 4096, N = 14336, activations
    N(0,1), weights N(0,1)/64, BF16 C, beta 0; weights and C sharded by columns, A replicated.
    Reports the no-gather step and the gathered one (whole C on every rank)."""
    m, n, k = 16384, 14336, 4096
    op = sharded.ShardedGemm(ckl, m, n, k, ckl.BF16, ckl.BF16, world, rank)
    w, col0 = op.shard.width, op.shard.col0
    g = torch.Generator(device="cuda").manual_seed(0x2222 + n)      # same stream on every rank
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b_full = (torch.randn(k, n, device="cuda", generator=g) / 64.0).to(torch.bfloat16)
    b = b_full[:, col0:col0 + w].contiguous()
    c = torch.zeros(m, w, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream()
    launches = 10
    step = lambda: op.run(a, b, c, 1.0, 0.0, stream=stream)
    for _ in range(3):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(launches):
        step()
    e1.record(stream)
    barrier()
    ms = all_max(e0.elapsed_time(e1)) / launches
    out = {"workload": "bf16_mlp_16384x14336x4096", "shard_width": w, "launches": launches,
           "algo": ckl.algo_name(ckl.last_plan().algo),
           "no_gather": {"ms_per_step": ms, "value": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
                         "unit": "TFLOP/s"}}
    if sharded.even_shards(n, world):
        full_ptr = comm.alloc_shared(m * n * 2)
        gstep = lambda: op.gathered(comm, a, b, c, full_ptr, 1.0, 0.0, stream=stream)
        for _ in range(2):
            gstep()
        barrier()
        e0.record(stream)
        for _ in range(launches):
            gstep()
        e1.record(stream)
        barrier()
        gms = all_max(e0.elapsed_time(e1)) / launches
        # parity: the neighbour's block of the assembled C against that block recomputed here
        nb = (rank + 1) % world
        ncol0, nw = ckl.column_shard(n, world, nb)
        got = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ckl.stream_copy(got, full_ptr, m * n * 2, stream)
        ref = torch.zeros(m, nw, device="cuda", dtype=torch.bfloat16)
        ckl.gemm_ex(ckl.BF16, a, b_full[:, ncol0:ncol0 + nw].contiguous(), ref, ckl.BF16, m, nw, k, k, nw, nw,
                    1.0, 0.0, 0, stream)
        torch.cuda.synchronize()
        cmp = compare(torch, got[:, ncol0:ncol0 + nw], ref)
        tol = 2e-2 * math.sqrt(k / 4096.0) * cmp["max_abs_value"]
        ok = torch.equal(got[:, col0:col0 + w], c) and cmp["rel_frobenius"] <= 1e-3 and \
            cmp["max_abs_diff"] <= tol
        out["gathered"] = {"ms_per_step": gms, "value": 2.0 * m * n * k / (gms * 1e-3) / 1e12,
                           "unit": "TFLOP/s",
                           "parity_ok_on_every_rank": all_max(0.0 if ok else 1.0) == 0.0,
                           "neighbour_block_rel_frobenius": all_max(cmp["rel_frobenius"]),
                           "neighbour_block_max_abs_diff": all_max(cmp["max_abs_diff"]),
                           "checked": "own block of the assembled C bit for bit against the local "
                                      "c_shard; the next rank's block against the same GEMM run here "
                                      "in one piece (rel. Frobenius <= 1e-3, max error <= "
                                      "2e-2*sqrt(K/4096)*max|C|; the row panels of the gathered form "
                                      "may split k differently, so the last bits can differ)"}
        del got, ref
        comm.free_shared(full_ptr)
    return out


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


_RESULT_FD = None


def keep_stdout_for_the_result() -> None:
    """The contract is ONE JSON line on stdout.  Libraries may write there too (NCCL prints its
    version line to stdout when NCCL_DEBUG is set in the environment), so file descriptor 1 is
    pointed at stderr for the whole run and the result goes to a saved copy of the original."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--algo", default="auto",
                    help="pin a kernel (auto, simt, umma_1cta, umma_1cta_streamk, umma_2cta, "
                         "umma_2cta_streamk, umma_2cta_wide, umma_2cta_wide_streamk); the default "
                         "is what every caller gets")
    args = ap.parse_args()
    if args.gpus <= 1 or "WORLD_SIZE" in os.environ:
        keep_stdout_for_the_result()   # (the torchrun re-launch below passes its child's stdout through)
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
               str(free_port()), os.path.abspath(__file__), "--gpus", str(args.gpus), "--steps",
               str(args.steps), "--warmup", str(args.warmup), "--algo", args.algo]
        raise SystemExit(subprocess.call(cmd))
    run_ours(args)


if __name__ == "__main__":
    main()
