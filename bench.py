#!/usr/bin/env python
"""Headline benchmark: BF16 GEMM 8192^3, C = alpha*A*B + beta*C, TFLOP/s on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the GEMM hot path over the whole problem: at N GPUs the 8192^3
problem is split by N-column blocks (B and C sharded, A replicated, no collective in the
timed step), each rank launching its shard through the C ABI of libckl_gemm.so.  Prints ONE
JSON line on rank 0.  For N > 1 run under torchrun (one rank per GPU); a bare
`python bench.py --gpus N` re-launches itself that way.

`value`      device-resident inputs, CUDA events on the launching stream, max over ranks.
`e2e`        the same problem through ckl_gemm_host with pinned HOST buffers: H2D of A, B,
             C, the GEMM, D2H of C, all inside the timed region.
`roofline`   tensor-bound: 2*M*N*K FLOP per launch / mean launch duration, against the
             measured cuBLAS BF16 burst rate in MEASURED_PEAKS.json.
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

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the
# ncu capture summarised in profiles/umma_gemm_kernel_pairwide_bf16_8192_cubed.md (1 GPU, whole problem).
NCU_DRAM_TRAFFIC_BYTES = {"bf16_8192_cubed": 1_233_121_168}  # 1.112922 GB read + 0.120199 GB written


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

    def __init__(self, device_index: int):
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
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
                "window": "warm-up + timed region + a 1 s back-to-back loop of the same launch"}


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
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    ckl = load_ckl()
    sharded = load_module("ckl_b200_sharded", os.path.join(PKG_DIR, "sharded.py"))
    op = sharded.ShardedGemm(ckl, M, N, K, ckl.BF16, ckl.BF16, world, rank)
    w, col0 = op.shard.width, op.shard.col0

    # ---- synthetic inputs: generated on the host, rounded to BF16, kept in pinned memory ----
    rng = np.random.default_rng(0x1111 + M)
    def draw(rows, cols):
        return torch.from_numpy((rng.standard_normal((rows, cols)) * INPUT_SCALE)
                                .astype(np.float32)).to(torch.bfloat16)
    a_host = draw(M, K).pin_memory()
    b_full = draw(K, N)
    c_full = draw(M, N)
    b_host = b_full[:, col0:col0 + w].contiguous().pin_memory()
    c_host = c_full[:, col0:col0 + w].contiguous().pin_memory()
    del b_full, c_full
    a = a_host.cuda()
    b = b_host.cuda()
    c = c_host.cuda()
    stream = torch.cuda.current_stream()

    algos = {ckl.algo_name(i): i for i in range(ckl.NUM_ALGOS)}
    if args.algo not in algos:
        raise SystemExit(f"--algo must be one of {sorted(algos)}")
    algo = algos[args.algo]

    plan = ckl.plan_gemm(M, w, K, K, w, w, algo=algos.get(args.algo, 0),
                         sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
    launches_per_step = 1 + (1 if plan.sk_tiles > 0 else 0)

    def step():
        op.run(a, b, c, ALPHA, BETA, algo=algo, stream=stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_total = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_per_step = ms_total.item() / args.steps
    ckl.device_status()

    # ---- gathered variant (N > 1): same step followed by the all-gather and the interleave ----
    gathered = None
    if world > 1 and sharded.even_shards(N, world):
        staging = torch.empty(world, M, w, dtype=torch.bfloat16, device="cuda")
        full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        def gstep():
            step()
            op.gather(c, staging, full, stream=stream)
        for _ in range(3):
            gstep()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(args.steps):
            gstep()
        g1.record(stream)
        barrier()
        gms = torch.tensor([g0.elapsed_time(g1)], device="cuda", dtype=torch.float64)
        dist.all_reduce(gms, op=dist.ReduceOp.MAX)
        gms = gms.item() / args.steps
        gathered = {"value": 2.0 * M * N * K / (gms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": gms,
                    "note": "GEMM + NCCL all-gather of the C column blocks + interleave kernel"}
        del staging, full

    # ---- end to end through the host-buffer entry point --------------------------------------
    e2e_steps = max(3, min(args.steps, 10))
    def host_step():
        ckl.gemm_host(ckl.BF16, a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr(), ckl.BF16,
                      M, w, K, ALPHA, BETA)
    for _ in range(2):
        host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_step()
    torch.cuda.synchronize()
    e2e_sec = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_sec, op=dist.ReduceOp.MAX)
    e2e_sec = e2e_sec.item() / e2e_steps
    h2d = world * M * K * 2 + K * N * 2 + M * N * 2      # A on every rank, B and C shards
    d2h = M * N * 2

    # ---- a short sustained loop so the clock samples are taken under load ---------------------
    if sampler:
        t_end = time.perf_counter() + 1.0
        while time.perf_counter() < t_end:
            for _ in range(20):
                step()
            torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()

    # ---- comparator on the same box: cuBLAS through torch.matmul (not the product) ------------
    cublas_tflops = None
    cublas_beta_tflops = None
    if rank == 0:
        ref_b = b if world == 1 else torch.empty(K, N, dtype=torch.bfloat16, device="cuda").normal_()
        for _ in range(3):
            torch.matmul(a, ref_b)
        torch.cuda.synchronize()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            torch.matmul(a, ref_b)
        r1.record()
        torch.cuda.synchronize()
        cublas_tflops = 2.0 * M * N * K / (r0.elapsed_time(r1) / args.steps * 1e-3) / 1e12
        # the same workload (beta 0.5, C read and written in place) through cuBLAS
        c_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda").normal_(std=0.02)
        for _ in range(3):
            torch.addmm(c_ref, a, ref_b, beta=BETA, alpha=ALPHA, out=c_ref)
        torch.cuda.synchronize()
        r0.record()
        for _ in range(args.steps):
            torch.addmm(c_ref, a, ref_b, beta=BETA, alpha=ALPHA, out=c_ref)
        r1.record()
        torch.cuda.synchronize()
        cublas_beta_tflops = 2.0 * M * N * K / (r0.elapsed_time(r1) / args.steps * 1e-3) / 1e12
        del c_ref

    if rank == 0:
        peaks, peak_src = measured_peaks()
        tflops = 2.0 * M * N * K / (ms_per_step * 1e-3) / 1e12
        per_gpu = tflops / world
        peak = float(peaks["bf16_tflops"])
        line = {
            "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, ckl.algo_name(plan.algo)),
            "roofline": {
                "bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                "frac": per_gpu / peak,
                "traffic": NCU_DRAM_TRAFFIC_BYTES["bf16_8192_cubed"] if world == 1 else None,
                "peak_source": peak_src,
                "flop_per_launch": 2.0 * M * w * K,
                "frac_of_datasheet_dense_bf16": per_gpu / DATASHEET_DENSE_BF16_TFLOPS,
                "algorithmic_bytes_per_launch": 2 * (M * K + K * w) + 2 * 2 * M * w,
                "achieved_hbm_gbs": (2 * (M * K + K * w) + 4 * M * w) / (ms_per_step * 1e-3) / 1e9,
            },
            "e2e": {"value": 2.0 * M * N * K / e2e_sec / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps,
                    "api": "ckl_gemm_host (pinned host A, B, C; copies inside the timed region)"},
            "gpu_launches": args.steps * launches_per_step * world,
            "clocks": clocks,
            "cublas_same_box_tflops": cublas_tflops,
            "cublas_same_box_same_workload_tflops": cublas_beta_tflops,
        }
        if gathered is not None:
            line["gathered"] = gathered
        if world == 1:
            sec, kind, rows = time_cpu_reference(16, 1, 1, 0)
            line["cpu_baseline"] = {
                "value": 2.0 * rows * N * K / sec / 1e12, "unit": "TFLOP/s", "cores": 1,
                "kind": kind,
                "sample": f"{rows} of the 8192 rows of C (all 8192 columns, K = 8192), one pass of "
                          "the reference's single-threaded ckl::gemm_reference"}
        emit(line)

    if world > 1:
        dist.destroy_process_group()


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
