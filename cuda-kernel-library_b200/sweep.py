"""Resumable benchmark sweep: run a matrix of GEMM configurations, one process each, and keep
the rows.

Counterpart of the reference's benchmarks/sweep.py:36-184.  Each configuration is one run of
`build/bench_all gemm <variant> <dtype> <m> <n> <k> <commit>` (a separate process, so a fault in
one configuration cannot take the sweep down); its JSON row is appended to `sweep.jsonl`, and
`summary.csv` is rewritten from all rows.  A configuration whose key
(family, variant, dtype, m, n, k, gpus, commit) is already in the file is skipped unless
`--force` is given, so an interrupted sweep continues where it stopped.

    python cuda-kernel-library_b200/sweep.py --out sweep_results [--quick] [--force] [--gpus 2,4,8]

The matrix holds the reference's square sizes and the benchmark configurations of this
library's headline path (4096^3, 8192^3, the two stream-K stress shapes, one tensor-parallel
MLP shard).  With --gpus it also holds, for every listed GPU count the machine has, the
N-sharded form of the two multi-GPU configurations (8192^3 and the MLP-shaped GEMM), each
run as one torchrun job of sharded_row.py.

Beside the reference's columns every row carries `pct_peak_measured` (against the measured
cuBLAS BF16 burst rate of this pool's GPUs in MEASURED_PEAKS.json at the repository root, when
that file exists; 16-bit rows only) and the CPU baseline of the same run: `cpu_baseline_gflops`
is the reference's single-threaded CPU GEMM (ckl/reference.hpp) timed once per sweep on
512^3 on this host (`bench_all cpu reference fp32 512 512 512`), `cpu_cores` the threads it
used (1).
"""

from __future__ import annotations

import argparse
import csv
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BENCH_ALL = os.path.join(HERE, "build", "bench_all")

SQUARE = [512, 1024, 2048, 4096, 8192]                      # benchmarks/sweep.py:47-50 there
SHAPES = [(4000, 3000, 5000), (1024, 1024, 32768), (16384, 1792, 4096)]
VARIANTS = ["auto", "umma_1cta", "umma_2cta", "umma_2cta_wide", "umma_1cta_streamk"]
DTYPES = ["fp16", "bf16", "bf16_c16"]
FIELDS = ["family", "variant", "dtype", "m", "n", "k", "gpus", "median_ms", "iqr_ms", "gflops",
          "tflops", "pct_peak_datasheet", "pct_peak_measured", "baseline_gflops", "pct_baseline",
          "cpu_baseline_gflops", "cpu_cores", "median_sm_clock_mhz", "max_temp_c", "max_power_w",
          "throttled", "power_capped", "commit"]
MULTI_GPU_SHAPES = [("bf16_c16", 8192, 8192, 8192), ("bf16_c16", 16384, 14336, 4096)]
SHARDED_ROW = os.path.join(HERE, "sharded_row.py")


FP32_SIZES = [512, 1024, 2048, 4096]                        # benchmarks/sweep.py:38 there
TRSM_SIZES = [512, 1024, 2048]                              # benchmarks/sweep.py:42,66-68 there


def matrix(quick: bool, gpu_counts=()):
    for cfg in single_gpu_matrix(quick):
        yield cfg
    for gpus in gpu_counts:
        for dtype, m, n, k in (MULTI_GPU_SHAPES[:1] if quick else MULTI_GPU_SHAPES):
            yield {"family": "gemm", "variant": "auto", "dtype": dtype, "m": m, "n": n, "k": k,
                   "gpus": gpus}


def single_gpu_matrix(quick: bool):
    sizes = [(s, s, s) for s in (SQUARE[:3] if quick else SQUARE)]
    shapes = sizes + ([] if quick else SHAPES)
    for variant in (VARIANTS[:2] if quick else VARIANTS):
        for dtype in (DTYPES[:1] if quick else DTYPES):
            for m, n, k in shapes:
                yield {"family": "gemm", "variant": variant, "dtype": dtype, "m": m, "n": n, "k": k,
                       "gpus": 1}
    for s in (FP32_SIZES[1:3] if quick else FP32_SIZES):
        yield {"family": "gemm", "variant": "sgemm", "dtype": "fp32", "m": s, "n": s, "k": s, "gpus": 1}
    for s in (TRSM_SIZES[1:2] if quick else TRSM_SIZES):
        yield {"family": "trsm", "variant": "blocked", "dtype": "fp32", "m": s, "n": 256, "k": 0,
               "gpus": 1}


def key_of(row: dict) -> tuple:
    return tuple(row.get(f) for f in ("family", "variant", "dtype", "m", "n", "k", "gpus", "commit"))


def load_rows(path: str) -> list[dict]:
    rows = []
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    rows.append(json.loads(line))
    return rows


def write_summary(rows: list[dict], path: str) -> None:
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=FIELDS, extrasaction="ignore")
        w.writeheader()
        for row in sorted(rows, key=lambda r: (r["variant"], r["dtype"], r["m"], r["n"], r["k"])):
            w.writerow(row)


def current_commit() -> str:
    try:
        return subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], check=True,
                              capture_output=True, text=True).stdout.strip()
    except Exception:
        return "unknown"


def measured_peak_tflops() -> float | None:
    """Measured cuBLAS BF16 burst rate of this pool's GPUs, when the file is there."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except (OSError, ValueError, KeyError):
        return None


def cpu_baseline(commit: str, runner=None) -> dict:
    """The reference's CPU GEMM timed once on this host (512^3, one thread)."""
    cmd = [BENCH_ALL, "cpu", "reference", "fp32", "512", "512", "512", commit]
    try:
        proc = (runner or subprocess.run)(cmd, capture_output=True, text=True, timeout=600,
                                          env=dict(os.environ, CKL_REPO_ROOT=ROOT))
        row = json.loads(proc.stdout.strip().splitlines()[-1]) if proc.returncode == 0 else {}
    except Exception:
        row = {}
    return {"cpu_baseline_gflops": row.get("gflops", ""), "cpu_cores": row.get("cpu_cores", "")}


def run_one(cfg: dict, commit: str, runner=None) -> dict | None:
    """Runs one configuration in its own process; returns the parsed row or None."""
    if cfg.get("gpus", 1) > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={cfg['gpus']}", "--master-addr", "127.0.0.1", "--master-port",
               str(29700 + cfg["gpus"]), SHARDED_ROW, cfg["variant"], cfg["dtype"], str(cfg["m"]),
               str(cfg["n"]), str(cfg["k"]), commit]
    else:
        cmd = [BENCH_ALL, cfg["family"], cfg["variant"], cfg["dtype"], str(cfg["m"]), str(cfg["n"]),
               str(cfg["k"]), commit]
    env = dict(os.environ, CKL_REPO_ROOT=ROOT)
    proc = (runner or subprocess.run)(cmd, capture_output=True, text=True, env=env, timeout=600)
    if proc.returncode != 0:
        sys.stderr.write(f"[sweep] {' '.join(cmd[1:])} failed ({proc.returncode}): "
                         f"{proc.stderr.strip()[-300:]}\n")
        return None
    return json.loads(proc.stdout.strip().splitlines()[-1])


def sweep(out_dir: str, quick: bool = False, force: bool = False, commit: str | None = None,
          runner=None, gpu_counts=()) -> tuple[int, int]:
    """Returns (configurations run, configurations skipped as already done)."""
    os.makedirs(out_dir, exist_ok=True)
    jsonl = os.path.join(out_dir, "sweep.jsonl")
    commit = commit or current_commit()
    rows = load_rows(jsonl)
    done = {key_of(r) for r in rows}
    ran = skipped = 0
    peak = measured_peak_tflops()
    cpu = None
    for cfg in matrix(quick, gpu_counts):
        if not force and key_of(dict(cfg, commit=commit)) in done:
            skipped += 1
            continue
        row = run_one(cfg, commit, runner)
        if row is None:
            continue
        if cpu is None:
            cpu = cpu_baseline(commit, runner)      # once per sweep, beside the first GPU row
        row.update(cpu)
        sixteen_bit = row.get("dtype", "").startswith(("fp16", "bf16"))
        row["pct_peak_measured"] = (round(100.0 * row["tflops"] / (peak * max(row.get("gpus", 1), 1)), 2)
                                    if peak and sixteen_bit and "tflops" in row else "")
        rows.append(row)
        done.add(key_of(row))
        with open(jsonl, "a") as f:
            f.write(json.dumps(row) + "\n")
        write_summary(rows, os.path.join(out_dir, "summary.csv"))
        ran += 1
    write_summary(rows, os.path.join(out_dir, "summary.csv"))
    return ran, skipped


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "sweep_results"))
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--gpus", default="", help="comma-separated GPU counts above 1 for the N-sharded rows, "
                                               "e.g. 2,4,8 (counts the machine lacks are left out)")
    args = ap.parse_args()
    if not os.path.exists(BENCH_ALL):
        raise SystemExit(f"{BENCH_ALL} is missing: run `make -C {os.path.join(HERE, 'tools')}`")
    counts = [int(x) for x in args.gpus.split(",") if x.strip()]
    if counts:
        import torch
        counts = [c for c in counts if 1 < c <= torch.cuda.device_count()]
    ran, skipped = sweep(args.out, args.quick, args.force, gpu_counts=counts)
    print(f"[sweep] ran {ran}, skipped {skipped} already present; results in {args.out}")


if __name__ == "__main__":
    main()
