"""One Nsight Compute diagnostic round over a list of kernel variants and sizes.

Counterpart of the reference's benchmarks/run_ncu_round.sh:40-81: for every "variant:size"
pair, profile one settled launch of that kernel with a curated set of sections and keep the
report, a readable detail page and a record of the commit, toolkit and driver.

    python cuda-kernel-library_b200/ncu_round.py <round_name> <variant:size[:kernel]> [...]
    e.g.  ncu_round.py wide_vs_pair umma_2cta_wide:8192 umma_2cta:8192 umma_1cta:4096
          ncu_round.py shard umma_2cta_wide:8192x1024x8192 --beta 0.5
          ncu_round.py fixup umma_1cta_streamk:1024x1024x32768:streamk_fixup_kernel

`size` is one number (a cube) or MxNxK; `kernel` overrides the kernel-name filter (default:
umma_gemm_kernel; sgemm_kernel, simt_gemm_kernel and trsm_diag_block_kernel for the variants
sgemm, simt and trsm; the variant helpers captures one launch of each memory-bound helper
kernel).

Output: <out>/<round_name>/<variant>_<size>.ncu-rep, the matching .txt (details page) and
round_meta.txt; <out> defaults to ./ncu_rounds (--out to change).

Differences from the reference script, all deliberate:
  * every ncu call carries --clock-control none, so the GPU's clocks are never locked;
  * each configuration is first run once WITHOUT ncu and is only profiled if that run exits 0;
  * the kernel filter is this library's one tensor-core kernel (umma_gemm_kernel) or, for the
    variant "sgemm", the FP32 kernel (sgemm_kernel);
  * split (stream-K) schedules run in their two-kernel form (CKL_STREAMK_FIXUP=pass is set for
    the child processes): the fused form launches cooperatively, and under the profiler's
    kernel replay that launch failed;
  * one launch is captured after two warm ones, with the same curated sections as the
    reference (SpeedOfLight, Occupancy, MemoryWorkloadAnalysis, WarpStateStats,
    SchedulerStats, LaunchStats, ComputeWorkloadAnalysis): a handful of passes, not --set full.
Times printed by a run under ncu are not benchmark figures.
"""

from __future__ import annotations

import argparse
import datetime
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DRIVER = os.path.join(HERE, "ncu_driver.py")
SECTIONS = ["SpeedOfLight", "Occupancy", "MemoryWorkloadAnalysis", "WarpStateStats",
            "SchedulerStats", "LaunchStats", "ComputeWorkloadAnalysis"]


def tool_output(cmd: list[str]) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, check=True).stdout.strip()
    except Exception:
        return "unknown"


DEFAULT_KERNEL = {"sgemm": "sgemm_kernel", "simt": "simt_gemm_kernel", "trsm": "trsm_diag_block_kernel",
                  "helpers": "bias_relu|scale_c_kernel|assemble_column_blocks_kernel|"
                             "scatter_column_block_kernel|copy_rows_kernel|stream_copy_kernel"}
# launches captured per configuration (after two skipped): the helpers variant wants one of each
LAUNCH_COUNT = {"helpers": 6}


def parse_pair(pair: str) -> tuple[str, tuple[int, int, int], str]:
    """"variant:size[:kernel]" -> (variant, (m, n, k), kernel-name filter)."""
    fields = pair.split(":")
    if len(fields) not in (2, 3) or not fields[0]:
        raise ValueError(f"expected variant:size[:kernel], got {pair!r}")
    dims = [int(x) for x in fields[1].lower().split("x")]
    if len(dims) == 1:
        dims = dims * 3
    if len(dims) != 3 or min(dims) <= 0:
        raise ValueError(f"size must be N or MxNxK with positive numbers, got {fields[1]!r}")
    kernel = fields[2] if len(fields) == 3 else DEFAULT_KERNEL.get(fields[0], "umma_gemm_kernel")
    return fields[0], (dims[0], dims[1], dims[2]), kernel


def driver_command(variant: str, shape: tuple[int, int, int], dtype: str, beta: float) -> list[str]:
    m, n, k = shape
    return [sys.executable, DRIVER, "--m", str(m), "--n", str(n), "--k", str(k), "--in", dtype,
            "--out", dtype, "--beta", str(beta), "--algo", variant, "--iters", "3"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("round")
    ap.add_argument("pairs", nargs="+", metavar="variant:size")
    ap.add_argument("--out", default="ncu_rounds")
    ap.add_argument("--dtype", choices=["f16", "bf16"], default="bf16")
    ap.add_argument("--beta", type=float, default=0.0)
    ap.add_argument("--ncu", default="ncu")
    args = ap.parse_args()

    out_dir = os.path.join(args.out, args.round)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "round_meta.txt"), "w") as f:
        f.write(f"round: {args.round}\n")
        f.write(f"date: {datetime.datetime.now().astimezone().isoformat(timespec='seconds')}\n")
        f.write(f"commit: {tool_output(['git', '-C', ROOT, 'rev-parse', 'HEAD'])}\n")
        nvcc = tool_output(["nvcc", "--version"]).splitlines()
        f.write(f"nvcc: {nvcc[-1] if nvcc else 'unknown'}\n")
        f.write("driver: " + tool_output(["nvidia-smi", "--query-gpu=driver_version",
                                          "--format=csv,noheader"]) + "\n")

    failures = 0
    for pair in args.pairs:
        variant, shape, kernel = parse_pair(pair)
        size = str(shape[0]) if shape[0] == shape[1] == shape[2] else "x".join(map(str, shape))
        base = os.path.join(out_dir, f"{variant}_{size}" +
                            ("" if kernel in ("umma_gemm_kernel", DEFAULT_KERNEL.get(variant)) else f"_{kernel}"))
        cmd = driver_command(variant, shape, args.dtype, args.beta)
        # Split schedules are profiled in their two-kernel form: under the profiler's kernel
        # replay the cooperative launch of the fused form ended with a launch failure reported
        # by the driver, while the same command passes on its own.
        os.environ["CKL_STREAMK_FIXUP"] = "pass"
        print(f"profiling {variant} at {size} (kernel {kernel})", flush=True)
        plain = subprocess.run(cmd, capture_output=True, text=True)
        if plain.returncode != 0:
            print(f"  not profiled: the plain run exited {plain.returncode}\n{plain.stderr[-800:]}")
            failures += 1
            continue
        ncu = [args.ncu, "--clock-control", "none"]
        for section in SECTIONS:
            ncu += ["--section", section]
        # skip the two warm launches of the driver; trsm launches several diagonal-block kernels
        # per solve, any settled one serves
        skip = "6" if variant == "helpers" else "2"      # one whole warm round of the six helpers
        ncu += ["--kernel-name", f"regex:{kernel}", "--launch-skip", skip, "--launch-count",
                str(LAUNCH_COUNT.get(variant, 1)),
                "--force-overwrite", "--export", base, *cmd]
        run = subprocess.run(ncu, capture_output=True, text=True)
        if run.returncode != 0:
            print(f"  ncu exited {run.returncode}\n{run.stdout[-800:]}{run.stderr[-800:]}")
            failures += 1
            continue
        details = subprocess.run([args.ncu, "--import", base + ".ncu-rep", "--page", "details"],
                                 capture_output=True, text=True)
        with open(base + ".txt", "w") as f:
            f.write(details.stdout)
        print(f"  wrote {base}.ncu-rep and {base}.txt")
    return 1 if failures else 0


if __name__ == "__main__":
    raise SystemExit(main())
