"""In-kernel timers of the tensor-core GEMM (instrumented build, not a benchmark).

    python cuda-kernel-library_b200/build.py --timers          # libckl_gemm_timers.so, -DCKL_TIMERS
    python cuda-kernel-library_b200/kernel_timers.py epilogue  # cycles per epilogue phase and tile
    python cuda-kernel-library_b200/kernel_timers.py timeline  # wall-clock timeline of a stream-K launch

`epilogue`: per 8192^3 BF16 launch and kernel (256x512 and 256x256 pair tiles, beta 0.5 and 0),
the MMA thread's wait for a drained accumulator and the time epilogue warp 0 spends in each
phase of its chunk loop, in SM cycles per tile.  `timeline`: for a split (stream-K) and an
unsplit launch, when the CTAs' last MMA and last store happen, in microseconds from the first
CTA's start, and the time spent waiting for other CTAs' partials.

The counters perturb the kernel (clock reads in the epilogue loop), so the throughput printed
beside them is for orientation only.
"""

from __future__ import annotations

import ctypes
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libckl_gemm_timers.so")
BF16 = 2
ALGO_2CTA, ALGO_2CTA_SK, ALGO_2CTA_WIDE = 4, 5, 6


def load(timer_mode: int):
    if not os.path.exists(LIB):
        raise SystemExit(f"{LIB} is missing: python cuda-kernel-library_b200/build.py --timers")
    os.environ["CKL_TIMER_MODE"] = str(timer_mode)
    lib = ctypes.CDLL(LIB)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ckl_gemm_ex.argtypes = [i, vp, vp, vp, i, i, i, i, i, i, i, f, f, i, vp]
    lib.ckl_read_timers.argtypes = [vp, i]
    return lib


def operands(m, n, k):
    a = (torch.randn(m, k, device="cuda") * 0.02).bfloat16()
    b = (torch.randn(k, n, device="cuda") * 0.02).bfloat16()
    c = (torch.randn(m, n, device="cuda") * 0.02).bfloat16()
    return a, b, c


def launch(lib, a, b, c, m, n, k, beta, algo):
    rc = lib.ckl_gemm_ex(BF16, a.data_ptr(), b.data_ptr(), c.data_ptr(), BF16, m, n, k, k, n, n, 1.0,
                         beta, algo, None)
    if rc != 0:
        raise SystemExit(f"ckl_gemm_ex returned {rc}")


def timed(lib, a, b, c, m, n, k, beta, algo, warm=5):
    for _ in range(warm):
        launch(lib, a, b, c, m, n, k, beta, algo)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch(lib, a, b, c, m, n, k, beta, algo)
    e1.record()
    torch.cuda.synchronize()
    out = np.zeros((148, 8), dtype=np.uint64)
    lib.ckl_read_timers(out.ctypes.data_as(ctypes.c_void_p), 148)
    return e0.elapsed_time(e1), out


def epilogue() -> None:
    lib = load(0)
    m = n = k = 8192
    a, b, c = operands(m, n, k)
    for algo, name, k_blocks in [(ALGO_2CTA_WIDE, "pair 256x512", 128), (ALGO_2CTA, "pair 256x256", 64)]:
        for beta in (0.5, 0.0):
            ms, t = timed(lib, a, b, c, m, n, k, beta, algo)
            rows = t[t[:, 0] > 0]            # leader CTAs: the MMA thread wrote slot 0
            tiles = rows[:, 6].astype(float) / k_blocks
            per_tile = lambda col: round(float((rows[:, col] / tiles).mean()))
            print(json.dumps({
                "kernel": name, "beta": beta, "ms": round(ms, 4), "tflops": round(2 * m * n * k / ms / 1e9),
                "cycles_per_tile": per_tile(0), "mma_wait_for_drained_accumulator": per_tile(5),
                "tmem_load_and_release": per_tile(1), "wait_for_c_in": per_tile(2),
                "wait_for_store_and_issue_c_in": per_tile(3), "arithmetic_and_shared_stores": per_tile(4),
                "fence_and_store_issue": per_tile(7)}), flush=True)


def timeline() -> None:
    lib = load(1)
    for m, n, k in [(4096, 4096, 4096), (8192, 4096, 8192)]:
        a, b, c = operands(m, n, k)
        for algo, name in [(ALGO_2CTA, "whole tiles"), (ALGO_2CTA_SK, "stream-K")]:
            ms, t = timed(lib, a, b, c, m, n, k, 0.0, algo)
            lead = t[0::2]
            t0 = int(t[:, 1][t[:, 1] > 0].min())
            us = lambda col, rows: (rows[:, col].astype(np.int64) - t0) / 1000.0
            mma_end, store_end = us(3, lead), us(4, t)
            wait_us = t[:, 7].astype(float) / 1000.0
            spread = lambda x: [round(float(x.min()), 1), round(float(np.median(x)), 1), round(float(x.max()), 1)]
            print(json.dumps({
                "shape": f"{m}x{n}x{k}", "schedule": name, "ms": round(ms, 4),
                "last_mma_us_min_median_max": spread(mma_end),
                "last_store_us_min_median_max": spread(store_end),
                "acc_and_partial_wait_us_min_median_max": spread(wait_us),
                "k_blocks_per_pair": [int(lead[:, 6].min()), int(lead[:, 6].max())]}), flush=True)


if __name__ == "__main__":
    mode = sys.argv[1] if len(sys.argv) > 1 else "epilogue"
    {"epilogue": epilogue, "timeline": timeline}[mode]()
