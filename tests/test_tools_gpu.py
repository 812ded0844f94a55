"""The command-line tools on a GPU: they run, and their rows have the reference's keys
(benchmarks/bench_all.cpp:292-301, src/tools/device_probe.cu:108-131 of the reference)."""

import json
import os
import subprocess

import pytest

from conftest import tool_binary

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "cuda-kernel-library_b200", "build")


def _run(args):
    exe = tool_binary(args[0])
    env = dict(os.environ, CKL_REPO_ROOT=ROOT)
    out = subprocess.run([exe, *args[1:]], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return out.stdout


def test_device_probe_json():
    info = json.loads(_run(["device_probe", "--json"]))
    for key in ("name", "compute_capability", "sm_count", "global_mem_mib", "l2_cache_kib",
                "theoretical_bw_gbps", "measured_bw_gbps", "runtime_version", "driver_version"):
        assert key in info
    assert info["compute_capability"].startswith("10.") and info["sm_count"] > 0
    # a real HBM3e figure, not a few hundred GB/s of an under-filled probe
    assert info["measured_bw_gbps"] > 3000


def test_bench_all_row():
    row = json.loads(_run(["bench_all", "gemm", "auto", "bf16_c16", "2048", "2048", "2048", "t"]).strip())
    for key in ("family", "variant", "dtype", "m", "n", "k", "median_ms", "iqr_ms", "gflops",
                "baseline_gflops", "pct_baseline", "nvml_available", "median_sm_clock_mhz",
                "throttled", "cuda_runtime", "cuda_driver", "commit", "gpus", "tflops"):
        assert key in row
    assert row["family"] == "gemm" and row["gflops"] > 1000 and row["commit"] == "t"
    # unknown variant: exit code 3, like the reference
    exe = os.path.join(BUILD, "bench_all")
    bad = subprocess.run([exe, "gemm", "nope", "bf16", "64", "64", "64"], capture_output=True)
    assert bad.returncode == 3


def test_bench_all_fp32_and_trsm_rows():
    row = json.loads(_run(["bench_all", "gemm", "sgemm", "fp32", "1024", "1024", "1024", "t"]).strip())
    assert row["family"] == "gemm" and row["dtype"] == "fp32" and row["gflops"] > 1000
    row = json.loads(_run(["bench_all", "trsm", "blocked", "fp32", "1024", "512", "0", "t"]).strip())
    assert row["family"] == "trsm" and row["variant"] == "blocked" and row["gflops"] > 100


def test_roofline_writes_the_figure_inputs(tmp_path):
    """The two CSV files the reference's scripts/plot_roofline.py reads (its lines 53-61, 84-91,
    139-141): ceilings by quantity, points with label / intensity / achieved / ceiling."""
    import csv
    _run(["roofline", str(tmp_path)])
    with open(tmp_path / "roofline_ceilings.csv") as f:
        ceilings = {r["quantity"]: float(r["value"]) for r in csv.DictReader(f)}
    for key in ("bandwidth_gbps", "fp32_gflops", "tensor_gflops", "ridge_fp32", "ridge_tensor"):
        assert ceilings[key] > 0, key
    assert ceilings["tensor_gflops"] > 10 * ceilings["fp32_gflops"]
    with open(tmp_path / "roofline.csv") as f:
        points = list(csv.DictReader(f))
    assert {"label", "intensity_flop_per_byte", "achieved_gflops", "roof_gflops", "ceiling",
            "bound"} <= set(points[0])
    assert {p["ceiling"] for p in points} == {"tensor", "fp32"}


def test_stream_copy_is_exact(ckl):
    import torch
    for nbytes in (1 << 26, 1_000_016, 16):
        a = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
        b = torch.zeros_like(a)
        ckl.stream_copy(b, a, nbytes)
        torch.cuda.synchronize()
        assert torch.equal(a, b)
    with pytest.raises(ckl.CklError):
        ckl.stream_copy(b, a, 8)      # not a multiple of 16 bytes
