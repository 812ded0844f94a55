"""bench.py on a machine without a GPU: the reference arm (the reference's CPU GEMM timed on
the host cores) prints one JSON line with the contract's keys, other ranks of a multi-rank
launch stay silent, the product arm refuses to run without a CUDA device, and the DRAM-traffic
lookup only answers for a kernel and shape that was really captured."""

import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(args, env=None):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=600,
                          env=dict(os.environ, **(env or {})))


def test_reference_arm_prints_the_contract_line():
    out = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["config"]["workload"] == "bf16_8192_cubed" and line["n_gpus"] == 1
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("reference", "port") and cpu["cores"] == (os.cpu_count() or 1)
    assert cpu["value"] == line["value"] and "rows" in cpu["sample"]


def test_reference_arm_runs_on_rank_zero_only():
    out = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
               env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_product_arm_has_no_cpu_path():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present; this checks the behaviour of a machine without one")
    out = _run(["--steps", "1", "--warmup", "0"])
    assert out.returncode != 0 and "no CPU path" in (out.stderr + out.stdout)


def test_dram_traffic_lookup_answers_only_for_captured_kernels():
    spec = importlib.util.spec_from_file_location("ckl_bench", BENCH)
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    got = bench.ncu_dram_traffic("umma_2cta_wide", 8192, 8192, 8192)
    assert got is not None and 0.5e9 < got < 2.5e9
    assert bench.ncu_dram_traffic("umma_2cta", 8192, 8192, 8192) is None      # never captured
    assert bench.ncu_dram_traffic("umma_2cta_wide", 4096, 4096, 4096) is None
