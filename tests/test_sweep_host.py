"""The sweep driver's resume logic, on CPU with a stand-in for the benchmark process
(reference behaviour: benchmarks/sweep.py:79-93,139-145 skips configurations already present
under the same key, --force redoes them)."""

import importlib.util
import json
import os
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    path = os.path.join(ROOT, "cuda-kernel-library_b200", "sweep.py")
    spec = importlib.util.spec_from_file_location("ckl_b200_sweep", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_sweep_resumes_and_forces(tmp_path):
    sw = _load()
    calls, cpu_calls = [], []

    def fake_run(cmd, **kwargs):
        if "torch.distributed.run" in cmd:            # an N-sharded row: one torchrun job
            gpus = int([c for c in cmd if c.startswith("--nproc-per-node=")][0].split("=")[1])
            assert cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"
            assert cmd[-7].endswith("sharded_row.py")
            variant, dtype, m, n, k, commit = cmd[-6:]
            family = "gemm"
        else:
            _, family, variant, dtype, m, n, k, commit = cmd
            gpus = 1
        if family == "cpu":                            # the CPU baseline, once per sweep
            cpu_calls.append(tuple(cmd[1:]))
            row = {"family": "cpu", "gflops": 2.5, "cpu_cores": 1}
            return types.SimpleNamespace(returncode=0, stdout=json.dumps(row) + "\n", stderr="")
        calls.append(tuple(cmd[1:]))
        if variant == "umma_1cta" and m == "1024":      # one configuration fails
            return types.SimpleNamespace(returncode=3, stdout="", stderr="boom")
        row = {"family": family, "variant": variant, "dtype": dtype, "m": int(m), "n": int(n),
               "k": int(k), "gpus": gpus, "median_ms": 1.0, "iqr_ms": 0.0, "gflops": 1.0,
               "tflops": 0.001, "commit": commit}
        return types.SimpleNamespace(returncode=0, stdout=json.dumps(row) + "\n", stderr="")

    total = len(list(sw.matrix(quick=True)))
    ran, skipped = sw.sweep(str(tmp_path), quick=True, commit="abc", runner=fake_run)
    assert (ran, skipped) == (total - 1, 0) and len(calls) == total
    # second pass: everything present is skipped, only the failed one is tried again
    calls.clear()
    ran, skipped = sw.sweep(str(tmp_path), quick=True, commit="abc", runner=fake_run)
    assert (ran, skipped) == (0, total - 1) and len(calls) == 1
    # another commit is another key; --force reruns regardless
    ran, _ = sw.sweep(str(tmp_path), quick=True, commit="def", runner=fake_run)
    assert ran == total - 1
    ran, skipped = sw.sweep(str(tmp_path), quick=True, commit="abc", force=True, runner=fake_run)
    assert (ran, skipped) == (total - 1, 0)
    header = open(tmp_path / "summary.csv").readline().strip().split(",")
    assert header[:7] == ["family", "variant", "dtype", "m", "n", "k", "gpus"]
    assert {"pct_peak_measured", "cpu_baseline_gflops", "cpu_cores"} <= set(header)
    # the CPU baseline is timed once per sweep that runs anything and lands in every row
    assert all(c[:3] == ("cpu", "reference", "fp32") for c in cpu_calls) and len(cpu_calls) == 3
    rows = [json.loads(line) for line in open(tmp_path / "sweep.jsonl")]
    assert all(r["cpu_baseline_gflops"] == 2.5 and r["cpu_cores"] == 1 for r in rows)
    # GPU counts above one add the N-sharded rows, keyed by `gpus`, one torchrun job each
    multi = [c for c in sw.matrix(quick=True, gpu_counts=[2, 8]) if c["gpus"] > 1]
    assert [(c["gpus"], c["m"]) for c in multi] == [(2, 8192), (8, 8192)]
    calls.clear()
    ran, skipped = sw.sweep(str(tmp_path), quick=True, commit="abc", runner=fake_run, gpu_counts=[2])
    assert ran == 1 and skipped == total - 1           # (the failing single-GPU one is tried again)
    rows = [json.loads(line) for line in open(tmp_path / "sweep.jsonl")]
    assert sum(1 for r in rows if r["gpus"] == 2 and r["commit"] == "abc") == 1


def test_ncu_round_commands(tmp_path, monkeypatch):
    """The profiling round (counterpart of benchmarks/run_ncu_round.sh of the reference) on CPU,
    with stand-ins for ncu and for the GEMM driver: every ncu call leaves the clocks alone, the
    plain run comes first and a configuration whose plain run fails is not profiled."""
    import stat
    import sys
    path = os.path.join(ROOT, "cuda-kernel-library_b200", "ncu_round.py")
    spec = importlib.util.spec_from_file_location("ckl_b200_ncu_round", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    log = tmp_path / "calls.log"
    fake_ncu = tmp_path / "fake_ncu"
    fake_ncu.write_text(f"#!/bin/sh\necho \"$@\" >> {log}\n"
                        "case \"$1\" in --import) echo details page;; esac\nexit 0\n")
    fake_ncu.chmod(fake_ncu.stat().st_mode | stat.S_IEXEC)
    fake_driver = tmp_path / "driver.py"
    fake_driver.write_text("import sys\nsys.exit(7 if 'umma_1cta' in sys.argv else 0)\n")
    monkeypatch.setattr(mod, "DRIVER", str(fake_driver))
    monkeypatch.setattr(sys, "argv", ["ncu_round.py", "r1", "umma_2cta_wide:8192", "umma_1cta:4096",
                                      "sgemm:2048", "umma_2cta:8192x1024x8192",
                                      "umma_2cta_streamk:1024x1024x32768:streamk_fixup_kernel",
                                      "--out", str(tmp_path), "--ncu", str(fake_ncu)])
    assert mod.main() == 1                       # one configuration failed its plain run
    calls = log.read_text().splitlines()
    profiled = [c for c in calls if "--export" in c]
    assert len(profiled) == 4 and all("--clock-control none" in c for c in profiled)
    assert "regex:umma_gemm_kernel" in profiled[0] and "--launch-skip 2 --launch-count 1" in profiled[0]
    assert "regex:sgemm_kernel" in profiled[1]
    assert "--m 8192 --n 1024 --k 8192" in profiled[2] and "umma_2cta_8192x1024x8192" in profiled[2]
    assert "regex:streamk_fixup_kernel" in profiled[3]
    assert "umma_2cta_streamk_1024x1024x32768_streamk_fixup_kernel" in profiled[3]
    assert mod.parse_pair("simt:129x257x193")[2] == "simt_gemm_kernel"
    assert "scatter_column_block_kernel" in mod.parse_pair("helpers:8192")[2]
    assert not any("umma_1cta" in c for c in calls)
    assert (tmp_path / "r1" / "umma_2cta_wide_8192.txt").read_text().strip() == "details page"
    meta = (tmp_path / "r1" / "round_meta.txt").read_text()
    assert "round: r1" in meta and "commit:" in meta


def test_bench_all_cpu_baseline_row():
    """`bench_all cpu reference fp32 m n k` times the CPU GEMM of ckl/reference.hpp (the
    reference's include/ckl/reference.hpp:29-46) on the host; no GPU is needed."""
    import subprocess
    from conftest import tool_binary
    out = subprocess.run([tool_binary("bench_all"), "cpu", "reference", "fp32", "96", "64", "80", "t"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    row = json.loads(out.stdout.strip())
    assert (row["family"], row["variant"], row["m"], row["n"], row["k"]) == ("cpu", "reference", 96, 64, 80)
    assert row["cpu_cores"] == 1 and row["gflops"] > 0 and row["gpus"] == 0
