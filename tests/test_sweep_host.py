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
    calls = []

    def fake_run(cmd, **kwargs):
        _, family, variant, dtype, m, n, k, commit = cmd
        calls.append(tuple(cmd[1:]))
        if variant == "umma_1cta" and m == "1024":      # one configuration fails
            return types.SimpleNamespace(returncode=3, stdout="", stderr="boom")
        row = {"family": family, "variant": variant, "dtype": dtype, "m": int(m), "n": int(n),
               "k": int(k), "gpus": 1, "median_ms": 1.0, "iqr_ms": 0.0, "gflops": 1.0,
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
