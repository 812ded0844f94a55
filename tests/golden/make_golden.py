"""Regenerates tests/golden/oracle_kat.json from the REFERENCE's own code.

Run in a container where the reference tree is mounted (it cannot travel to
the GPU box, so the vectors are committed):

    make -C oracle ref_cpu && python tests/golden/make_golden.py

Every value comes from oracle/_ref/libckl_ref.so, i.e. from the reference
header include/ckl/reference.hpp compiled unmodified (see oracle/ref_shim.cpp).
Shapes and seeds are the ones the reference's tensor GEMM test uses
(tests/test_gemm_tensor.cpp:62-63,105-110: A seed 0x1111+m, B seed 0x2222+n)
plus the FP32 512^3 plumbing case.
"""

import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ref = oracle.Reference()
    out = {"generator": "oracle/_ref/libckl_ref.so (reference include/ckl/reference.hpp, g++ -O2)",
           "random_matrix": [], "gemm_reference": [], "frobenius": []}

    for rows, cols, seed in [(512, 512, 0x1111 + 512), (512, 512, 0x2222 + 512), (7, 11, 0x1111 + 7),
                             (11, 5, 0x2222 + 5), (129, 193, 0x1111 + 129), (1, 1, 0), (3, 1000, 7),
                             (0, 5, 1)]:
        x = ref.random_matrix(rows, cols, seed)
        out["random_matrix"].append({
            "rows": rows, "cols": cols, "seed": seed, "sha256": sha(x),
            "head_bits": [int(v) for v in x.ravel()[:8].view(np.uint32)],
            "head": [float(v) for v in x.ravel()[:4]],
        })

    shapes = [(256, 256, 256), (384, 512, 128), (129, 257, 193), (7, 5, 11), (512, 384, 640),
              (64, 64, 0), (512, 512, 512)]
    for m, n, k in shapes:
        for alpha, beta in [(1.0, 0.0), (1.25, 0.5)]:
            a = ref.random_matrix(m, k, 0x1111 + m)
            b = ref.random_matrix(k, n, 0x2222 + n)
            c_in = ref.random_matrix(m, n, 0x9ABC + k) if beta != 0.0 else np.zeros((m, n), np.float32)
            c = ref.gemm_reference(a, b, c_in, alpha, beta)
            entry = {"m": m, "n": n, "k": k, "alpha": alpha, "beta": beta, "sha256": sha(c),
                     "first": float(c.ravel()[0]), "last": float(c.ravel()[-1]),
                     "sum": float(c.sum())}
            if m * n <= 64:
                entry["full"] = [float(v) for v in c.ravel()]
            out["gemm_reference"].append(entry)

    # relative_frobenius_error, including its absolute fallback for a zero reference
    a = ref.random_matrix(64, 64, 1)
    b = ref.random_matrix(64, 64, 2)
    c = ref.gemm_reference(a, b, None, 1.0, 0.0)
    noisy = (c + 1e-3 * ref.random_matrix(64, 64, 3)).astype(np.float32)
    out["frobenius"].append({"case": "noisy", "value": ref.relative_frobenius_error(noisy, c)})
    out["frobenius"].append({"case": "zero_ref", "value": ref.relative_frobenius_error(
        noisy, np.zeros_like(c))})
    out["frobenius"].append({"case": "exact", "value": ref.relative_frobenius_error(
        c.astype(np.float32), c.astype(np.float32).astype(np.float64))})

    path = os.path.join(ROOT, "tests", "golden", "oracle_kat.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


def trsm_main() -> None:
    """tests/golden/trsm_kat.json from the helpers of the reference's TRSM test
    (oracle/_ref/libckl_ref_trsm.so = tests/test_trsm.cpp of the reference, compiled where it
    lies); shapes, seeds and alpha are that test's (lines 92-95, 122-126)."""
    gemm_ref = oracle.Reference()
    ref = oracle.TrsmHelpers(from_reference=True)
    out = {"generator": "oracle/_ref/libckl_ref_trsm.so (reference tests/test_trsm.cpp, g++ -O2)",
           "cases": []}
    for m, n in [(256, 128), (512, 64), (129, 200), (5, 3), (64, 1), (65, 130)]:
        alpha = 1.5
        a = ref.make_lower(m, 0x71 + m)
        b = gemm_ref.random_matrix(m, n, 0x92 + n)
        x = ref.trsm_reference(a, b, alpha)
        entry = {"m": m, "n": n, "alpha": alpha, "lower_sha256": sha(a), "x_sha256": sha(x),
                 "x_first": float(x.ravel()[0]), "x_last": float(x.ravel()[-1]), "x_sum": float(x.sum()),
                 "residual_of_rounded_x": ref.trsm_residual(a, x.astype(np.float32), b, alpha)}
        if m * n <= 64:
            entry["x_full"] = [float(v) for v in x.ravel()]
        out["cases"].append(entry)
    path = os.path.join(ROOT, "tests", "golden", "trsm_kat.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    if "--trsm-only" not in sys.argv:
        main()
    trsm_main()
