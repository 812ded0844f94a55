"""CPU checks of the triangular-solve oracle: the plain-C restatement of the helpers in the
reference's TRSM test (tests/test_trsm.cpp:20-69) against golden vectors produced by that
reference code itself (tests/golden/trsm_kat.json, generator tests/golden/make_golden.py), and,
where oracle/_ref is built, against the reference code directly."""

import hashlib
import json
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def kat():
    with open(os.path.join(ROOT, "tests", "golden", "trsm_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def trsm(oracle_mod):
    return oracle_mod.TrsmHelpers()


def test_port_matches_golden_bit_for_bit(kat, trsm, orc):
    assert len(kat["cases"]) >= 6
    for case in kat["cases"]:
        m, n, alpha = case["m"], case["n"], case["alpha"]
        a = trsm.make_lower(m, 0x71 + m)                  # tests/test_trsm.cpp:92-93
        b = orc.random_matrix(m, n, 0x92 + n)
        assert sha(a) == case["lower_sha256"], (m, n)
        x = trsm.trsm_reference(a, b, alpha)
        assert sha(x) == case["x_sha256"], (m, n)
        assert float(x.ravel()[0]) == case["x_first"] and float(x.ravel()[-1]) == case["x_last"]
        if "x_full" in case:
            assert [float(v) for v in x.ravel()] == case["x_full"]
        res = trsm.trsm_residual(a, x.astype(np.float32), b, alpha)
        assert res == pytest.approx(case["residual_of_rounded_x"], rel=1e-12)
        assert res < 1e-6


def test_lower_matrix_structure(trsm):
    a = trsm.make_lower(33, 5)
    assert (np.triu(a, 1) == 0).all()
    assert (np.diag(a) == 34.0).all()
    assert np.abs(np.tril(a, -1)).max() <= 1.0


def test_solution_satisfies_the_system(trsm, orc):
    m, n, alpha = 97, 41, -0.75
    a = trsm.make_lower(m, 11)
    b = orc.random_matrix(m, n, 12)
    x = trsm.trsm_reference(a, b, alpha)
    lhs = np.tril(a).astype(np.float64) @ x
    assert np.allclose(lhs, alpha * b.astype(np.float64), rtol=0, atol=1e-12)


def test_port_matches_reference_code_directly(oracle_mod, trsm, orc):
    if not oracle_mod.have_reference_trsm():
        pytest.skip("oracle/_ref/libckl_ref_trsm.so not built (needs the reference tree)")
    ref = oracle_mod.TrsmHelpers(from_reference=True)
    for m, n, alpha in [(70, 9, 1.5), (128, 128, 1.0), (1, 4, 2.0), (200, 3, -0.5)]:
        a = trsm.make_lower(m, 0x71 + m)
        assert np.array_equal(a, ref.make_lower(m, 0x71 + m))
        b = orc.random_matrix(m, n, 0x92 + n)
        x = trsm.trsm_reference(a, b, alpha)
        assert np.array_equal(x, ref.trsm_reference(a, b, alpha))
        xf = x.astype(np.float32)
        assert trsm.trsm_residual(a, xf, b, alpha) == ref.trsm_residual(a, xf, b, alpha)
