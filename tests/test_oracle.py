"""The CPU oracle against the reference's own outputs.

tests/golden/oracle_kat.json was generated from the reference header compiled unmodified
(tests/golden/make_golden.py); the plain-C restatement in oracle/ckl_oracle.c must reproduce
it bit for bit.  Where the reference build itself is present (oracle/_ref, only in a container
with the reference tree) the two are also compared directly on fresh inputs.
"""

import hashlib
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "oracle_kat.json")) as f:
    GOLD = json.load(f)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_mt19937_64_standard_value(orc):
    # The C++ standard fixes the 10000th output of a default-seeded mt19937_64.
    assert orc.mt64_nth(5489, 10000) == 9981545732273789042


@pytest.mark.parametrize("entry", GOLD["random_matrix"], ids=lambda e: f"{e['rows']}x{e['cols']}")
def test_random_matrix_matches_reference(orc, entry):
    x = orc.random_matrix(entry["rows"], entry["cols"], entry["seed"])
    assert x.shape == (entry["rows"], entry["cols"])
    assert sha(x) == entry["sha256"]
    head = [int(v) for v in x.ravel()[:8].view(np.uint32)]
    assert head == entry["head_bits"]
    if x.size:
        assert x.min() >= -1.0 and x.max() < 1.0


def test_random_matrix_known_answers(orc):
    a = orc.random_matrix(512, 512, 0x1111 + 512)
    b = orc.random_matrix(512, 512, 0x2222 + 512)
    assert a.ravel()[0] == np.float32(-0.767540812)
    assert a.ravel()[1] == np.float32(0.474851489)
    assert b.ravel()[0] == np.float32(0.170882821)


@pytest.mark.parametrize("entry", GOLD["gemm_reference"],
                         ids=lambda e: f"{e['m']}x{e['n']}x{e['k']}-b{e['beta']}")
def test_gemm_reference_matches_reference(orc, entry):
    m, n, k = entry["m"], entry["n"], entry["k"]
    a = orc.random_matrix(m, k, 0x1111 + m)
    b = orc.random_matrix(k, n, 0x2222 + n)
    beta = entry["beta"]
    c_in = orc.random_matrix(m, n, 0x9ABC + k) if beta != 0.0 else np.zeros((m, n), np.float32)
    if m * n * k > 256 ** 3:
        c, _ = orc.gemm_reference_mt(a, b, c_in, entry["alpha"], beta)  # bit-identical, faster
    else:
        c = orc.gemm_reference(a, b, c_in, entry["alpha"], beta)
    assert sha(c) == entry["sha256"]
    assert c.ravel()[0] == entry["first"] and c.ravel()[-1] == entry["last"]
    if "full" in entry:
        assert [float(v) for v in c.ravel()] == entry["full"]


def test_threaded_and_sampled_forms_are_bit_identical(orc):
    a = orc.random_matrix(96, 80, 1)
    b = orc.random_matrix(80, 72, 2)
    c_in = orc.random_matrix(96, 72, 3)
    full = orc.gemm_reference(a, b, c_in, 1.25, 0.5)
    mt, used = orc.gemm_reference_mt(a, b, c_in, 1.25, 0.5)
    assert used >= 1 and np.array_equal(full, mt)
    rows, cols = [0, 17, 95], [0, 71, 33]
    r, c = orc.gemm_sampled(a, b, c_in, 1.25, 0.5, rows, cols)
    assert np.array_equal(r, full[rows, :])
    assert np.array_equal(c, full[:, cols].T)


def test_frobenius_matches_reference(orc):
    a = orc.random_matrix(64, 64, 1)
    b = orc.random_matrix(64, 64, 2)
    c = orc.gemm_reference(a, b, None, 1.0, 0.0)
    noisy = (c + 1e-3 * orc.random_matrix(64, 64, 3)).astype(np.float32)
    gold = {e["case"]: e["value"] for e in GOLD["frobenius"]}
    assert orc.relative_frobenius_error(noisy, c) == gold["noisy"]
    assert orc.relative_frobenius_error(noisy, np.zeros_like(c)) == gold["zero_ref"]
    assert orc.relative_frobenius_error(c.astype(np.float32),
                                        c.astype(np.float32).astype(np.float64)) == gold["exact"]


def test_narrowing_is_round_to_nearest_even(orc, oracle_mod):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.uniform(-70000, 70000, 50000), rng.normal(0, 1e-4, 50000), rng.normal(0, 1e-7, 20000),
        [0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.98e-8, 2.9802322e-8, 3e-8, 6.1e-5, np.inf, -np.inf],
    ]).astype(np.float32)
    h = orc.narrow(x, oracle_mod.F16)
    with np.errstate(over="ignore"):
        assert np.array_equal(h, x.astype(np.float16).view(np.uint16))
    assert np.array_equal(orc.widen(h, oracle_mod.F16), h.view(np.float16).astype(np.float32))
    # bf16: round to nearest even on the upper half of the binary32 pattern
    u = x.view(np.uint32).astype(np.uint64)
    expect = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    b = orc.narrow(x, oracle_mod.BF16)
    assert np.array_equal(b, expect)
    assert np.array_equal(orc.widen(b, oracle_mod.BF16).view(np.uint32), b.astype(np.uint32) << 16)
    assert orc.narrow(np.array([np.nan], np.float32), oracle_mod.BF16)[0] & 0x7F80 == 0x7F80


def test_checksum_identity_agrees_with_full_oracle(orc, oracle_mod):
    a = orc.random_matrix(40, 56, 5)
    b = orc.random_matrix(56, 24, 6)
    c_in = orc.random_matrix(40, 24, 7)
    c = orc.gemm_reference(a, b, c_in, 0.75, -0.5)
    rs, cs = oracle_mod.checksum_identity(a, b, c_in, 0.75, -0.5)
    assert np.allclose(rs, c.sum(axis=1), rtol=0, atol=1e-10)
    assert np.allclose(cs, c.sum(axis=0), rtol=0, atol=1e-10)


def test_restatement_equals_reference_build(orc, oracle_mod):
    if not oracle_mod.have_reference():
        pytest.skip("oracle/_ref not built (reference tree not mounted on this machine)")
    ref = oracle_mod.Reference()
    for (m, n, k, seed) in [(33, 17, 65, 11), (64, 64, 64, 12), (1, 200, 3, 13)]:
        a, b = orc.random_matrix(m, k, seed), orc.random_matrix(k, n, seed + 100)
        assert np.array_equal(a.view(np.uint32), ref.random_matrix(m, k, seed).view(np.uint32))
        c_in = orc.random_matrix(m, n, seed + 200)
        c1, c2 = orc.gemm_reference(a, b, c_in, 1.5, 0.25), ref.gemm_reference(a, b, c_in, 1.5, 0.25)
        assert np.array_equal(c1, c2)
        x = c1.astype(np.float32) + np.float32(1e-4)
        assert orc.relative_frobenius_error(x, c1) == ref.relative_frobenius_error(x, c2)


def test_cpp_harness_header_matches_golden(tmp_path, orc):
    """include/ckl/reference.hpp (used by the C++ drivers) produces the reference's values."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("g++ not available")
    root = os.path.dirname(HERE)
    src = tmp_path / "probe.cpp"
    src.write_text(r'''
#include <cstdio>
#include "ckl/reference.hpp"
int main() {
    const int m = 129, n = 257, k = 193;
    auto a = ckl::random_matrix(m, k, 0x1111 + m);
    auto b = ckl::random_matrix(k, n, 0x2222 + n);
    std::vector<float> c0(static_cast<size_t>(m) * n, 0.0f);
    auto c = ckl::gemm_reference(a, b, c0, m, n, k, 1.0f, 0.0f);
    std::FILE* f = std::fopen("c.bin", "wb");
    std::fwrite(c.data(), sizeof(double), c.size(), f);
    std::fclose(f);
    std::vector<float> cf(c.begin(), c.end());
    std::printf("%.17g\n", ckl::relative_frobenius_error(cf, c));
}
''')
    exe = tmp_path / "probe"
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", os.path.join(root, "include"), str(src), "-o",
                    str(exe)], check=True)
    subprocess.run([str(exe)], check=True, cwd=tmp_path, capture_output=True)
    c = np.fromfile(tmp_path / "c.bin", dtype=np.float64)
    gold = next(e for e in GOLD["gemm_reference"]
                if (e["m"], e["n"], e["k"], e["beta"]) == (129, 257, 193, 0.0))
    assert sha(c) == gold["sha256"]
