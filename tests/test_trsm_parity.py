"""GPU parity of the blocked triangular solve (ckl_strsm_lower, behind ckl::trsm_naive /
trsm_blocked) against the CPU oracle, through the C ABI.

Gates are the reference's own (tests/test_trsm.cpp:101,113): relative Frobenius error against
the double-precision forward substitution < 1e-3 and residual ||L X - alpha B|| / ||alpha B||
< 1e-3; FP32 arithmetic on these well-conditioned systems lands near 1e-7, which is also
asserted.  Shapes, seeds and alpha are that test's (lines 92-95, 122-126), plus block-edge and
leading-dimension cases.
"""

import numpy as np
import pytest

from conftest import dropin_binary

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

SHAPES = [(256, 128), (512, 64), (129, 200), (5, 3), (64, 1), (65, 130), (1000, 257), (0, 8), (8, 0)]


@pytest.fixture(scope="module")
def trsm(oracle_mod):
    return oracle_mod.TrsmHelpers()


@pytest.fixture(autouse=True)
def device_healthy(ckl):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    yield
    ckl.device_status()


@pytest.mark.parametrize("rung", ["trsm_naive", "trsm_blocked"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_trsm_matrix(ckl, orc, trsm, shape, rung):
    m, n = shape
    alpha = 1.5
    a = trsm.make_lower(m, 0x71 + m)
    b = orc.random_matrix(m, n, 0x92 + n)
    da = torch.from_numpy(a).cuda()
    db = torch.from_numpy(b).cuda()
    getattr(ckl, rung)(da, db, m, n, alpha)
    torch.cuda.synchronize()
    if m * n == 0:
        return
    x = db.cpu().numpy()
    ref = trsm.trsm_reference(a, b, alpha)
    err = orc.relative_frobenius_error(x, ref)
    res = trsm.trsm_residual(a, x, b, alpha)
    print(f"  {rung} m={m} n={n}: vs oracle {err:.3e} residual {res:.3e}")
    assert err < 1e-3 and res < 1e-3
    assert err < 5e-6 and res < 5e-6


def test_leading_dimensions_and_upper_part_ignored(ckl, orc, trsm):
    m, n, alpha = 200, 77, -0.5
    lda, ldb = m + 4, n + 3
    a = trsm.make_lower(m, 3)
    b = orc.random_matrix(m, n, 4)
    big_a = torch.full((m, lda), float("nan"), dtype=torch.float32, device="cuda")
    big_a[:, :m] = torch.from_numpy(a).cuda()
    # NaN above the diagonal and in the padding: neither may be read
    iu = torch.triu_indices(m, m, 1, device="cuda")
    big_a[iu[0], iu[1]] = float("nan")
    big_b = torch.full((m, ldb), 9.0, dtype=torch.float32, device="cuda")
    big_b[:, :n] = torch.from_numpy(b).cuda()
    ckl.strsm_lower(big_a, big_b, m, n, lda, ldb, alpha)
    torch.cuda.synchronize()
    host = big_b.cpu().numpy()
    ref = trsm.trsm_reference(a, b, alpha)
    assert orc.relative_frobenius_error(np.ascontiguousarray(host[:, :n]), ref) < 5e-6
    assert (host[:, n:] == 9.0).all()


def test_large_system_residual(ckl, orc, trsm):
    """2048 x 2048 system with 512 right-hand sides: 31 trailing GEMM updates.  Checked by the
    residual (size-independent) and by the exact oracle on a few columns."""
    m, n, alpha = 2048, 512, 1.0
    a = trsm.make_lower(m, 21)
    b = orc.random_matrix(m, n, 22)
    db = torch.from_numpy(b).cuda()
    ckl.trsm_blocked(torch.from_numpy(a).cuda(), db, m, n, alpha)
    torch.cuda.synchronize()
    x = db.cpu().numpy()
    cols = [0, 127, 128, 511]
    ref = trsm.trsm_reference(a, np.ascontiguousarray(b[:, cols]), alpha)
    assert orc.relative_frobenius_error(np.ascontiguousarray(x[:, cols]), ref) < 5e-6
    lhs = torch.from_numpy(np.tril(a)).cuda().double() @ db.double()
    num = (lhs - alpha * torch.from_numpy(b).cuda().double()).norm().item()
    den = (alpha * torch.from_numpy(b).double()).norm().item()
    assert num / den < 5e-6


def test_reference_trsm_test_driver_runs_unchanged():
    """The reference's own tests/test_trsm.cpp, compiled without edits against this repository's
    include/ckl headers and library (oracle/Makefile target `dropin`), passes."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = dropin_binary("test_trsm_dropin")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "all TRSM cases passed" in out.stdout
