"""GPU parity of the FP32 GEMM (ckl_sgemm, behind ckl::gemm_naive / gemm_tiled / gemm_register /
gemm_cp_async) against the CPU oracle, through the C ABI.

Gate: the reference's own one for its FP32 ladder, relative Frobenius error < 1e-4
(tests/test_gemm.cpp:50 there), here against the double-accumulate CPU GEMM on the same
float inputs instead of against SGEMM; true FP32 arithmetic lands near 1e-7.
Shapes, alpha, beta and seeds are the reference's (tests/test_gemm.cpp:71-76,108-114).
"""

import numpy as np
import pytest

from conftest import dropin_binary

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

FP32_GATE = 1e-4
SHAPES = [  # tests/test_gemm.cpp:108-114 of the reference
    (256, 256, 256), (384, 512, 128), (129, 257, 193), (7, 5, 11), (512, 384, 640),
    (0, 128, 128), (128, 0, 128), (64, 64, 0),
]


@pytest.fixture(autouse=True)
def device_healthy(ckl):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    yield
    ckl.device_status()


def _inputs(orc, m, n, k):
    a = orc.random_matrix(m, k, 0x1234 + m)
    b = orc.random_matrix(k, n, 0x5678 + n)
    c0 = orc.random_matrix(m, n, 0x9ABC + k)
    return a, b, c0


def _dev(x, rows, cols):
    return torch.from_numpy(np.ascontiguousarray(x).reshape(rows, cols)).cuda()


@pytest.mark.parametrize("rung", ["gemm_naive", "gemm_tiled", "gemm_register", "gemm_cp_async"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_fp32_matrix(ckl, orc, shape, rung):
    m, n, k = shape
    alpha, beta = 1.25, 0.5
    a, b, c0 = _inputs(orc, m, n, k)
    da, db, dc = _dev(a, m, k), _dev(b, k, n), _dev(c0, m, n)
    getattr(ckl, rung)(da, db, dc, m, n, k, alpha, beta)
    torch.cuda.synchronize()
    if m * n == 0:
        return
    got = dc.cpu().numpy()
    if k == 0:
        np.testing.assert_array_equal(got, (np.float32(beta) * c0.reshape(m, n)).astype(np.float32))
        return
    ref, _ = orc.gemm_reference_mt(a, b, c0, alpha, beta)
    err = orc.relative_frobenius_error(got, ref)
    print(f"  {rung} {m}x{n}x{k}: rel_frob={err:.3e}")
    assert err < FP32_GATE
    assert err < 5e-6     # true FP32 multiply-add, not TF32


def test_beta_zero_does_not_read_c(ckl, orc):
    m, n, k = 130, 70, 33
    a, b, _ = _inputs(orc, m, n, k)
    dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    ckl.sgemm(_dev(a, m, k), _dev(b, k, n), dc, m, n, k, alpha=1.0, beta=0.0)
    torch.cuda.synchronize()
    got = dc.cpu().numpy()
    assert np.isfinite(got).all()
    ref, _ = orc.gemm_reference_mt(a, b, None, 1.0, 0.0)
    assert orc.relative_frobenius_error(got, ref) < 5e-6


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "misaligned"])
def test_leading_dimensions_and_alignment(ckl, orc, offset):
    """Sub-matrices of larger buffers (the layout a blocked solver hands to its trailing update):
    ld > width, and a base pointer that is only 4-byte aligned."""
    m, n, k = 200, 136, 72
    lda, ldb, ldc = k + 8, n + 4, n + 12
    a, b, c0 = _inputs(orc, m, n, k)
    big_a = torch.zeros(m * lda + offset, dtype=torch.float32, device="cuda")
    big_b = torch.zeros(k * ldb + offset, dtype=torch.float32, device="cuda")
    big_c = torch.full((m * ldc + offset,), 7.0, dtype=torch.float32, device="cuda")
    va = big_a[offset:].view(m, lda)
    vb = big_b[offset:].view(k, ldb)
    vc = big_c[offset:].view(m, ldc)
    va[:, :k] = _dev(a, m, k)
    vb[:, :n] = _dev(b, k, n)
    vc[:, :n] = _dev(c0, m, n)
    ckl.sgemm(va.data_ptr(), vb.data_ptr(), vc.data_ptr(), m, n, k, lda, ldb, ldc, -1.0, 1.0)
    torch.cuda.synchronize()
    host = vc.cpu().numpy()
    ref, _ = orc.gemm_reference_mt(a, b, c0, -1.0, 1.0)
    assert orc.relative_frobenius_error(np.ascontiguousarray(host[:, :n]), ref) < 5e-6
    assert (host[:, n:] == 7.0).all()      # padding columns untouched


@pytest.mark.parametrize("offset", [0, 1], ids=["aligned", "misaligned"])
def test_large_tile_with_ragged_edges_inside_padded_buffers(ckl, orc, offset):
    """Enough 128 x 128 tiles for the large-tile kernel, with n and k that end inside a group of
    four and leading dimensions that keep 16-byte alignment: the aligned case stages B with
    partial asynchronous copies at the right edge and whole zero-filled ones past k."""
    m, n, k = 2000, 1290, 333
    lda, ldb, ldc = 336, 1292, 1296
    a, b, c0 = _inputs(orc, m, n, k)
    big_a = torch.zeros(m * lda + offset, dtype=torch.float32, device="cuda")
    big_b = torch.full((k * ldb + offset,), float("nan"), dtype=torch.float32, device="cuda")
    big_c = torch.full((m * ldc + offset,), 7.0, dtype=torch.float32, device="cuda")
    va = big_a[offset:].view(m, lda)
    vb = big_b[offset:].view(k, ldb)
    vc = big_c[offset:].view(m, ldc)
    va[:, :k] = _dev(a, m, k)
    vb[:, :n] = _dev(b, k, n)          # the padding columns of B stay NaN: they must not be used
    vc[:, :n] = _dev(c0, m, n)
    ckl.sgemm(va.data_ptr(), vb.data_ptr(), vc.data_ptr(), m, n, k, lda, ldb, ldc, 0.5, -1.0)
    torch.cuda.synchronize()
    host = vc.cpu().numpy()
    ref, _ = orc.gemm_reference_mt(a, b, c0, 0.5, -1.0)
    assert orc.relative_frobenius_error(np.ascontiguousarray(host[:, :n]), ref) < 5e-6
    assert (host[:, n:] == 7.0).all()      # padding columns untouched


def test_larger_square_matches_sampled_oracle(ckl, orc):
    """2048^3: full rows and columns of the exact oracle (the whole matrix would take minutes)."""
    m = n = k = 2048
    a, b, _ = _inputs(orc, m, n, k)
    dc = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    ckl.sgemm(_dev(a, m, k), _dev(b, k, n), dc, m, n, k)
    torch.cuda.synchronize()
    got = dc.cpu().numpy()
    rows = np.array([0, 127, 128, 1023, 2047], dtype=np.int32)
    cols = np.array([0, 127, 128, 1500, 2047], dtype=np.int32)
    ref_rows, ref_cols = orc.gemm_sampled(a, b, None, 1.0, 0.0, rows, cols)
    assert orc.relative_frobenius_error(np.ascontiguousarray(got[rows, :]), ref_rows) < 5e-6
    assert orc.relative_frobenius_error(np.ascontiguousarray(got[:, cols].T), ref_cols) < 5e-6


def test_reference_fp32_test_driver_runs_unchanged():
    """The reference's own tests/test_gemm.cpp, compiled without edits against this repository's
    include/ckl headers and library (oracle/Makefile target `dropin`), passes: every FP32 rung
    within 1e-4 of SGEMM on the reference's shapes."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = dropin_binary("test_gemm_dropin")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "all GEMM cases passed" in out.stdout


def test_reference_fp32_bench_driver_runs_unchanged():
    """The reference's benchmarks/bench_gemm.cpp, compiled without edits against this
    repository's headers and library, times its four FP32 rungs and SGEMM at 256^3."""
    import subprocess
    exe = dropin_binary("bench_gemm_dropin")
    out = subprocess.run([exe, "256"], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    rows = [ln.split() for ln in out.stdout.splitlines()[1:] if ln.strip()]
    assert [r[1] for r in rows] == ["naive", "tiled", "register", "cp_async", "cublas"]
    for r in rows:
        assert r[0] == "256" and float(r[3]) > 0.0
