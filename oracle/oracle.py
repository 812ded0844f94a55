"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product package never does.  It loads

* ``oracle/libckl_oracle.so`` -- the plain-C restatement (``ckl_oracle.c``) of
  the reference's host helpers (``include/ckl/reference.hpp:16-63`` and the
  16-bit narrowing of ``tests/test_gemm_tensor.cpp:40-56``), and
* ``oracle/_ref/libckl_ref.so`` when present -- the reference's own header
  compiled through ``ref_shim.cpp``.

Arrays are numpy, row-major, float32 in and float64 out, exactly as the
reference's ``std::vector<float>`` / ``std::vector<double>`` interfaces.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libckl_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libckl_ref.so")
_REF_TRSM_PATH = os.path.join(_HERE, "_ref", "libckl_ref_trsm.so")

F16 = 1
BF16 = 2

_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_ip = ctypes.POINTER(ctypes.c_int)


def reference_tree() -> str:
    """Where the reference library's source tree is looked for: $CKL_REFERENCE, else a
    checkout named ``reference`` beside this repository.  It may be absent."""
    return os.environ.get("CKL_REFERENCE") or os.path.join(
        os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force: bool = False) -> None:
    """Compile the plain-C oracle (and the reference shim where the reference
    tree is mounted).  Building the checker is not using it."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "ckl_oracle.c")
    ):
        subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    reference = reference_tree()
    if os.path.isdir(os.path.join(reference, "include", "ckl")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REFERENCE={reference}"], check=True)


def _f(a):
    return a.ctypes.data_as(_fp)


def _d(a):
    return a.ctypes.data_as(_dp)


class _Lib:
    def __init__(self, path: str, prefix: str):
        self.lib = ctypes.CDLL(path)
        self.prefix = prefix
        L = self.lib
        rm = getattr(L, prefix + "random_matrix")
        rm.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_uint64, _fp]
        rm.restype = None
        gr = getattr(L, prefix + "gemm_reference")
        gr.argtypes = [_fp, _fp, _fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                       ctypes.c_float, _dp]
        gr.restype = None
        fe = getattr(L, prefix + "relative_frobenius_error")
        fe.argtypes = [_fp, _dp, ctypes.c_size_t]
        fe.restype = ctypes.c_double

    def random_matrix(self, rows: int, cols: int, seed: int) -> np.ndarray:
        out = np.empty((rows, cols), dtype=np.float32)
        if out.size:
            getattr(self.lib, self.prefix + "random_matrix")(rows, cols, seed, _f(out))
        return out

    def gemm_reference(self, a, b, c_in, alpha: float, beta: float) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        m, k = a.shape
        n = b.shape[1]
        assert b.shape[0] == k
        if c_in is None:
            c_in = np.zeros((m, n), dtype=np.float32)
        c_in = np.ascontiguousarray(c_in, dtype=np.float32)
        out = np.empty((m, n), dtype=np.float64)
        if out.size:
            getattr(self.lib, self.prefix + "gemm_reference")(
                _f(a), _f(b), _f(c_in), m, n, k, alpha, beta, _d(out))
        return out

    def relative_frobenius_error(self, actual, ref) -> float:
        actual = np.ascontiguousarray(actual, dtype=np.float32).ravel()
        ref = np.ascontiguousarray(ref, dtype=np.float64).ravel()
        assert actual.size == ref.size
        return float(getattr(self.lib, self.prefix + "relative_frobenius_error")(
            _f(actual), _d(ref), actual.size))


class Oracle(_Lib):
    """The plain-C restatement plus the helpers that only it has."""

    def __init__(self):
        if not os.path.exists(_LIB_PATH):
            build()
        super().__init__(_LIB_PATH, "ckl_oracle_")
        L = self.lib
        L.ckl_oracle_mt64_nth.argtypes = [ctypes.c_uint64, ctypes.c_uint64]
        L.ckl_oracle_mt64_nth.restype = ctypes.c_uint64
        L.ckl_oracle_gemm_reference_mt.argtypes = [
            _fp, _fp, _fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
            ctypes.c_float, _dp, ctypes.c_int]
        L.ckl_oracle_gemm_reference_mt.restype = ctypes.c_int
        L.ckl_oracle_gemm_sampled.argtypes = [
            _fp, _fp, _fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
            ctypes.c_float, _ip, ctypes.c_int, _ip, ctypes.c_int, _dp, _dp]
        L.ckl_oracle_gemm_sampled.restype = None
        L.ckl_oracle_narrow.argtypes = [_fp, _u16p, ctypes.c_size_t, ctypes.c_int]
        L.ckl_oracle_narrow.restype = None
        L.ckl_oracle_widen.argtypes = [_u16p, _fp, ctypes.c_size_t, ctypes.c_int]
        L.ckl_oracle_widen.restype = None
        L.ckl_oracle_max_threads.restype = ctypes.c_int

    def mt64_nth(self, seed: int, n: int) -> int:
        return int(self.lib.ckl_oracle_mt64_nth(seed, n))

    def max_threads(self) -> int:
        return int(self.lib.ckl_oracle_max_threads())

    def gemm_reference_mt(self, a, b, c_in, alpha: float, beta: float, threads: int = 0):
        """Row-parallel form of gemm_reference; returns (C, threads_used)."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        m, k = a.shape
        n = b.shape[1]
        if c_in is None:
            c_in = np.zeros((m, n), dtype=np.float32)
        c_in = np.ascontiguousarray(c_in, dtype=np.float32)
        out = np.empty((m, n), dtype=np.float64)
        used = self.lib.ckl_oracle_gemm_reference_mt(
            _f(a), _f(b), _f(c_in), m, n, k, alpha, beta, _d(out), threads)
        return out, int(used)

    def gemm_sampled(self, a, b, c_in, alpha: float, beta: float, rows, cols):
        """Exact reference values of the listed full rows and full columns of C.
        Returns (rows_out [len(rows), n], cols_out [len(cols), m])."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        m, k = a.shape
        n = b.shape[1]
        if c_in is None:
            c_in = np.zeros((m, n), dtype=np.float32)
        c_in = np.ascontiguousarray(c_in, dtype=np.float32)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        cols = np.ascontiguousarray(cols, dtype=np.int32)
        rows_out = np.empty((rows.size, n), dtype=np.float64)
        cols_out = np.empty((cols.size, m), dtype=np.float64)
        self.lib.ckl_oracle_gemm_sampled(
            _f(a), _f(b), _f(c_in), m, n, k, alpha, beta,
            rows.ctypes.data_as(_ip), rows.size, cols.ctypes.data_as(_ip), cols.size,
            _d(rows_out), _d(cols_out))
        return rows_out, cols_out

    def narrow(self, x, dtype: int) -> np.ndarray:
        """float32 -> FP16/BF16 bit patterns (uint16), round to nearest even."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint16)
        if x.size:
            self.lib.ckl_oracle_narrow(_f(x), out.ctypes.data_as(_u16p), x.size, dtype)
        return out

    def widen(self, bits, dtype: int) -> np.ndarray:
        """FP16/BF16 bit patterns (uint16) -> float32, exact."""
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, dtype=np.float32)
        if bits.size:
            self.lib.ckl_oracle_widen(bits.ctypes.data_as(_u16p), _f(out), bits.size, dtype)
        return out

    def round_through(self, x, dtype: int) -> np.ndarray:
        """The float32 values a 16-bit kernel actually sees: narrow, then widen."""
        return self.widen(self.narrow(x, dtype), dtype)


class Reference(_Lib):
    """The reference's own header, when it was compiled in this container."""

    def __init__(self):
        super().__init__(_REF_PATH, "ckl_ref_")


class TrsmHelpers:
    """make_lower / trsm_reference / residual of the reference's TRSM test
    (tests/test_trsm.cpp:20-69): the plain-C port by default, or the reference's own code
    from oracle/_ref/libckl_ref_trsm.so with ``from_reference=True``."""

    def __init__(self, from_reference: bool = False):
        if from_reference:
            self.lib, prefix = ctypes.CDLL(_REF_TRSM_PATH), "ckl_ref_"
        else:
            if not os.path.exists(_LIB_PATH):
                build()
            self.lib, prefix = ctypes.CDLL(_LIB_PATH), "ckl_oracle_"
        self._make_lower = getattr(self.lib, prefix + "make_lower")
        self._make_lower.argtypes = [ctypes.c_int, ctypes.c_uint64, _fp]
        self._make_lower.restype = None
        self._solve = getattr(self.lib, prefix + "trsm_reference")
        self._solve.argtypes = [_fp, _fp, ctypes.c_int, ctypes.c_int, ctypes.c_float, _dp]
        self._solve.restype = None
        self._residual = getattr(self.lib, prefix + "trsm_residual")
        self._residual.argtypes = [_fp, _fp, _fp, ctypes.c_int, ctypes.c_int, ctypes.c_float]
        self._residual.restype = ctypes.c_double

    def make_lower(self, m: int, seed: int) -> np.ndarray:
        out = np.empty((m, m), dtype=np.float32)
        if out.size:
            self._make_lower(m, seed, _f(out))
        return out

    def trsm_reference(self, a, b, alpha: float) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        m, n = b.shape
        assert a.shape == (m, m)
        x = np.empty((m, n), dtype=np.float64)
        if x.size:
            self._solve(_f(a), _f(b), m, n, alpha, _d(x))
        return x

    def trsm_residual(self, a, x, b, alpha: float) -> float:
        a = np.ascontiguousarray(a, dtype=np.float32)
        x = np.ascontiguousarray(x, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        m, n = b.shape
        return float(self._residual(_f(a), _f(x), _f(b), m, n, alpha))


def have_reference_trsm() -> bool:
    return os.path.exists(_REF_TRSM_PATH)


class RowBlockTimer:
    """Runs the CPU GEMM on blocks of rows of one problem, B prepared once.  Uses the
    reference's own function when oracle/_ref is built (kind "reference"), else the plain-C
    port (kind "port").  Thread-safe: ctypes drops the GIL during the call."""

    def __init__(self, b):
        self.b = np.ascontiguousarray(b, dtype=np.float32)
        self.k, self.n = self.b.shape
        if have_reference():
            self.kind = "reference"
            self.lib = ctypes.CDLL(_REF_PATH)
            self.lib.ckl_ref_bench_create.argtypes = [_fp, ctypes.c_int, ctypes.c_int]
            self.lib.ckl_ref_bench_create.restype = ctypes.c_void_p
            self.lib.ckl_ref_bench_run.argtypes = [ctypes.c_void_p, _fp, _fp, ctypes.c_int,
                                                   ctypes.c_float, ctypes.c_float, _dp]
            self.lib.ckl_ref_bench_run.restype = None
            self.lib.ckl_ref_bench_destroy.argtypes = [ctypes.c_void_p]
            self.handle = self.lib.ckl_ref_bench_create(_f(self.b), self.k, self.n)
        else:
            self.kind = "port"
            self.port = Oracle()
            self.handle = None

    def run(self, a_rows, c_rows, alpha: float, beta: float, out):
        rows = a_rows.shape[0]
        if self.kind == "reference":
            self.lib.ckl_ref_bench_run(self.handle, _f(a_rows), _f(c_rows), rows, alpha, beta, _d(out))
        else:
            self.port.lib.ckl_oracle_gemm_reference(_f(a_rows), _f(self.b), _f(c_rows), rows,
                                                    self.n, self.k, alpha, beta, _d(out))

    def close(self):
        if self.handle is not None:
            self.lib.ckl_ref_bench_destroy(self.handle)
            self.handle = None


def have_reference() -> bool:
    return os.path.exists(_REF_PATH)


def checksum_identity(a, b, c_in, alpha: float, beta: float):
    """Row sums and column sums of the exact C, in double, at O(mk + kn + mn):
    C @ 1 = alpha * A @ (B @ 1) + beta * C_in @ 1 and 1^T @ C likewise.  A
    size-independent property used where the full oracle is unaffordable."""
    a64 = np.asarray(a, dtype=np.float64)
    b64 = np.asarray(b, dtype=np.float64)
    row_sums = alpha * (a64 @ b64.sum(axis=1))
    col_sums = alpha * (a64.sum(axis=0) @ b64)
    if c_in is not None and beta != 0.0:
        c64 = np.asarray(c_in, dtype=np.float64)
        row_sums = row_sums + beta * c64.sum(axis=1)
        col_sums = col_sums + beta * c64.sum(axis=0)
    return row_sums, col_sums
