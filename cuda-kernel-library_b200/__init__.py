"""B200 (sm_100a) tensor-core GEMM: Python front end of the C ABI.

The product is ``libckl_gemm.so`` (hand-written CUDA, C ABI declared in
``include/ckl_gemm.h``).  This module only binds it with ctypes and mirrors
the reference library's entry points (``include/ckl/gemm.hpp:68-100`` there):
same names, same argument order and meaning, row-major device pointers,
``stream`` last, an exception where the C++ launchers throw.

Pointers may be given as integers or as anything with ``data_ptr()`` (a torch
tensor is only a convenient owner of device memory; nothing here computes with
torch).  There is no CPU path: without the compiled library the import fails,
and without an sm_100 GPU every call raises ``CklError``.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libckl_gemm.so")

# ckl_status
OK, ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE, ERR_TOO_LARGE = range(6)
# ckl_dtype
F32, F16, BF16 = 0, 1, 2
# ckl_algo
(ALGO_AUTO, ALGO_SIMT, ALGO_UMMA_1CTA, ALGO_UMMA_SK, ALGO_UMMA_2CTA, ALGO_UMMA_2CTA_SK,
 ALGO_UMMA_2CTA_WIDE, ALGO_UMMA_2CTA_WIDE_SK, ALGO_UMMA_1CTA_N128, ALGO_UMMA_1CTA_N128_SK) = range(10)
NUM_ALGOS = 10


class CklError(RuntimeError):
    """A non-zero ckl_status; ``status`` holds the code, the text is ckl_last_error()."""

    def __init__(self, status: int, message: str):
        super().__init__(f"ckl status {status}: {message}")
        self.status = status


class Plan(ctypes.Structure):
    _fields_ = [
        ("algo", ctypes.c_int), ("tile_m", ctypes.c_int), ("tile_n", ctypes.c_int),
        ("tile_k", ctypes.c_int), ("tiles_m", ctypes.c_int), ("tiles_n", ctypes.c_int),
        ("k_blocks", ctypes.c_int), ("grid", ctypes.c_int), ("units", ctypes.c_int),
        ("group_m", ctypes.c_int), ("dp_tiles", ctypes.c_int),
        ("sk_tiles", ctypes.c_int), ("sk_units", ctypes.c_int), ("sk_iters", ctypes.c_longlong),
        ("workspace_bytes", ctypes.c_size_t), ("repack", ctypes.c_int),
    ]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
        "(needs nvcc; there is no fallback implementation)")

_lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_lib.ckl_gemm_f16.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
_lib.ckl_gemm_bf16.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
_lib.ckl_gemm_ex.argtypes = [_i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _vp]
_lib.ckl_gemm_bias_relu_ex.argtypes = [_i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _f, _i,
                                       _vp]
_lib.ckl_bias_relu_f32.argtypes = [_vp, _vp, _i, _i, _i, _vp]
_lib.ckl_gemm_host.argtypes = [_i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f]
_lib.ckl_sgemm.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
_lib.ckl_strsm_lower.argtypes = [_vp, _vp, _i, _i, _i, _i, _f, _vp]
_lib.ckl_plan_gemm.argtypes = [_i, _i, _i, _i, _i, _i, _i, _i, _i, _i, ctypes.POINTER(Plan)]
_lib.ckl_plan_sk_range.argtypes = [ctypes.POINTER(Plan), _i, ctypes.POINTER(ctypes.c_longlong),
                                   ctypes.POINTER(ctypes.c_longlong)]
_lib.ckl_plan_unit_segments.argtypes = [ctypes.POINTER(Plan), _i, ctypes.POINTER(ctypes.c_int), _i]
_lib.ckl_plan_fixup_slots.argtypes = [ctypes.POINTER(Plan), _i, ctypes.POINTER(ctypes.c_int), _i]
_lib.ckl_assemble_column_blocks.argtypes = [_vp, _vp, _i, _i, _i, _i, _vp]
_lib.ckl_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
_lib.ckl_stream_copy.argtypes = [_vp, _vp, ctypes.c_size_t, _vp]
_lib.ckl_last_error.restype = ctypes.c_char_p
_lib.ckl_algo_name.argtypes = [_i]
_lib.ckl_algo_name.restype = ctypes.c_char_p
_lib.ckl_shutdown.restype = None
for _name in ("ckl_gemm_f16", "ckl_gemm_bf16", "ckl_gemm_ex", "ckl_gemm_bias_relu_ex",
              "ckl_bias_relu_f32", "ckl_gemm_host", "ckl_sgemm", "ckl_strsm_lower", "ckl_plan_gemm", "ckl_plan_sk_range",
              "ckl_device_status", "ckl_stream_copy", "ckl_plan_unit_segments",
              "ckl_plan_fixup_slots", "ckl_assemble_column_blocks"):
    getattr(_lib, _name).restype = ctypes.c_int


def _ptr(x) -> int | None:
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    return int(x)


def _stream(s) -> int | None:
    if s is None:
        return None
    if hasattr(s, "cuda_stream"):
        return int(s.cuda_stream)
    return int(s)


def _check(status: int) -> None:
    if status != OK:
        raise CklError(status, _lib.ckl_last_error().decode())


def last_error() -> str:
    return _lib.ckl_last_error().decode()


def algo_name(algo: int) -> str:
    return _lib.ckl_algo_name(algo).decode()


def gemm_ex(ab_dtype, a, b, c, c_dtype, m, n, k, lda, ldb, ldc, alpha, beta, algo=ALGO_AUTO,
            stream=None) -> None:
    """C = alpha*A*B + beta*C with explicit dtypes, leading dimensions and kernel choice."""
    _check(_lib.ckl_gemm_ex(ab_dtype, _ptr(a), _ptr(b), _ptr(c), c_dtype, m, n, k, lda, ldb, ldc,
                            alpha, beta, algo, _stream(stream)))


def gemm_f16(a, b, c, c_dtype, m, n, k, lda, ldb, ldc, alpha, beta, stream=None) -> None:
    _check(_lib.ckl_gemm_f16(_ptr(a), _ptr(b), _ptr(c), c_dtype, m, n, k, lda, ldb, ldc, alpha,
                             beta, _stream(stream)))


def gemm_bf16(a, b, c, c_dtype, m, n, k, lda, ldb, ldc, alpha, beta, stream=None) -> None:
    _check(_lib.ckl_gemm_bf16(_ptr(a), _ptr(b), _ptr(c), c_dtype, m, n, k, lda, ldb, ldc, alpha,
                              beta, _stream(stream)))


# --- the reference's entry points, FP32 C, lda = k, ldb = ldc = n ---------------------
# (include/ckl/gemm.hpp:68-86 of the reference; every FP16 rung is the same function.)

def gemm_wmma_fp16(a, b, c, m, n, k, alpha, beta, stream=None) -> None:
    gemm_f16(a, b, c, F32, m, n, k, k, n, n, alpha, beta, stream)


def gemm_wmma_bf16(a, b, c, m, n, k, alpha, beta, stream=None) -> None:
    gemm_bf16(a, b, c, F32, m, n, k, k, n, n, alpha, beta, stream)


gemm_mma_ptx = gemm_wmma_fp16
gemm_mma_ldm = gemm_wmma_fp16
gemm_mma_opt = gemm_wmma_fp16


def gemm_naive(a, b, c, m, n, k, alpha, beta, stream=None) -> None:
    """FP32 ladder (include/ckl/gemm.hpp:40-58 of the reference): every rung is ckl_sgemm."""
    sgemm(a, b, c, m, n, k, k, n, n, alpha, beta, stream)


gemm_tiled = gemm_naive
gemm_register = gemm_naive
gemm_cp_async = gemm_naive


def gemm_mma_opt_bias(a, b, c, bias, m, n, k, alpha, stream=None) -> None:
    """C = relu(alpha*A*B + bias[col]); include/ckl/gemm.hpp:91-92 of the reference."""
    _check(_lib.ckl_gemm_bias_relu_ex(F16, _ptr(a), _ptr(b), _ptr(c), F32, _ptr(bias), m, n, k, k,
                                      n, n, alpha, ALGO_AUTO, _stream(stream)))


def gemm_bias_relu_ex(ab_dtype, a, b, c, c_dtype, bias, m, n, k, lda, ldb, ldc, alpha,
                      algo=ALGO_AUTO, stream=None) -> None:
    _check(_lib.ckl_gemm_bias_relu_ex(ab_dtype, _ptr(a), _ptr(b), _ptr(c), c_dtype, _ptr(bias), m,
                                      n, k, lda, ldb, ldc, alpha, algo, _stream(stream)))


def gemm_bias_relu(c, bias, m, n, stream=None) -> None:
    """Unfused pass C = relu(C + bias[col]); include/ckl/gemm.hpp:93 of the reference."""
    _check(_lib.ckl_bias_relu_f32(_ptr(c), _ptr(bias), m, n, n, _stream(stream)))


def sgemm(a, b, c, m, n, k, lda=None, ldb=None, ldc=None, alpha=1.0, beta=0.0, stream=None) -> None:
    """FP32 C = alpha*A*B + beta*C on the CUDA cores (the reference's gemm_naive / gemm_tiled /
    gemm_register / gemm_cp_async, include/ckl/gemm.hpp:40-58)."""
    _check(_lib.ckl_sgemm(_ptr(a), _ptr(b), _ptr(c), m, n, k, k if lda is None else lda,
                          n if ldb is None else ldb, n if ldc is None else ldc, alpha, beta,
                          _stream(stream)))


def strsm_lower(l, b, m, n, lda=None, ldb=None, alpha=1.0, stream=None) -> None:
    """Solve L X = alpha B in place (L lower triangular m x m, B m x n, FP32, row-major)."""
    _check(_lib.ckl_strsm_lower(_ptr(l), _ptr(b), m, n, m if lda is None else lda,
                                n if ldb is None else ldb, alpha, _stream(stream)))


def trsm_blocked(a, b, m, n, alpha, stream=None) -> None:
    """include/ckl/trsm.hpp:19-24 of the reference: both of its rungs are the blocked solve here."""
    strsm_lower(a, b, m, n, m, n, alpha, stream)


trsm_naive = trsm_blocked


def gemm_host(ab_dtype, a_host, b_host, c_host, c_dtype, m, n, k, alpha, beta) -> None:
    """Whole call on HOST buffers (upload, GEMM, download, wait)."""
    _check(_lib.ckl_gemm_host(ab_dtype, _ptr(a_host), _ptr(b_host), _ptr(c_host), c_dtype, m, n, k,
                              alpha, beta))


def plan_gemm(m, n, k, lda=None, ldb=None, ldc=None, a_align=16, b_align=16, algo=ALGO_AUTO,
              sm_count=148) -> Plan:
    """What a call would launch on a device with ``sm_count`` SMs.  Pure host arithmetic."""
    plan = Plan()
    _check(_lib.ckl_plan_gemm(m, n, k, k if lda is None else lda, n if ldb is None else ldb,
                              n if ldc is None else ldc, a_align, b_align, algo, sm_count,
                              ctypes.byref(plan)))
    return plan


_lib.ckl_plan_gemm_ex.argtypes = [_i] * 13 + [ctypes.POINTER(Plan)]
_lib.ckl_plan_gemm_ex.restype = ctypes.c_int
_lib.ckl_last_plan.argtypes = [ctypes.POINTER(Plan)]
_lib.ckl_last_plan.restype = ctypes.c_int
_lib.ckl_debug_counter.argtypes = [ctypes.c_char_p]
_lib.ckl_debug_counter.restype = ctypes.c_ulonglong


def plan_gemm_ex(m, n, k, lda=None, ldb=None, ldc=None, a_align=16, b_align=16, algo=ALGO_AUTO,
                 sm_count=148, max_pairs=0, c_dtype=BF16, c_is_read=False) -> Plan:
    """plan_gemm with the output type, whether C is read and the resident CTA-pair count."""
    plan = Plan()
    _check(_lib.ckl_plan_gemm_ex(m, n, k, k if lda is None else lda, n if ldb is None else ldb,
                                 n if ldc is None else ldc, a_align, b_align, algo, sm_count,
                                 max_pairs, c_dtype, 1 if c_is_read else 0, ctypes.byref(plan)))
    return plan


def last_plan() -> Plan:
    """What the calling thread's last gemm call launched (on the real device)."""
    plan = Plan()
    _check(_lib.ckl_last_plan(ctypes.byref(plan)))
    return plan


_lib.ckl_test_arm_wait_fault.argtypes = [_i, ctypes.c_ulonglong]
_lib.ckl_test_arm_wait_fault.restype = ctypes.c_int


def arm_wait_fault(kind: int, wait_limit_ns: int = 0) -> None:
    """Test hook: one bounded wait of this thread's next tensor-core launch runs out
    (kind 1: a pipeline stage that never completes; kind 2: a stream-K flag nobody sets)."""
    _check(_lib.ckl_test_arm_wait_fault(kind, wait_limit_ns))


def debug_counter(name: str) -> int:
    return int(_lib.ckl_debug_counter(name.encode()))


def plan_sk_range(plan: Plan, unit: int) -> tuple[int, int]:
    b, e = ctypes.c_longlong(), ctypes.c_longlong()
    _check(_lib.ckl_plan_sk_range(ctypes.byref(plan), unit, ctypes.byref(b), ctypes.byref(e)))
    return b.value, e.value


def plan_unit_segments(plan: Plan, unit: int) -> list[tuple[int, int, int, int, int, int]]:
    """Work list of one unit: (tile, tile_row, tile_col, kb_begin, kb_end, slot) tuples."""
    count = _lib.ckl_plan_unit_segments(ctypes.byref(plan), unit, None, 0)
    if count < 0:
        raise CklError(-count, last_error())
    buf = (ctypes.c_int * (6 * max(count, 1)))()
    _lib.ckl_plan_unit_segments(ctypes.byref(plan), unit, buf, count)
    return [tuple(buf[6 * i:6 * i + 6]) for i in range(count)]


def plan_fixup_slots(plan: Plan, sk_tile: int) -> list[int]:
    """Workspace slots the fix-up pass adds for one split tile, in order."""
    buf = (ctypes.c_int * 512)()
    count = _lib.ckl_plan_fixup_slots(ctypes.byref(plan), sk_tile, buf, 512)
    if count < 0:
        raise CklError(-count, last_error())
    return list(buf[:count])


def assemble_column_blocks(dst, src, elem_size: int, m: int, n_shard: int, parts: int,
                           stream=None) -> None:
    """[parts][m][n_shard] -> row-major [m][parts*n_shard] on the device."""
    _check(_lib.ckl_assemble_column_blocks(_ptr(dst), _ptr(src), elem_size, m, n_shard, parts,
                                           _stream(stream)))


def device_status() -> list[int]:
    """Synchronise and read the device health word; raises CklError(ERR_DEVICE) if a
    kernel gave up a bounded wait."""
    info = (ctypes.c_uint * 4)()
    _check(_lib.ckl_device_status(info))
    return list(info)


def stream_copy(dst, src, nbytes: int, stream=None) -> None:
    _check(_lib.ckl_stream_copy(_ptr(dst), _ptr(src), nbytes, _stream(stream)))


# --- several GPUs of one box: communicator, host-buffer sharded GEMM, gathered GEMM -----------

COMM_ID_BYTES = 128


class HostShardPlan(ctypes.Structure):
    _fields_ = [("rows_per_rank", _i), ("row0", _i), ("rows", _i), ("panels", _i),
                ("panel_rows", _i), ("padded_rows", _i)]


_lib.ckl_column_shard.argtypes = [_i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]
_lib.ckl_plan_host_sharded.argtypes = [_i, _i, _i, ctypes.POINTER(HostShardPlan)]
_lib.ckl_comm_get_unique_id.argtypes = [_vp]
_lib.ckl_comm_init.argtypes = [ctypes.POINTER(_vp), _i, _i, _vp]
_lib.ckl_comm_world.argtypes = [_vp]
_lib.ckl_comm_rank.argtypes = [_vp]
_lib.ckl_comm_destroy.argtypes = [_vp]
_lib.ckl_comm_alloc_shared.argtypes = [_vp, ctypes.c_size_t, ctypes.POINTER(_vp)]
_lib.ckl_comm_free_shared.argtypes = [_vp, _vp]
_lib.ckl_gemm_host_sharded.argtypes = [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f]
_lib.ckl_gemm_gathered.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
_lib.ckl_scatter_column_block.argtypes = [ctypes.POINTER(_vp), _i, _vp, _i, _i, _i, _i, _i, _vp]
for _name in ("ckl_column_shard", "ckl_plan_host_sharded", "ckl_comm_get_unique_id", "ckl_comm_init",
              "ckl_comm_world", "ckl_comm_rank", "ckl_comm_destroy", "ckl_comm_alloc_shared",
              "ckl_comm_free_shared", "ckl_gemm_host_sharded", "ckl_gemm_gathered",
              "ckl_scatter_column_block"):
    getattr(_lib, _name).restype = ctypes.c_int


def column_shard(n: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """(first column, width) of rank `rank`'s column block; the C form of sharded.column_shard."""
    col0, width = _i(), _i()
    _check(_lib.ckl_column_shard(n, world, rank, align, ctypes.byref(col0), ctypes.byref(width)))
    return col0.value, width.value


def plan_host_sharded(m: int, world: int, rank: int) -> HostShardPlan:
    """Which rows of A rank `rank` uploads in gemm_host_sharded, and in how many panels."""
    plan = HostShardPlan()
    _check(_lib.ckl_plan_host_sharded(m, world, rank, ctypes.byref(plan)))
    return plan


def comm_unique_id() -> bytes:
    """Drawn on rank 0 and handed to every rank (any transport) before Comm(...)."""
    buf = ctypes.create_string_buffer(COMM_ID_BYTES)
    _check(_lib.ckl_comm_get_unique_id(buf))
    return buf.raw


class Comm:
    """The ranks of one job (one rank per GPU; the current device is the rank's).  Collective
    to create and to close."""

    def __init__(self, world: int, rank: int, unique_id: bytes | None = None):
        handle = _vp()
        uid = None
        if unique_id is not None:
            if len(unique_id) != COMM_ID_BYTES:
                raise ValueError(f"unique_id must be {COMM_ID_BYTES} bytes")
            uid = ctypes.create_string_buffer(bytes(unique_id), COMM_ID_BYTES)
        _check(_lib.ckl_comm_init(ctypes.byref(handle), world, rank, uid))
        self._h = handle
        self.world, self.rank = world, rank

    def alloc_shared(self, nbytes: int) -> int:
        """A buffer of nbytes on every rank, every copy mapped into every rank; returns this
        rank's device address.  Collective."""
        out = _vp()
        _check(_lib.ckl_comm_alloc_shared(self._h, nbytes, ctypes.byref(out)))
        return int(out.value)

    def free_shared(self, ptr: int) -> None:
        _check(_lib.ckl_comm_free_shared(self._h, ptr))

    def gemm_host_sharded(self, ab_dtype, a_rows_host, b_shard_host, c_shard_host, c_dtype, m,
                          n_shard, k, alpha, beta) -> None:
        """N-sharded GEMM on host buffers: this rank's rows of A, its blocks of B and C."""
        _check(_lib.ckl_gemm_host_sharded(self._h, ab_dtype, _ptr(a_rows_host), _ptr(b_shard_host),
                                          _ptr(c_shard_host), c_dtype, m, n_shard, k, alpha, beta))

    def gemm_gathered(self, ab_dtype, a, b_shard, c_shard, c_full, c_dtype, m, n, k, lda, ldb,
                      alpha, beta, stream=None) -> None:
        """N-sharded GEMM on device buffers; c_full (from alloc_shared) ends with the whole C on
        every rank."""
        _check(_lib.ckl_gemm_gathered(self._h, ab_dtype, _ptr(a), _ptr(b_shard), _ptr(c_shard),
                                      _ptr(c_full), c_dtype, m, n, k, lda, ldb, alpha, beta,
                                      _stream(stream)))

    def close(self) -> None:
        if self._h is not None and self._h.value:
            _check(_lib.ckl_comm_destroy(self._h))
            self._h = None


def scatter_column_block(dsts, src, elem_size: int, rows: int, width: int, n: int, col0: int,
                         stream=None) -> None:
    """Write the packed rows x width block src to columns [col0, col0 + width) of each row-major
    rows x n matrix in dsts."""
    arr = (_vp * len(dsts))(*[_ptr(d) for d in dsts])
    _check(_lib.ckl_scatter_column_block(arr, len(dsts), _ptr(src), elem_size, rows, width, n, col0,
                                         _stream(stream)))


_lib.ckl_gemm_streamk_noalloc.argtypes = [_i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]
_lib.ckl_gemm_streamk_noalloc.restype = ctypes.c_int
_lib.ckl_noalloc_last_error.restype = ctypes.c_char_p
_lib.ckl_noalloc_scratch_bytes.restype = ctypes.c_size_t


def gemm_streamk_noalloc(ab_dtype, a, b, c, c_dtype, m, n, k, lda, ldb, ldc, alpha, beta,
                         stream=None) -> None:
    """Stream-K GEMM that never allocates device memory (built-in scratch); for hosts that own
    all device memory themselves or cannot afford cudaMalloc's synchronisation.  One call at a
    time per device; make the first call before any stream capture."""
    status = _lib.ckl_gemm_streamk_noalloc(ab_dtype, _ptr(a), _ptr(b), _ptr(c), c_dtype, m, n, k,
                                           lda, ldb, ldc, alpha, beta, _stream(stream))
    if status != OK:
        raise CklError(status, _lib.ckl_noalloc_last_error().decode())


_lib.ckl_noalloc_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
_lib.ckl_noalloc_device_status.restype = ctypes.c_int


def noalloc_device_status() -> list[int]:
    """Health word of the allocation-free entry point (its kernels do not share the regular
    entry points' word); synchronises, raises CklError(ERR_DEVICE) if a wait ran out.  Allocates
    nothing."""
    info = (ctypes.c_uint * 4)()
    status = _lib.ckl_noalloc_device_status(info)
    if status != OK:
        raise CklError(status, _lib.ckl_noalloc_last_error().decode())
    return list(info)


def noalloc_scratch_bytes() -> int:
    return int(_lib.ckl_noalloc_scratch_bytes())


def shutdown() -> None:
    _lib.ckl_shutdown()
