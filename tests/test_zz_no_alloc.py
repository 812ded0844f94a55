"""The allocation-free stream-K entry point against the CPU oracle and the regular entry point.

ckl_gemm_streamk_noalloc exists for hosts that cannot let a library call cudaMalloc: they
have committed all device memory to their own arena, or they sit in a latency-critical loop
where cudaMalloc's device-wide synchronisation is not acceptable.  It keeps its partial-tile
workspace in an array built into the library instead.  The first test calls it through the C
ABI twice in a row, with different inputs, so the second call runs on scratch that still holds
the first call's partial tiles.  Each result is gated against the CPU oracle under the parity
tolerance used throughout the GPU tests (relative Frobenius <= 1e-3, max error
<= 2e-2*sqrt(K/4096)*max|C|) and, as a second assertion, must carry the same bits as
ckl_gemm_ex(CKL_ALGO_UMMA_SK).  The second test runs the entry point alone in a fresh process
(no other entry point before it) and checks that no device memory disappears across calls.
This file is collected last on purpose: a failure here cannot hide the results of the other
tests in a run that stops at the first failure.
"""

import math
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _host(ckl, orc, t, cdt):
    if cdt == ckl.F32:
        return t.cpu().numpy()
    return orc.widen(t.view(torch.int16).cpu().numpy().view(np.uint16), cdt)


def _gate(ckl, orc, got, ref64, k, cdt, label):
    """got (device tensor) against the oracle's float64 result rounded to the output type."""
    g = _host(ckl, orc, got, cdt)
    target = ref64 if cdt == ckl.F32 else \
        orc.round_through(ref64.astype(np.float32), cdt).astype(np.float64)
    rel = orc.relative_frobenius_error(g, target)
    scale = float(np.abs(ref64).max())
    mx = float(np.abs(g.astype(np.float64) - target).max())
    print(f"  {label}: rel_frob={rel:.3e} max_err/max|C|={mx / scale:.3e}")
    assert rel <= 1e-3, (label, rel)
    assert mx <= 2e-2 * math.sqrt(k / 4096.0) * scale, (label, mx, scale)


def _inputs(ckl, orc, m, n, k, dt, cdt, seed):
    tdt = {ckl.F32: torch.float32, ckl.F16: torch.float16, ckl.BF16: torch.bfloat16}
    abits = orc.narrow(orc.random_matrix(m, k, seed), dt)
    bbits = orc.narrow(orc.random_matrix(k, n, seed + 100), dt)
    a = torch.from_numpy(abits.view(np.int16)).view(tdt[dt]).cuda()
    b = torch.from_numpy(bbits.view(np.int16)).view(tdt[dt]).cuda()
    c0 = torch.from_numpy(orc.random_matrix(m, n, seed + 200)).cuda().to(tdt[cdt])
    return a, b, c0, orc.widen(abits, dt), orc.widen(bbits, dt), _host(ckl, orc, c0, cdt)


def test_noalloc_entry_matches_regular_entry_twice(ckl, orc):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    assert ckl.noalloc_scratch_bytes() == 2 * 148 * 128 * 256 * 4
    # two calls in a row; every tile of both shapes is split, so both use the scratch
    calls = [
        (1024, 1024, 4096, ckl.BF16, ckl.BF16, 1.0, 0.5, 11),
        (1000, 776, 2056, ckl.F16, ckl.F32, 1.25, 0.0, 12),
    ]
    for m, n, k, dt, cdt, alpha, beta, seed in calls:
        assert ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK).sk_tiles > 0
        a, b, c0, ra, rb, rc = _inputs(ckl, orc, m, n, k, dt, cdt, seed)
        got = c0.clone()
        ckl.gemm_streamk_noalloc(dt, a, b, got, cdt, m, n, k, k, n, n, alpha, beta)
        assert ckl.noalloc_device_status() == [0, 0, 0, 0]
        ref, _ = orc.gemm_reference_mt(ra, rb, rc if beta != 0.0 else None, alpha, beta)
        _gate(ckl, orc, got, ref, k, cdt, f"{m}x{n}x{k} vs oracle")
        want = c0.clone()
        ckl.gemm_ex(dt, a, b, want, cdt, m, n, k, k, n, n, alpha, beta, ckl.ALGO_UMMA_SK)
        torch.cuda.synchronize()
        ckl.device_status()
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    # One full wave of whole tiles plus a split remainder: the regular entry point adds the
    # partials inside the GEMM kernel (the unit holding a tile's first k blocks does it), this one
    # in the separate fix-up pass.  Both add in ascending unit order: the bits must agree.
    m, n, k = 2048, 2816, 2048
    plan = ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK)
    assert plan.sk_tiles > 0 and plan.dp_tiles >= plan.units
    a, b, c0, ra, rb, rc = _inputs(ckl, orc, m, n, k, ckl.BF16, ckl.F32, 31)
    want, got = c0.clone(), c0.clone()
    ckl.gemm_streamk_noalloc(ckl.BF16, a, b, got, ckl.F32, m, n, k, k, n, n, 1.0, 0.5)
    assert ckl.noalloc_device_status() == [0, 0, 0, 0]
    ckl.gemm_ex(ckl.BF16, a, b, want, ckl.F32, m, n, k, k, n, n, 1.0, 0.5, ckl.ALGO_UMMA_SK)
    torch.cuda.synchronize()
    ckl.device_status()
    ref, _ = orc.gemm_reference_mt(ra, rb, rc, 1.0, 0.5)
    _gate(ckl, orc, got, ref, k, ckl.F32, f"{m}x{n}x{k} vs oracle")
    assert torch.equal(got, want)
    # shapes the tensor-core kernel cannot take are refused, not computed some other way
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_streamk_noalloc(ckl.F16, a, b, got, ckl.F32, 129, 257, 193, 193, 257, 257, 1.0, 0.0)
    assert e.value.status == ckl.ERR_UNSUPPORTED
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_streamk_noalloc(ckl.BF16, a, b, got, ckl.F32, 128, 256, 0, 8, 256, 256, 1.0, 0.0)
    assert e.value.status == ckl.ERR_UNSUPPORTED


_ALONE = r"""
import math, os, sys
import numpy as np
import torch
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
from conftest import load_package
import oracle
ckl, orc = load_package(), oracle.Oracle()
torch.cuda.set_device(0)
m, n, k = 1024, 1024, 4096
abits = orc.narrow(orc.random_matrix(m, k, 51), ckl.BF16)
bbits = orc.narrow(orc.random_matrix(k, n, 52), ckl.BF16)
a = torch.from_numpy(abits.view(np.int16)).view(torch.bfloat16).cuda()
b = torch.from_numpy(bbits.view(np.int16)).view(torch.bfloat16).cuda()
c_in = orc.random_matrix(m, n, 53)
outs = [torch.from_numpy(c_in).cuda() for _ in range(3)]
torch.cuda.synchronize()
# first call: one-time set-up and the load of the library's device code (built-in scratch)
ckl.gemm_streamk_noalloc(ckl.BF16, a, b, outs[0], ckl.F32, m, n, k, k, n, n, 1.0, 0.5)
assert ckl.noalloc_device_status() == [0, 0, 0, 0]
free_before, _ = torch.cuda.mem_get_info()
for c in outs[1:]:
    ckl.gemm_streamk_noalloc(ckl.BF16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.5)
assert ckl.noalloc_device_status() == [0, 0, 0, 0]
free_after, _ = torch.cuda.mem_get_info()
assert free_after == free_before, (free_before, free_after)
ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.BF16), orc.widen(bbits, ckl.BF16), c_in, 1.0, 0.5)
scale = float(np.abs(ref).max())
for c in outs:
    g = c.cpu().numpy()
    rel = orc.relative_frobenius_error(g, ref)
    mx = float(np.abs(g.astype(np.float64) - ref).max())
    assert rel <= 1e-3 and mx <= 2e-2 * math.sqrt(k / 4096.0) * scale, (rel, mx, scale)
print("noalloc alone ok: rel_frob=%.3e free=%d" % (rel, free_after))
"""


def test_noalloc_entry_alone_in_a_fresh_process_keeps_free_memory():
    """Only ckl_gemm_streamk_noalloc and its status reader are called in the child process, so
    its own set-up (not the regular entry points') raises the kernels' shared-memory limit; after
    the first call the device's free memory must not move, and every result meets the oracle."""
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    out = subprocess.run([sys.executable, "-c", f"ROOT = {ROOT!r}\n" + _ALONE], capture_output=True,
                         text=True, timeout=600)
    print(out.stdout[-2000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "noalloc alone ok" in out.stdout
