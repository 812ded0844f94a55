"""The allocation-free stream-K entry point against the regular one.

ckl_gemm_streamk_noalloc exists for hosts that cannot let a library call cudaMalloc: they
have committed all device memory to their own arena, or they sit in a latency-critical loop
where cudaMalloc's device-wide synchronisation is not acceptable.  It keeps its partial-tile
workspace in an array built into the library instead.  This test calls it through the C ABI
twice in a row, with different inputs, so the second call runs on scratch that still holds the
first call's partial tiles, and compares each result with ckl_gemm_ex(CKL_ALGO_UMMA_SK) under
the parity tolerance used throughout the GPU tests (relative Frobenius <= 1e-3, max error
<= 2e-2*sqrt(K/4096)*max|C|).  It is collected last on purpose: a failure here cannot hide
the results of the other tests in a run that stops at the first failure.
"""

import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _compare(ckl, orc, got, want, k, cdt, label):
    def host(t):
        if cdt == ckl.F32:
            return t.cpu().numpy()
        return orc.widen(t.view(torch.int16).cpu().numpy().view(np.uint16), cdt)

    g, w = host(got), host(want).astype(np.float64)
    rel = orc.relative_frobenius_error(g, w)
    scale = float(np.abs(w).max())
    mx = float(np.abs(g.astype(np.float64) - w).max())
    print(f"  {label}: rel_frob={rel:.3e} max_err/max|C|={mx / scale:.3e}")
    assert rel <= 1e-3, (label, rel)
    assert mx <= 2e-2 * math.sqrt(k / 4096.0) * scale, (label, mx, scale)


def test_noalloc_entry_matches_regular_entry_twice(ckl, orc):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    assert ckl.noalloc_scratch_bytes() == 2 * 148 * 128 * 256 * 4
    tdt = {ckl.F32: torch.float32, ckl.F16: torch.float16, ckl.BF16: torch.bfloat16}
    # two calls in a row; every tile of both shapes is split, so both use the scratch
    calls = [
        (1024, 1024, 4096, ckl.BF16, ckl.BF16, 1.0, 0.5, 11),
        (1000, 776, 2056, ckl.F16, ckl.F32, 1.25, 0.0, 12),
    ]
    for m, n, k, dt, cdt, alpha, beta, seed in calls:
        assert ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK).sk_tiles > 0
        a = torch.from_numpy(orc.narrow(orc.random_matrix(m, k, seed), dt).view(np.int16)) \
            .view(tdt[dt]).cuda()
        b = torch.from_numpy(orc.narrow(orc.random_matrix(k, n, seed + 100), dt).view(np.int16)) \
            .view(tdt[dt]).cuda()
        c0 = torch.from_numpy(orc.random_matrix(m, n, seed + 200)).cuda().to(tdt[cdt])
        want = c0.clone()
        ckl.gemm_ex(dt, a, b, want, cdt, m, n, k, k, n, n, alpha, beta, ckl.ALGO_UMMA_SK)
        got = c0.clone()
        ckl.gemm_streamk_noalloc(dt, a, b, got, cdt, m, n, k, k, n, n, alpha, beta)
        torch.cuda.synchronize()
        ckl.device_status()
        _compare(ckl, orc, got, want, k, cdt, f"{m}x{n}x{k}")
    # One full wave of whole tiles plus a split remainder: the regular entry point adds the
    # partials inside the GEMM kernel (the unit holding a tile's first k blocks does it), this one
    # in the separate fix-up pass.  Both add in ascending unit order: the bits must agree.
    m, n, k = 2048, 2816, 2048
    plan = ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK)
    assert plan.sk_tiles > 0 and plan.dp_tiles >= plan.units
    a = torch.from_numpy(orc.narrow(orc.random_matrix(m, k, 31), ckl.BF16).view(np.int16)) \
        .view(torch.bfloat16).cuda()
    b = torch.from_numpy(orc.narrow(orc.random_matrix(k, n, 32), ckl.BF16).view(np.int16)) \
        .view(torch.bfloat16).cuda()
    c0 = torch.from_numpy(orc.random_matrix(m, n, 33)).cuda()
    want, got = c0.clone(), c0.clone()
    ckl.gemm_ex(ckl.BF16, a, b, want, ckl.F32, m, n, k, k, n, n, 1.0, 0.5, ckl.ALGO_UMMA_SK)
    ckl.gemm_streamk_noalloc(ckl.BF16, a, b, got, ckl.F32, m, n, k, k, n, n, 1.0, 0.5)
    torch.cuda.synchronize()
    ckl.device_status()
    assert torch.equal(got, want)
    _compare(ckl, orc, got, want, k, ckl.F32, f"{m}x{n}x{k}")
    # shapes the tensor-core kernel cannot take are refused, not computed some other way
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_streamk_noalloc(ckl.F16, a, b, got, ckl.F32, 129, 257, 193, 193, 257, 257, 1.0, 0.0)
    assert e.value.status == ckl.ERR_UNSUPPORTED
