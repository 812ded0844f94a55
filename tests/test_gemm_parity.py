"""GPU parity of the tensor-core GEMM against the CPU oracle, through the C ABI.

Tolerance (the one stated for this path): relative Frobenius error <= 1e-3 and maximum
elementwise error <= 2e-2 * sqrt(K / 4096) * max|C|, against the reference's CPU GEMM
(double accumulate) on IDENTICAL inputs, i.e. the oracle is fed the FP16/BF16-rounded values
the kernel sees, widened to float.  A 16-bit C is compared with the oracle's C rounded to the
same type (output quantisation alone is 2e-4 for FP16 and 1.7e-3 for BF16, so an unrounded
oracle cannot be met at 1e-3 by any correct BF16-output kernel); the unrounded figure is
printed beside it.

torch only owns device memory here; every product call goes through ckl_* in
libckl_gemm.so.
"""

import math
import os
import subprocess

import numpy as np
import pytest

from conftest import dropin_binary

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL_FROB_GATE = 1e-3


def max_gate(k):
    return 2e-2 * math.sqrt(max(k, 1) / 4096.0)


# ---------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------

class Env:
    def __init__(self, ckl, oracle_mod, orc):
        self.ckl, self.om, self.orc = ckl, oracle_mod, orc
        self.tdt = {ckl.F32: torch.float32, ckl.F16: torch.float16, ckl.BF16: torch.bfloat16}

    def to_dev16(self, bits, dt):
        t = torch.from_numpy(bits.view(np.int16)).view(self.tdt[dt])
        return t.cuda()

    def narrow_dev(self, x, dt):
        """float32 host matrix -> (device 16-bit tensor, the float32 values it holds)."""
        bits = self.orc.narrow(x, dt)
        return self.to_dev16(bits, dt), self.orc.widen(bits, dt)

    def c_to_host(self, c, cdt):
        """Device C -> float32 host array (exact widening for 16-bit types)."""
        if cdt == self.ckl.F32:
            return c.cpu().numpy()
        bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
        return self.orc.widen(bits, cdt)

    def round_ref(self, ref64, cdt):
        if cdt == self.ckl.F32:
            return ref64
        return self.orc.round_through(ref64.astype(np.float32), cdt).astype(np.float64)

    def gate(self, got_f32, ref64, k, cdt, label=""):
        target = self.round_ref(ref64, cdt)
        rel = self.orc.relative_frobenius_error(got_f32, target)
        raw = self.orc.relative_frobenius_error(got_f32, ref64)
        scale = float(np.abs(ref64).max()) if ref64.size else 0.0
        mx = float(np.abs(got_f32.astype(np.float64) - target).max()) if ref64.size else 0.0
        print(f"  {label} rel_frob={rel:.3e} (vs unrounded oracle {raw:.3e}) "
              f"max_err/max|C|={mx / scale if scale else 0.0:.3e}")
        assert rel <= REL_FROB_GATE, (label, rel)
        if scale > 0:
            assert mx <= max_gate(k) * scale, (label, mx, scale)
        return rel


@pytest.fixture(scope="module")
def env(ckl, oracle_mod, orc):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    major, _ = torch.cuda.get_device_capability(0)
    assert major == 10, "this library targets sm_100a (B200)"
    return Env(ckl, oracle_mod, orc)


@pytest.fixture(autouse=True)
def device_healthy(ckl):
    yield
    ckl.device_status()      # raises if a kernel gave up a bounded wait


REF_SHAPES = [  # tests/test_gemm_tensor.cpp:105-110 of the reference
    (256, 256, 256), (384, 512, 128), (129, 257, 193), (7, 5, 11), (512, 384, 640),
    (64, 0, 128), (64, 64, 0),
]
ENTRY_POINTS = [  # tests/test_gemm_tensor.cpp:115-130 of the reference
    ("fp16", "gemm_wmma_fp16", "F16"), ("bf16", "gemm_wmma_bf16", "BF16"),
    ("ptx", "gemm_mma_ptx", "F16"), ("ldm", "gemm_mma_ldm", "F16"), ("opt", "gemm_mma_opt", "F16"),
]


# ---------------------------------------------------------------------------------------
# the reference's own test matrix, CPU oracle as ground truth
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("entry", ENTRY_POINTS, ids=lambda e: e[0])
@pytest.mark.parametrize("shape", REF_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_reference_shapes(env, shape, entry):
    m, n, k = shape
    _, fn_name, dt_name = entry
    ckl, orc = env.ckl, env.orc
    dt = getattr(ckl, dt_name)
    fa = orc.random_matrix(m, k, 0x1111 + m)      # seeds: tests/test_gemm_tensor.cpp:62-63
    fb = orc.random_matrix(k, n, 0x2222 + n)
    da, ra = env.narrow_dev(fa, dt)
    db, rb = env.narrow_dev(fb, dt)
    c = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    getattr(ckl, fn_name)(da, db, c, m, n, k, 1.0, 0.0)
    torch.cuda.synchronize()
    got = c.cpu().numpy()
    if m * n == 0:
        return
    ref, _ = orc.gemm_reference_mt(ra, rb, None, 1.0, 0.0)
    env.gate(got, ref, k, ckl.F32, f"{fn_name} {m}x{n}x{k}")
    # the figure the reference prints as vs_fp32 (unrounded inputs, not gated there;
    # docs/gemm.md:45-48 puts it at 2.6e-4 for FP16 and 2.1e-3 for BF16)
    raw_ref, _ = orc.gemm_reference_mt(fa, fb, None, 1.0, 0.0)
    if k > 0:
        vs_fp32 = orc.relative_frobenius_error(got, raw_ref)
        assert vs_fp32 <= (2e-3 if dt == ckl.F16 else 1e-2)
        # and the reference's own gate against its oracle (5e-2) holds with huge margin
        assert vs_fp32 < 5e-2


def test_empty_contraction_scales_c(env):
    # k == 0: C = beta * C (include/ckl/detail/wmma_gemm.cuh:133-139 of the reference)
    ckl = env.ckl
    for cdt in (ckl.F32, ckl.F16, ckl.BF16):
        c0 = (torch.rand(64, 64, device="cuda") * 2 - 1).to(env.tdt[cdt])
        for beta in (0.0, 0.5):
            c = c0.clone()
            ckl.gemm_ex(ckl.F16, None, None, c, cdt, 64, 64, 0, 0, 64, 64, 1.0, beta)
            expect = (beta * c0.float()).to(env.tdt[cdt])
            assert torch.equal(c, expect)
    # m == 0 / n == 0: nothing is written
    c = torch.full((4, 4), 7.0, device="cuda")
    ckl.gemm_wmma_fp16(c, c, c, 0, 4, 4, 1.0, 0.0)
    ckl.gemm_wmma_fp16(c, c, c, 4, 0, 4, 1.0, 0.0)
    assert torch.all(c == 7.0)


def test_beta_zero_does_not_read_c(env):
    ckl, orc = env.ckl, env.orc
    m, n, k = 256, 512, 128
    da, ra = env.narrow_dev(orc.random_matrix(m, k, 1), ckl.F16)
    db, rb = env.narrow_dev(orc.random_matrix(k, n, 2), ckl.F16)
    for algo in (ckl.ALGO_SIMT, ckl.ALGO_UMMA_1CTA, ckl.ALGO_UMMA_2CTA, ckl.ALGO_UMMA_2CTA_WIDE):
        c = torch.full((m, n), float("nan"), device="cuda")
        ckl.gemm_ex(ckl.F16, da, db, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0, algo)
        assert not torch.isnan(c).any()


# ---------------------------------------------------------------------------------------
# every kernel, every output type, alpha / beta, ragged shapes
# ---------------------------------------------------------------------------------------

ALGO_NAMES = ["ALGO_SIMT", "ALGO_UMMA_1CTA", "ALGO_UMMA_SK", "ALGO_UMMA_2CTA", "ALGO_UMMA_2CTA_SK",
              "ALGO_UMMA_2CTA_WIDE", "ALGO_UMMA_2CTA_WIDE_SK", "ALGO_UMMA_1CTA_N128",
              "ALGO_UMMA_1CTA_N128_SK"]
RAGGED = [(128, 256, 64), (200, 264, 72), (1000, 776, 520), (130, 8, 8), (1, 2048, 4096),
          (513, 1032, 1000), (2304, 1280, 2048)]


@pytest.mark.parametrize("algo_name", ALGO_NAMES)
@pytest.mark.parametrize("shape", RAGGED, ids=lambda s: "x".join(map(str, s)))
def test_kernels_output_types_alpha_beta(env, shape, algo_name):
    m, n, k = shape
    ckl, orc = env.ckl, env.orc
    algo = getattr(ckl, algo_name)
    cases = [(ckl.F16, ckl.F32, 1.0, 0.0), (ckl.BF16, ckl.BF16, 1.0, 0.5),
             (ckl.F16, ckl.F16, 1.25, 0.5), (ckl.BF16, ckl.F32, -0.75, 1.0)]
    fa = orc.random_matrix(m, k, 0x1111 + m)
    fb = orc.random_matrix(k, n, 0x2222 + n)
    fc = orc.random_matrix(m, n, 0x9ABC + k)
    for dt, cdt, alpha, beta in cases:
        da, ra = env.narrow_dev(fa, dt)
        db, rb = env.narrow_dev(fb, dt)
        if cdt == ckl.F32:
            dc, rc = torch.from_numpy(fc).cuda(), fc
        else:
            dc, rc = env.narrow_dev(fc, cdt)
        ckl.gemm_ex(dt, da, db, dc, cdt, m, n, k, k, n, n, alpha, beta, algo)
        torch.cuda.synchronize()
        ref, _ = orc.gemm_reference_mt(ra, rb, rc, alpha, beta)
        env.gate(env.c_to_host(dc, cdt), ref, k, cdt,
                 f"{algo_name} {m}x{n}x{k} in={dt} out={cdt} a={alpha} b={beta}")


def test_results_are_deterministic(env):
    ckl, orc = env.ckl, env.orc
    m, n, k = 4000, 3000, 1000
    da, _ = env.narrow_dev(orc.random_matrix(m, k, 3), ckl.F16)
    db, _ = env.narrow_dev(orc.random_matrix(k, n, 4), ckl.F16)
    for algo in (ckl.ALGO_AUTO, ckl.ALGO_UMMA_SK, ckl.ALGO_UMMA_2CTA_SK, ckl.ALGO_UMMA_2CTA_WIDE_SK):
        outs = []
        for _ in range(3):
            c = torch.zeros(m, n, device="cuda")
            ckl.gemm_ex(ckl.F16, da, db, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0, algo)
            outs.append(c)
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_leading_dimensions_and_virtual_sharding(env):
    """Column blocks of a wider B and C (ld > width): P shards computed one after another on
    one GPU assemble to exactly the unsharded result."""
    ckl, orc = env.ckl, env.orc
    m, n, k, parts = 512, 2048, 384, 4
    da, ra = env.narrow_dev(orc.random_matrix(m, k, 5), ckl.BF16)
    db, rb = env.narrow_dev(orc.random_matrix(k, n, 6), ckl.BF16)
    dc0, rc = env.narrow_dev(orc.random_matrix(m, n, 7), ckl.BF16)
    whole = dc0.clone()
    ckl.gemm_ex(ckl.BF16, da, db, whole, ckl.BF16, m, n, k, k, n, n, 1.0, 0.5, ckl.ALGO_UMMA_1CTA)
    sharded = dc0.clone()
    w = n // parts
    esz = 2
    for r in range(parts):
        ckl.gemm_ex(ckl.BF16, da, db.data_ptr() + r * w * esz, sharded.data_ptr() + r * w * esz,
                    ckl.BF16, m, w, k, k, n, n, 1.0, 0.5, ckl.ALGO_UMMA_1CTA)
    torch.cuda.synchronize()
    assert torch.equal(whole, sharded)
    ref, _ = orc.gemm_reference_mt(ra, rb, rc, 1.0, 0.5)
    env.gate(env.c_to_host(whole, ckl.BF16), ref, k, ckl.BF16, "ld>width")
    # a padded C (ldc > n) leaves the padding untouched
    cpad = torch.full((m, n + 24), 3.0, device="cuda")
    ckl.gemm_ex(ckl.BF16, da, db, cpad, ckl.F32, m, n, k, k, n, n + 24, 1.0, 0.0)
    torch.cuda.synchronize()
    assert torch.all(cpad[:, n:] == 3.0)
    env.gate(cpad[:, :n].contiguous().cpu().numpy(),
             orc.gemm_reference_mt(ra, rb, None, 1.0, 0.0)[0], k, ckl.F32, "ldc>n")


def test_misaligned_pointers_take_the_general_kernel(env):
    ckl, orc = env.ckl, env.orc
    m, n, k = 96, 136, 200
    fa, fb = orc.random_matrix(m, k, 8), orc.random_matrix(k, n, 9)
    abits, bbits = orc.narrow(fa, ckl.F16), orc.narrow(fb, ckl.F16)
    # place A and B one element past a 16-byte boundary
    abuf = torch.zeros(m * k + 8, dtype=torch.float16, device="cuda")
    bbuf = torch.zeros(k * n + 8, dtype=torch.float16, device="cuda")
    abuf[1:1 + m * k] = env.to_dev16(abits, ckl.F16).reshape(-1)
    bbuf[1:1 + k * n] = env.to_dev16(bbits, ckl.F16).reshape(-1)
    c = torch.zeros(m, n, device="cuda")
    ckl.gemm_wmma_fp16(abuf.data_ptr() + 2, bbuf.data_ptr() + 2, c, m, n, k, 1.0, 0.0)
    torch.cuda.synchronize()
    ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.F16), orc.widen(bbits, ckl.F16), None, 1.0,
                                   0.0)
    env.gate(c.cpu().numpy(), ref, k, ckl.F32, "misaligned")
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(ckl.F16, abuf.data_ptr() + 2, bbuf.data_ptr() + 2, c, ckl.F32, m, n, k, k, n,
                    n, 1.0, 0.0, ckl.ALGO_UMMA_1CTA)
    assert e.value.status == ckl.ERR_UNSUPPORTED


# ---------------------------------------------------------------------------------------
# the benchmark configurations at full size: sampled exact oracle + checksum identity
# ---------------------------------------------------------------------------------------

def _sample_indices(size, count, tile, seed):
    rng = np.random.default_rng(seed)
    fixed = {0, size - 1, min(tile - 1, size - 1), min(tile, size - 1), (size // tile) * tile - 1,
             min((size // tile) * tile, size - 1)}
    fixed = {i for i in fixed if 0 <= i < size}
    extra = rng.choice(size, size=min(size, count), replace=False).tolist()
    out = sorted(fixed)
    for i in extra:
        if len(out) >= max(count, len(fixed)):
            break
        if i not in fixed:
            out.append(i)
    return np.array(sorted(out), dtype=np.int32)


def _run_large(env, m, n, k, dt, cdt, alpha, beta, dist, n_rows, n_cols, algo=None):
    ckl, orc, om = env.ckl, env.orc, env.om
    rng = np.random.default_rng(0x1111 + m + n + k)
    if dist == "uniform":
        fa = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        fb = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        fc = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    elif dist == "normal002":
        fa = (rng.standard_normal((m, k)) * 0.02).astype(np.float32)
        fb = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        fc = (rng.standard_normal((m, n)) * 0.02).astype(np.float32)
    else:  # mlp: activations N(0,1), weights N(0,1)/sqrt(K)
        fa = rng.standard_normal((m, k)).astype(np.float32)
        fb = (rng.standard_normal((k, n)) / math.sqrt(k)).astype(np.float32)
        fc = np.zeros((m, n), np.float32)
    da, ra = env.narrow_dev(fa, dt)
    db, rb = env.narrow_dev(fb, dt)
    if cdt == ckl.F32:
        dc, rc = torch.from_numpy(fc).cuda(), fc
    else:
        dc, rc = env.narrow_dev(fc, cdt)
    ckl.gemm_ex(dt, da, db, dc, cdt, m, n, k, k, n, n, alpha, beta,
                ckl.ALGO_AUTO if algo is None else algo)
    torch.cuda.synchronize()
    got = env.c_to_host(dc, cdt)

    rows = _sample_indices(m, n_rows, 128, 1)
    cols = _sample_indices(n, n_cols, 256, 2)
    r_ref, c_ref = orc.gemm_sampled(ra, rb, rc, alpha, beta, rows, cols)
    env.gate(got[rows, :], r_ref, k, cdt, f"{m}x{n}x{k} rows")
    env.gate(np.ascontiguousarray(got[:, cols].T), c_ref, k, cdt, f"{m}x{n}x{k} cols")

    # whole-matrix property: row and column sums of C equal those of the exact product
    rs, cs = om.checksum_identity(ra, rb, rc if beta != 0.0 else None, alpha, beta)
    g64 = dc.double() if cdt == ckl.F32 else dc.float().double()
    got_rs = g64.sum(dim=1).cpu().numpy()
    got_cs = g64.sum(dim=0).cpu().numpy()
    abs_row = g64.abs().sum(dim=1).cpu().numpy()
    abs_col = g64.abs().sum(dim=0).cpu().numpy()
    l2_row = g64.pow(2).sum(dim=1).sqrt().cpu().numpy()
    l2_col = g64.pow(2).sum(dim=0).sqrt().cpu().numpy()
    # Output rounding errors are independent with |e| <= eps/2 * |c|: their sum stays within
    # a few eps * ||c||_2; FP32 accumulation may add a small one-sided drift, allowed as
    # 2^-16 of the absolute sum.  One wrong 8-column group in a row breaks this.
    eps = {ckl.F32: 2.0 ** -23, ckl.F16: 2.0 ** -10, ckl.BF16: 2.0 ** -7}[cdt]
    assert np.all(np.abs(got_rs - rs) <= 8 * eps * l2_row + 2.0 ** -16 * abs_row + 1e-9)
    assert np.all(np.abs(got_cs - cs) <= 8 * eps * l2_col + 2.0 ** -16 * abs_col + 1e-9)


def test_config_fp16_4096_cubed(env):
    _run_large(env, 4096, 4096, 4096, env.ckl.F16, env.ckl.F16, 1.0, 0.0, "uniform", 12, 12)


def test_config_bf16_8192_cubed_beta(env):
    _run_large(env, 8192, 8192, 8192, env.ckl.BF16, env.ckl.BF16, 1.0, 0.5, "normal002", 8, 8)


def test_config_bf16_8192_cubed_pair_kernel(env):
    _run_large(env, 8192, 8192, 8192, env.ckl.BF16, env.ckl.BF16, 1.0, 0.5, "normal002", 6, 6,
               algo=env.ckl.ALGO_UMMA_2CTA)


def test_config_bf16_8192_cubed_single_cta_kernel(env):
    _run_large(env, 8192, 8192, 8192, env.ckl.BF16, env.ckl.F32, 1.0, 0.0, "normal002", 6, 6,
               algo=env.ckl.ALGO_UMMA_SK)


@pytest.mark.parametrize("algo_name", ["ALGO_AUTO", "ALGO_UMMA_SK", "ALGO_UMMA_2CTA_SK",
                                       "ALGO_UMMA_2CTA_WIDE_SK"])
def test_config_streamk_ragged(env, algo_name):
    algo = getattr(env.ckl, algo_name)
    if algo != env.ckl.ALGO_AUTO:
        assert env.ckl.plan_gemm(4000, 3000, 5000, algo=algo).sk_tiles > 0
    _run_large(env, 4000, 3000, 5000, env.ckl.F16, env.ckl.F16, 1.0, 0.0, "uniform", 12, 12,
               algo=algo)


def test_config_streamk_skinny(env):
    assert env.ckl.plan_gemm(1024, 1024, 32768).sk_tiles > 0
    _run_large(env, 1024, 1024, 32768, env.ckl.F16, env.ckl.F16, 1.0, 0.0, "uniform", 10, 10)


def test_config_mlp_shard(env):
    # one rank's share of M=16384, K=4096, N=14336 split over 8 GPUs: 1792 columns
    _run_large(env, 16384, 1792, 4096, env.ckl.BF16, env.ckl.BF16, 1.0, 0.0, "mlp", 6, 4)


def test_config_mlp_whole(env):
    # the same MLP-shaped problem unsharded on one GPU: M=16384, K=4096, N=14336
    _run_large(env, 16384, 14336, 4096, env.ckl.BF16, env.ckl.BF16, 1.0, 0.0, "mlp", 4, 4)


# ---------------------------------------------------------------------------------------
# neighbours of the path: fused epilogue, host-buffer call, column-block assembly
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(256, 384, 192), (300, 200, 104), (129, 257, 193)],
                         ids=lambda s: "x".join(map(str, s)))
def test_bias_relu_fused_and_unfused(env, shape):
    m, n, k = shape
    ckl, orc = env.ckl, env.orc
    da, ra = env.narrow_dev(orc.random_matrix(m, k, 21), ckl.F16)
    db, rb = env.narrow_dev(orc.random_matrix(k, n, 22), ckl.F16)
    bias = orc.random_matrix(1, n, 23).ravel()
    dbias = torch.from_numpy(bias).cuda()
    ref = orc.gemm_reference_mt(ra, rb, None, 1.0, 0.0)[0] + bias[None, :].astype(np.float64)
    ref = np.maximum(ref, 0.0)
    fused = torch.full((m, n), float("nan"), device="cuda")
    ckl.gemm_mma_opt_bias(da, db, fused, dbias, m, n, k, 1.0)
    unfused = torch.zeros(m, n, device="cuda")
    ckl.gemm_mma_opt(da, db, unfused, m, n, k, 1.0, 0.0)
    ckl.gemm_bias_relu(unfused, dbias, m, n)
    torch.cuda.synchronize()
    env.gate(fused.cpu().numpy(), ref, k, ckl.F32, "fused bias+relu")
    env.gate(unfused.cpu().numpy(), ref, k, ckl.F32, "unfused bias+relu")


def test_host_buffer_call(env):
    ckl, orc = env.ckl, env.orc
    m, n, k = 640, 512, 448
    abits = orc.narrow(orc.random_matrix(m, k, 31), ckl.BF16)
    bbits = orc.narrow(orc.random_matrix(k, n, 32), ckl.BF16)
    cbits = orc.narrow(orc.random_matrix(m, n, 33), ckl.BF16)
    ha = torch.from_numpy(abits.view(np.int16)).pin_memory()
    hb = torch.from_numpy(bbits.view(np.int16)).pin_memory()
    hc = torch.from_numpy(cbits.view(np.int16).copy()).pin_memory()
    ckl.gemm_host(ckl.BF16, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), ckl.BF16, m, n, k, 1.0, 0.5)
    got = orc.widen(hc.numpy().view(np.uint16), ckl.BF16)
    ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.BF16), orc.widen(bbits, ckl.BF16),
                                   orc.widen(cbits, ckl.BF16), 1.0, 0.5)
    env.gate(got, ref, k, ckl.BF16, "host buffers")


def test_host_buffer_call_in_row_panels(env):
    """Large enough that the host call travels in several row panels (ragged last one): the
    result must equal what one device-buffer call on the same inputs gives."""
    ckl, orc = env.ckl, env.orc
    m, n, k = 3300, 768, 512
    abits = orc.narrow(orc.random_matrix(m, k, 41), ckl.F16)
    bbits = orc.narrow(orc.random_matrix(k, n, 42), ckl.F16)
    c0 = orc.random_matrix(m, n, 43)
    ha = torch.from_numpy(abits.view(np.int16)).pin_memory()
    hb = torch.from_numpy(bbits.view(np.int16)).pin_memory()
    hc = torch.from_numpy(c0.copy()).pin_memory()
    ckl.gemm_host(ckl.F16, ha.data_ptr(), hb.data_ptr(), hc.data_ptr(), ckl.F32, m, n, k, 1.25, -0.5)
    da, db = env.to_dev16(abits, ckl.F16), env.to_dev16(bbits, ckl.F16)
    dc = torch.from_numpy(c0).cuda()
    ckl.gemm_ex(ckl.F16, da, db, dc, ckl.F32, m, n, k, k, n, n, 1.25, -0.5)
    torch.cuda.synchronize()
    ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.F16), orc.widen(bbits, ckl.F16), c0, 1.25, -0.5)
    env.gate(hc.numpy(), ref, k, ckl.F32, "host buffers, 3 panels")
    assert orc.relative_frobenius_error(hc.numpy(), dc.cpu().numpy().astype(np.float64)) < 1e-6


def test_assemble_column_blocks(env):
    ckl = env.ckl
    for dtype, width in [(torch.bfloat16, 1024), (torch.float32, 20), (torch.float16, 7)]:
        parts, m = 4, 96
        src = torch.randn(parts, m, width, device="cuda").to(dtype)
        dst = torch.zeros(m, parts * width, device="cuda", dtype=dtype)
        ckl.assemble_column_blocks(dst, src, src.element_size(), m, width, parts)
        torch.cuda.synchronize()
        assert torch.equal(dst, src.permute(1, 0, 2).reshape(m, parts * width))


@pytest.mark.parametrize("shape", [(1000, 1001, 1003), (1024, 1001, 1024), (1000, 1024, 1003),
                                   (2049, 2055, 517)], ids=lambda s: "x".join(map(str, s)))
def test_unaligned_operands_are_repacked_and_match_the_oracle(env, shape):
    """Leading dimensions that are not multiples of 8 (and, in the last pass, bases that are not
    16-byte aligned) on problems large enough for the repack path: the tensor-core kernel runs
    on aligned copies, C keeps its own odd pitch, and the result meets the oracle."""
    m, n, k = shape
    ckl, orc = env.ckl, env.orc
    fa = orc.random_matrix(m, k, 0x1111 + m)
    fb = orc.random_matrix(k, n, 0x2222 + n)
    fc = orc.random_matrix(m, n, 0x9ABC + k)
    for dt, cdt, alpha, beta in [(ckl.F16, ckl.F32, 1.0, 0.0), (ckl.BF16, ckl.BF16, 1.0, 0.5)]:
        da, ra = env.narrow_dev(fa, dt)
        db, rb = env.narrow_dev(fb, dt)
        if cdt == ckl.F32:
            dc, rc = torch.from_numpy(fc).cuda(), fc
        else:
            dc, rc = env.narrow_dev(fc, cdt)
        ckl.gemm_ex(dt, da, db, dc, cdt, m, n, k, k, n, n, alpha, beta)
        torch.cuda.synchronize()
        plan = ckl.last_plan()
        assert plan.repack == 1 and plan.algo != ckl.ALGO_SIMT
        ref, _ = orc.gemm_reference_mt(ra, rb, rc, alpha, beta)
        env.gate(env.c_to_host(dc, cdt), ref, k, cdt, f"repack {m}x{n}x{k} in={dt} out={cdt}")
    # the same through bases that sit one element past a 16-byte boundary
    dt = ckl.F16
    da, ra = env.narrow_dev(fa, dt)
    db, rb = env.narrow_dev(fb, dt)
    pad_a = torch.zeros(m * k + 1, dtype=torch.float16, device="cuda")
    pad_b = torch.zeros(k * n + 1, dtype=torch.float16, device="cuda")
    pad_a[1:].copy_(da.reshape(-1))
    pad_b[1:].copy_(db.reshape(-1))
    dc = torch.zeros(m, n, device="cuda")
    ckl.gemm_ex(dt, pad_a.data_ptr() + 2, pad_b.data_ptr() + 2, dc, ckl.F32, m, n, k, k, n, n, 1.0, 0.0)
    torch.cuda.synchronize()
    assert ckl.last_plan().repack == 1
    ref, _ = orc.gemm_reference_mt(ra, rb, None, 1.0, 0.0)
    env.gate(dc.cpu().numpy(), ref, k, ckl.F32, f"repack, odd bases {m}x{n}x{k}")


def test_unaligned_c_alone_is_staged_and_neighbours_are_untouched(env):
    """A and B legal, C with an odd pitch (a view of a wider matrix): the result is written
    through an aligned copy and copied out; the column beside the view keeps its contents."""
    ckl, orc = env.ckl, env.orc
    m, n, k, ldc = 1024, 1000, 1024, 1001
    fa = orc.random_matrix(m, k, 0x1111 + m)
    fb = orc.random_matrix(k, n, 0x2222 + n)
    fc = orc.random_matrix(m, n, 0x9ABC + k)
    for dt, cdt, tdt, beta in [(ckl.BF16, ckl.BF16, torch.bfloat16, 0.5), (ckl.F16, ckl.F32, torch.float32, 1.0),
                               (ckl.F16, ckl.F16, torch.float16, 0.0)]:
        da, ra = env.narrow_dev(fa, dt)
        db, rb = env.narrow_dev(fb, dt)
        wide = torch.full((m, ldc), 7.0, device="cuda", dtype=tdt)
        if cdt == ckl.F32:
            rc = fc
            wide[:, :n] = torch.from_numpy(fc).cuda()
        else:
            dc, rc = env.narrow_dev(fc, cdt)
            wide[:, :n] = dc
        ckl.gemm_ex(dt, da, db, wide, cdt, m, n, k, k, n, ldc, 1.0, beta)
        torch.cuda.synchronize()
        assert ckl.last_plan().repack == 1
        assert bool((wide[:, n] == 7.0).all())
        ref, _ = orc.gemm_reference_mt(ra, rb, rc if beta != 0.0 else None, 1.0, beta)
        env.gate(env.c_to_host(wide[:, :n].contiguous(), cdt), ref, k, cdt, f"staged C out={cdt} beta={beta}")


def test_descriptors_are_cached_and_the_plan_is_reported(env):
    """A repeated call encodes no TMA descriptor (they are cached per device by address, shape,
    pitch, type and box), a call on other buffers encodes its own, and ckl_last_plan reports
    what was launched: the same plan ckl_plan_gemm_ex gives for the C type and beta used."""
    ckl = env.ckl
    m = n = k = 512
    a = torch.randn(m, k, device="cuda").half()
    b = torch.randn(k, n, device="cuda").half()
    c = torch.zeros(m, n, device="cuda")
    ckl.gemm_ex(ckl.F16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0)
    first = ckl.debug_counter("tensor_map_encodes")
    want = c.clone()
    for _ in range(5):
        ckl.gemm_ex(ckl.F16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0)
    assert ckl.debug_counter("tensor_map_encodes") == first
    torch.cuda.synchronize()
    assert torch.equal(c, want)
    c2 = torch.zeros(m, n, device="cuda")
    ckl.gemm_ex(ckl.F16, a, b, c2, ckl.F32, m, n, k, k, n, n, 1.0, 0.0)
    assert ckl.debug_counter("tensor_map_encodes") == first + 1      # only C's descriptor is new
    torch.cuda.synchronize()
    assert torch.equal(c2, want)
    # more distinct buffers than cache entries: entries are replaced, results stay right
    outs = [torch.zeros(m, n, device="cuda") for _ in range(60)]
    for o in outs:
        ckl.gemm_ex(ckl.F16, a, b, o, ckl.F32, m, n, k, k, n, n, 1.0, 0.0)
    torch.cuda.synchronize()
    assert all(torch.equal(o, want) for o in outs)
    # the reported plan is the launched one, FP32 C with beta != 0 included
    mm, nn, kk = 2048, 4096, 4096
    a = torch.randn(mm, kk, device="cuda").bfloat16()
    b = torch.randn(kk, nn, device="cuda").bfloat16()
    c = torch.zeros(mm, nn, device="cuda")
    ckl.gemm_ex(ckl.BF16, a, b, c, ckl.F32, mm, nn, kk, kk, nn, nn, 1.0, 0.5)
    got = ckl.last_plan()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    want_plan = ckl.plan_gemm_ex(mm, nn, kk, sm_count=sms, max_pairs=got.units if got.tile_m == 256 else 0,
                                 c_dtype=ckl.F32, c_is_read=True)
    assert (got.algo, got.tile_n, got.sk_tiles) == (want_plan.algo, want_plan.tile_n, want_plan.sk_tiles)
    assert got.tile_n == 256          # FP32 C read and written at k = 4096: not the wide tile
    torch.cuda.synchronize()


def test_reference_test_driver_runs_unchanged(env):
    """The reference's own tests/test_gemm_tensor.cpp, compiled without edits against this
    repository's include/ckl headers and library (oracle/Makefile target `dropin`), passes."""
    exe = dropin_binary("test_gemm_tensor_dropin")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "all tensor GEMM cases passed" in out.stdout


def test_reference_bench_driver_runs_unchanged(env):
    """The reference's benchmarks/bench_gemm_tensor.cpp, compiled without edits against this
    repository's headers and library, runs its five entry points at 512^3 and prints one row
    per entry point with a positive rate."""
    exe = dropin_binary("bench_gemm_tensor_dropin")
    out = subprocess.run([exe, "512"], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    rows = [ln.split() for ln in out.stdout.splitlines() if "gflops" in ln]
    assert [r[0] for r in rows] == ["fp16", "bf16", "ptx", "ldm", "opt"]
    for r in rows:
        assert r[1] == "512" and float(r[3]) > 0.0


def test_reference_fusion_study_runs_unchanged(env):
    """The reference's benchmarks/fusion_study.cpp (fused bias+ReLU epilogue against GEMM plus a
    separate pass), compiled without edits against this repository's headers and library."""
    exe = dropin_binary("fusion_study_dropin")
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]


def test_split_schedule_survives_graph_replay(env):
    """A launch whose last wave is split, captured into a CUDA graph and replayed: every replay
    must give what the same sequence of direct calls gives (C feeds back through beta, so a
    replay that consumed stale partial tiles would show)."""
    ckl = env.ckl
    m, n, k = 2048, 2816, 2048          # 176 single-CTA tiles: one whole wave + 28 split tiles
    plan = ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK)
    assert plan.sk_tiles > 0 and plan.dp_tiles >= plan.units
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.05).bfloat16()
    b = (torch.randn(k, n, device="cuda", generator=g) * 0.05).bfloat16()
    c0 = torch.randn(m, n, device="cuda", generator=g)
    want = c0.clone()
    for _ in range(3):
        ckl.gemm_ex(ckl.BF16, a, b, want, ckl.F32, m, n, k, k, n, n, 1.0, 0.25, ckl.ALGO_UMMA_SK)
    torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    got = c0.clone()
    scratch = c0.clone()
    with torch.cuda.stream(stream):     # first call on this stream allocates its workspace
        ckl.gemm_ex(ckl.BF16, a, b, scratch, ckl.F32, m, n, k, k, n, n, 1.0, 0.25, ckl.ALGO_UMMA_SK,
                    stream.cuda_stream)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        ckl.gemm_ex(ckl.BF16, a, b, got, ckl.F32, m, n, k, k, n, n, 1.0, 0.25, ckl.ALGO_UMMA_SK,
                    stream.cuda_stream)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(got, want)


_FORMS_SCRIPT = r"""
import hashlib, importlib.util, os, sys
import torch
root = sys.argv[1]
spec = importlib.util.spec_from_file_location("ckl_b200", os.path.join(root, "cuda-kernel-library_b200", "__init__.py"))
ckl = importlib.util.module_from_spec(spec); spec.loader.exec_module(ckl)
g = torch.Generator(device="cuda").manual_seed(9)
for algo, (m, n, k) in [(ckl.ALGO_UMMA_SK, (2048, 2816, 2048)), (ckl.ALGO_UMMA_2CTA_SK, (4000, 3000, 5000)),
                        (ckl.ALGO_UMMA_2CTA_WIDE_SK, (4000, 3000, 5000))]:
    plan = ckl.plan_gemm(m, n, k, algo=algo)
    assert plan.sk_tiles > 0 and plan.dp_tiles >= plan.units, (algo, plan.dp_tiles, plan.sk_tiles)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.05).half()
    b = (torch.randn(k, n, device="cuda", generator=g) * 0.05).half()
    c = torch.randn(m, n, device="cuda", generator=g).half()
    for _ in range(2):
        ckl.gemm_ex(ckl.F16, a, b, c, ckl.F16, m, n, k, k, n, n, 1.0, 0.5, algo)
    torch.cuda.synchronize()
    ckl.device_status()
    print(algo, hashlib.sha256(c.cpu().numpy().tobytes()).hexdigest())
"""


def test_fused_and_two_kernel_split_give_the_same_bits(env):
    """Split schedules with whole tiles behind them, all three tile shapes: the fused form (the
    holder of a tile's first k blocks adds the parked partials) and the two-kernel form
    (CKL_STREAMK_FIXUP=pass) must agree bit for bit.  The form is chosen once per process, so
    each runs in its own."""
    import sys
    outs = []
    for form in ("", "pass"):
        child_env = dict(os.environ, CKL_STREAMK_FIXUP=form)
        run = subprocess.run([sys.executable, "-c", _FORMS_SCRIPT, ROOT], capture_output=True, text=True,
                             timeout=600, env=child_env)
        assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
        outs.append(run.stdout.strip().splitlines())
    assert len(outs[0]) == 3 and outs[0] == outs[1]
