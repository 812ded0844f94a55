"""The multi-GPU entry points of the C ABI on ONE GPU (world size 1, and the copy kernel with
several local destinations standing in for peers): the host-buffer sharded GEMM and the
gathered GEMM against the CPU oracle under the parity tolerance of the GEMM tests (relative
Frobenius <= 1e-3, max error <= 2e-2*sqrt(K/4096)*max|C|), the column-block copy bit for bit.
World sizes above 1 are exercised by bench.py --gpus N, which checks every rank's gathered and
end-to-end results against the single-GPU kernel on the same inputs."""

import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm(ckl):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    torch.cuda.set_device(0)
    c = ckl.Comm(1, 0, None)
    yield c
    c.close()


def _gate(orc, got_f32, ref64, k, label):
    rel = orc.relative_frobenius_error(got_f32, ref64)
    scale = float(np.abs(ref64).max())
    mx = float(np.abs(got_f32.astype(np.float64) - ref64).max())
    print(f"  {label}: rel_frob={rel:.3e} max_err/max|C|={mx / scale:.3e}")
    assert rel <= 1e-3, (label, rel)
    assert mx <= 2e-2 * math.sqrt(k / 4096.0) * scale, (label, mx, scale)


@pytest.mark.parametrize("shape,dt_name,beta", [((1000, 776, 520), "F16", 0.5),
                                                ((2048, 1024, 1024), "BF16", 0.0),
                                                ((4096, 512, 2048), "BF16", 0.5),
                                                ((300, 256, 0), "F16", 0.5)])
def test_host_sharded_world1_matches_oracle(ckl, orc, comm, shape, dt_name, beta):
    m, n, k = shape
    dt = getattr(ckl, dt_name)
    tdt = torch.float16 if dt == ckl.F16 else torch.bfloat16
    abits = orc.narrow(orc.random_matrix(m, max(k, 1), 0x1111 + m), dt)[:, :k]
    bbits = orc.narrow(orc.random_matrix(max(k, 1), n, 0x2222 + n), dt)[:k]
    c_in = orc.random_matrix(m, n, 0x9ABC + k)
    a_host = torch.from_numpy(np.ascontiguousarray(abits).view(np.int16)).view(tdt).pin_memory()
    b_host = torch.from_numpy(np.ascontiguousarray(bbits).view(np.int16)).view(tdt).pin_memory()
    c_host = torch.from_numpy(c_in.copy()).pin_memory()
    plan = ckl.plan_host_sharded(m, 1, 0)
    assert (plan.row0, plan.rows) == (0, m)
    for _ in range(2):                       # the second call reuses the staging buffers
        c_host.copy_(torch.from_numpy(c_in))
        comm.gemm_host_sharded(dt, a_host, b_host, c_host, ckl.F32, m, n, k, 1.0, beta)
    ckl.device_status()
    if k == 0:
        assert np.array_equal(c_host.numpy(), np.float32(beta) * c_in)
        return
    ref, _ = orc.gemm_reference_mt(orc.widen(np.ascontiguousarray(abits), dt),
                                   orc.widen(np.ascontiguousarray(bbits), dt),
                                   c_in if beta != 0.0 else None, 1.0, beta)
    _gate(orc, c_host.numpy(), ref, k, f"host_sharded {m}x{n}x{k}")
    # same bits as the single-GPU host entry point fed the same buffers
    c_one = torch.from_numpy(c_in.copy()).pin_memory()
    ckl.gemm_host(dt, a_host, b_host, c_one, ckl.F32, m, n, k, 1.0, beta)
    _gate(orc, c_one.numpy(), ref, k, f"gemm_host {m}x{n}x{k}")


def test_gathered_world1_matches_oracle(ckl, orc, comm):
    m, n, k = 4096, 1024, 1024
    abits = orc.narrow(orc.random_matrix(m, k, 71), ckl.BF16)
    bbits = orc.narrow(orc.random_matrix(k, n, 72), ckl.BF16)
    c_in = orc.random_matrix(m, n, 73)
    a = torch.from_numpy(abits.view(np.int16)).view(torch.bfloat16).cuda()
    b = torch.from_numpy(bbits.view(np.int16)).view(torch.bfloat16).cuda()
    c_shard = torch.from_numpy(c_in).cuda()
    full = comm.alloc_shared(m * n * 4)
    try:
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream()
        comm.gemm_gathered(ckl.BF16, a, b, c_shard, full, ckl.F32, m, n, k, k, n, 1.0, 0.5, stream)
        out = torch.empty(m, n, dtype=torch.float32, device="cuda")
        ckl.stream_copy(out, full, m * n * 4, stream)     # ordered behind the call on `stream`
        torch.cuda.synchronize()
        ckl.device_status()
        assert torch.equal(out, c_shard)
        ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.BF16), orc.widen(bbits, ckl.BF16), c_in, 1.0, 0.5)
        _gate(orc, out.cpu().numpy(), ref, k, f"gathered {m}x{n}x{k}")
        with pytest.raises(ckl.CklError):                 # not a shared buffer of this communicator
            comm.gemm_gathered(ckl.BF16, a, b, c_shard, out, ckl.F32, m, n, k, k, n, 1.0, 0.5, stream)
    finally:
        comm.free_shared(full)


@pytest.mark.parametrize("dtype,width,n,col0", [(torch.bfloat16, 1024, 4096, 2048),
                                                (torch.float32, 20, 100, 60),
                                                (torch.float16, 7, 21, 14),
                                                (torch.bfloat16, 1792, 14336, 1792 * 3)])
def test_scatter_column_block_to_many_destinations(ckl, dtype, width, n, col0):
    """Four local matrices stand in for the ranks' copies of C: each must receive the block
    at the rank's column offset and keep every other element."""
    rows, parts = 300, 4
    src = torch.randn(rows, width, device="cuda").to(dtype)
    dsts = [torch.full((rows, n), float(i + 1), device="cuda", dtype=dtype) for i in range(parts)]
    ckl.scatter_column_block(dsts, src, src.element_size(), rows, width, n, col0)
    torch.cuda.synchronize()
    for i, d in enumerate(dsts):
        assert torch.equal(d[:, col0:col0 + width], src)
        keep = torch.ones(n, dtype=torch.bool, device="cuda")
        keep[col0:col0 + width] = False
        assert bool((d[:, keep] == float(i + 1)).all())
    with pytest.raises(ckl.CklError):
        ckl.scatter_column_block(dsts, src, src.element_size(), rows, width, n, n - width + 1)
