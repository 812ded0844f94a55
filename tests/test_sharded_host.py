"""Multi-GPU host logic on CPU ranks (gloo, world size 2): column-shard arithmetic, the
local-GEMM call each rank makes, the all-gather and the column-block assembly, and the row
dealing of the host-buffer entry point (each rank uploads its own rows of A, the ranks
all-gather them panel by panel).  The CUDA kernels are replaced by host stand-ins here; the
GPU tests cover the real ones."""

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _load_sharded():
    import importlib.util
    path = os.path.join(ROOT, "cuda-kernel-library_b200", "sharded.py")
    spec = importlib.util.spec_from_file_location("ckl_b200_sharded", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ckl_b200_sharded"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_column_shard_arithmetic():
    sh = _load_sharded()
    for n, world in [(8192, 8), (14336, 8), (8192, 2), (3000, 4), (5, 8), (0, 2), (1000, 3)]:
        shards = [sh.column_shard(n, world, r) for r in range(world)]
        assert sum(s.width for s in shards) == n
        pos = 0
        for s in shards:
            assert s.col0 == pos or s.width == 0
            assert s.col0 % 8 == 0 or s.width == 0
            pos += s.width
        assert all(s.width == shards[0].width for s in shards) == sh.even_shards(n, world) or n == 0
    assert sh.column_shard(14336, 8, 3).width == 1792 and sh.column_shard(8192, 8, 7).col0 == 7168
    with pytest.raises(ValueError):
        sh.column_shard(10, 2, 2)


def test_c_abi_column_shard_matches_python(ckl):
    sh = _load_sharded()
    for n, world in [(8192, 8), (14336, 8), (8192, 2), (3000, 4), (5, 8), (0, 2), (1000, 3)]:
        for r in range(world):
            s = sh.column_shard(n, world, r)
            assert ckl.column_shard(n, world, r) == (s.col0, s.width)
    with pytest.raises(ckl.CklError):
        ckl.column_shard(10, 2, 2)


def _device_rows(plan_of, world):
    """Global row held at each row position of the device layout [panel][rank][panel_rows] of
    ckl_gemm_host_sharded (-1 = padding), from the plans of all ranks."""
    p0 = plan_of(0)
    rows = np.full(p0.padded_rows, -1, dtype=np.int64)
    for r in range(world):
        p = plan_of(r)
        for j in range(p.panels):
            have = max(0, min(p.panel_rows, p.rows - j * p.panel_rows))
            base = (j * world + r) * p.panel_rows
            rows[base:base + have] = p.row0 + j * p.panel_rows + np.arange(have)
    return rows


def test_host_shard_plan_deals_every_row_once(ckl):
    for m, world in [(8192, 8), (8192, 1), (8192, 2), (16384, 8), (1000, 3), (7, 4), (129, 2),
                     (4000, 8), (1, 1), (0, 2)]:
        plans = [ckl.plan_host_sharded(m, world, r) for r in range(world)]
        assert sum(p.rows for p in plans) == m
        pos = 0
        for p in plans:
            assert p.rows == 0 or p.row0 == pos
            pos += p.rows
            assert p.rows <= p.rows_per_rank <= p.panels * p.panel_rows or m == 0
            assert p.panel_rows % 8 == 0 and 0 <= p.panels <= 8
            assert p.padded_rows == p.panels * world * p.panel_rows
            assert (p.rows_per_rank, p.panels, p.panel_rows) == \
                   (plans[0].rows_per_rank, plans[0].panels, plans[0].panel_rows)
        rows = _device_rows(lambda r: plans[r], world)
        assert sorted(rows[rows >= 0].tolist()) == list(range(m))
    assert ckl.plan_host_sharded(8192, 8, 3).rows == 1024
    assert ckl.plan_host_sharded(8192, 8, 3).panels == 8 and ckl.plan_host_sharded(8192, 8, 3).panel_rows == 128
    with pytest.raises(ckl.CklError):
        ckl.plan_host_sharded(8, 2, 2)


def _host_sharded_worker(rank, world, port, m, n, k, tmpdir):
    """Stand-in for ckl_gemm_host_sharded with the SAME row dealing (the plan comes from the C
    ABI): every rank holds only its rows of A, the row panels are all-gathered (gloo in place
    of NCCL) into the [panel][rank][panel_rows] layout, each panel is multiplied by a host
    GEMM, and the rank's column block of C is read back from that layout."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from conftest import load_package
        ckl = load_package()
        sh = _load_sharded()
        g = torch.Generator().manual_seed(3)
        a = torch.randn(m, k, generator=g)
        b = torch.randn(k, n, generator=g)
        c_in = torch.randn(m, n, generator=g)
        plan = ckl.plan_host_sharded(m, world, rank)
        shard = sh.column_shard(n, world, rank)
        a_rows = a[plan.row0:plan.row0 + plan.rows].contiguous()     # all this rank has of A
        b_shard = b[:, shard.col0:shard.col0 + shard.width].contiguous()
        c_shard = c_in[:, shard.col0:shard.col0 + shard.width].contiguous()
        pr = plan.panel_rows
        dev_a = torch.zeros(plan.padded_rows, k)
        for j in range(plan.panels):
            have = max(0, min(pr, plan.rows - j * pr))
            mine = torch.zeros(pr, k)
            mine[:have] = a_rows[j * pr:j * pr + have]
            block = dev_a[j * world * pr:(j + 1) * world * pr]
            dist.all_gather_into_tensor(block, mine)
        rows = _device_rows(lambda r: ckl.plan_host_sharded(m, world, r), world)
        valid = torch.from_numpy(rows >= 0)
        src = torch.from_numpy(rows[rows >= 0])
        dev_c = torch.zeros(plan.padded_rows, shard.width)
        dev_c[valid] = c_shard[src]                                  # upload of C_in
        for j in range(plan.panels):
            sl = slice(j * world * pr, (j + 1) * world * pr)
            dev_c[sl] = dev_a[sl] @ b_shard + 0.5 * dev_c[sl]
        out = torch.empty(m, shard.width)
        out[src] = dev_c[valid]                                      # download
        expect = (a @ b + 0.5 * c_in)[:, shard.col0:shard.col0 + shard.width]
        ok = torch.allclose(out, expect, rtol=1e-5, atol=1e-5) and torch.equal(dev_a[valid], a[src])
        np.save(os.path.join(tmpdir, f"hs{rank}.npy"), np.array([ok, plan.rows, plan.panels]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [512, 301])
def test_two_rank_host_sharded_row_dealing(tmp_path, m):
    world, n, k = 2, 64, 40
    port = 31500 + (os.getpid() % 2000) + m % 7
    mp.spawn(_host_sharded_worker, args=(world, port, m, n, k, str(tmp_path)), nprocs=world, join=True)
    got = [np.load(tmp_path / f"hs{r}.npy") for r in range(world)]
    assert all(g[0] == 1 for g in got)
    assert sum(int(g[1]) for g in got) == m


def _worker(rank, world, port, m, n, k, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = _load_sharded()
        g = torch.Generator().manual_seed(1)          # same A, B, C_in on every rank
        a = torch.randn(m, k, generator=g)
        b = torch.randn(k, n, generator=g)
        c_in = torch.randn(m, n, generator=g)
        calls = []

        def host_gemm(a_, b_, c_, lda, ldb, ldc, alpha, beta, algo, stream):
            calls.append((lda, ldb, ldc))
            c_.copy_(alpha * (a_ @ b_) + beta * c_)

        def host_assemble(dst, src, elem_size, rows, width, parts, stream):
            assert src.shape == (parts, rows, width) and elem_size == 4
            dst.copy_(src.permute(1, 0, 2).reshape(rows, parts * width))

        op = sh.ShardedGemm(None, m, n, k, 1, 0, world, rank, local_gemm=host_gemm,
                            assemble=host_assemble)
        s = op.shard
        b_shard = b[:, s.col0:s.col0 + s.width].contiguous()
        c_shard = c_in[:, s.col0:s.col0 + s.width].contiguous()
        op.run(a, b_shard, c_shard, 1.0, 0.5)
        assert calls == [(k, s.width, s.width)]
        staging = torch.empty(world, m, s.width)
        full = torch.empty(m, n)
        op.gather(c_shard, staging, full)
        expect = a @ b + 0.5 * c_in
        ok = torch.allclose(full, expect, rtol=1e-5, atol=1e-5)
        np.save(os.path.join(tmpdir, f"ok{rank}.npy"), np.array([ok, s.col0, s.width]))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_gemm_and_gather(tmp_path):
    world, m, n, k = 2, 48, 64, 40
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, m, n, k, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok, col0, width = np.load(tmp_path / f"ok{r}.npy")
        assert ok == 1 and col0 == r * 32 and width == 32


def test_gather_refuses_uneven_shards():
    sh = _load_sharded()
    op = sh.ShardedGemm(None, 8, 1000, 8, 1, 0, 3, 0, local_gemm=lambda *a: None,
                        assemble=lambda *a: None)
    with pytest.raises(ValueError):
        op.gather(torch.zeros(8, op.shard.width), None, None)


def test_communicator_validates_before_it_touches_a_device(ckl):
    """Bad arguments are refused by the C ABI without a GPU; a well-formed request on a machine
    without one fails with a CUDA error instead of pretending."""
    with pytest.raises(ckl.CklError) as e:
        ckl.Comm(0, 0, None)
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.Comm(2, 2, bytes(ckl.COMM_ID_BYTES))
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.Comm(2, 0, None)                      # several ranks need the shared id
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        ckl.Comm(2, 0, b"short")
    if not torch.cuda.is_available():
        with pytest.raises(ckl.CklError) as e:
            ckl.Comm(1, 0, None)
        assert e.value.status in (ckl.ERR_CUDA, ckl.ERR_UNSUPPORTED)
        with pytest.raises(ckl.CklError):
            ckl.scatter_column_block([1 << 20], 1 << 21, 2, 4, 8, 8, 4)   # col0 + width > n
