"""Multi-GPU host logic on CPU ranks (gloo, world size 2): column-shard arithmetic, the
local-GEMM call each rank makes, the all-gather and the column-block assembly.  The CUDA
kernels are replaced by host stand-ins here; the GPU tests cover the real ones."""

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
