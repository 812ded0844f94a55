"""CPU-only checks of the shipped library: it loads, exports what include/ckl_gemm.h
declares, validates arguments, refuses to compute without a GPU, and its tile schedule
(the same code the kernels execute) covers every (tile, k block) exactly once."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ckl_gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ckl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(ckl):
    lib = ctypes.CDLL(ckl.LIB_PATH)
    names = declared_symbols()
    assert "ckl_gemm_f16" in names and "ckl_gemm_bf16" in names and len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in ckl_gemm.h but not exported"


def test_reference_entry_points_are_mirrored(ckl):
    # include/ckl/gemm.hpp:68-100 of the reference: the tensor-core launchers.
    for name in ("gemm_wmma_fp16", "gemm_wmma_bf16", "gemm_mma_ptx", "gemm_mma_ldm",
                 "gemm_mma_opt", "gemm_mma_opt_bias", "gemm_bias_relu"):
        assert callable(getattr(ckl, name))
    header = open(os.path.join(ROOT, "include", "ckl", "gemm.hpp")).read()
    for name in ("gemm_wmma_fp16", "gemm_wmma_bf16", "gemm_mma_ptx", "gemm_mma_ldm", "gemm_mma_opt",
                 "gemm_mma_opt_bias", "gemm_bias_relu", "gemm_cublas_fp16", "gemm_cublas_bf16",
                 "gemm_variant_name"):
        assert re.search(rf"\b{name}\s*\(", header), name


def test_fp32_ladder_is_mirrored_and_validates(ckl):
    # include/ckl/gemm.hpp:40-58 of the reference: the four FP32 rungs.
    header = open(os.path.join(ROOT, "include", "ckl", "gemm.hpp")).read()
    for name in ("gemm_naive", "gemm_tiled", "gemm_register", "gemm_cp_async"):
        assert callable(getattr(ckl, name))
        assert re.search(rf"CKL_FP32_RUNG\({name}\)", header), name
    ckl.gemm_naive(None, None, None, 0, 128, 128, 1.25, 0.5)   # zero m: no-op, as the reference
    ckl.gemm_cp_async(None, None, None, 128, 0, 128, 1.25, 0.5)
    with pytest.raises(ckl.CklError) as e:
        ckl.sgemm(16, 16, None, 4, 4, 4)                       # C null
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.sgemm(16, 16, 16, 4, 8, 4, 4, 8, 4)                # ldc < n
    assert e.value.status == ckl.ERR_INVALID_ARG


def test_trsm_is_mirrored_and_validates(ckl):
    # include/ckl/trsm.hpp:19-24 of the reference: trsm_naive, trsm_blocked (+ the cuBLAS oracle)
    header = open(os.path.join(ROOT, "include", "ckl", "trsm.hpp")).read()
    for name in ("trsm_naive", "trsm_blocked", "trsm_cublas"):
        assert re.search(rf"\b{name}\s*\(", header), name
    for name in ("trsm_naive", "trsm_blocked"):
        assert callable(getattr(ckl, name))
    ckl.trsm_blocked(None, None, 0, 8, 1.5)          # zero m or n: no-op, as the reference
    ckl.trsm_naive(None, None, 8, 0, 1.5)
    with pytest.raises(ckl.CklError) as e:
        ckl.strsm_lower(None, 16, 4, 4)               # L null
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.strsm_lower(16, 16, 8, 4, 4, 4)           # lda < m
    assert e.value.status == ckl.ERR_INVALID_ARG


def test_argument_validation_needs_no_gpu(ckl):
    # bad dtypes / algo / leading dimension are rejected before any CUDA call
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(7, 16, 16, 16, ckl.F32, 4, 4, 4, 4, 4, 4, 1.0, 0.0)
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(ckl.F16, 16, 16, 16, 9, 4, 4, 4, 4, 4, 4, 1.0, 0.0)
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(ckl.F16, 16, 16, 16, ckl.F32, 4, 4, 4, 4, 4, 4, 1.0, 0.0, algo=99)
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(ckl.F16, 16, 16, 16, ckl.F32, 4, 8, 4, 4, 8, 4, 1.0, 0.0)  # ldc < n
    assert e.value.status == ckl.ERR_INVALID_ARG
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_ex(ckl.F16, 16, 16, None, ckl.F32, 4, 4, 4, 4, 4, 4, 1.0, 0.0)  # C null
    assert e.value.status == ckl.ERR_INVALID_ARG
    # m <= 0 or n <= 0: nothing to do, success, pointers not looked at
    # (reference: include/ckl/detail/wmma_gemm.cuh:145-147)
    ckl.gemm_wmma_fp16(None, None, None, 0, 64, 64, 1.0, 0.0)
    ckl.gemm_wmma_bf16(None, None, None, 64, 0, 128, 1.0, 0.0)


def test_no_cpu_fallback(ckl):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; this checks the behaviour of a machine without one")
    with pytest.raises(ckl.CklError) as e:
        ckl.gemm_wmma_fp16(16, 16, 16, 8, 8, 8, 1.0, 0.0)
    assert e.value.status in (ckl.ERR_CUDA, ckl.ERR_UNSUPPORTED)
    assert ckl.last_error()


def test_dispatch_follows_the_reference_contract(ckl):
    # TMA-illegal shapes go to the general kernel, like the reference's scalar fallback
    # (include/ckl/detail/wmma_gemm.cuh:148-158); legal ones to the tensor-core kernel.
    assert ckl.plan_gemm(129, 257, 193).algo == ckl.ALGO_SIMT      # lda=193, ldb=257
    assert ckl.plan_gemm(7, 5, 11).algo == ckl.ALGO_SIMT
    assert ckl.plan_gemm(256, 256, 256).algo == ckl.ALGO_UMMA_1CTA_N128    # small: 128x128 tiles
    assert ckl.plan_gemm(512, 384, 640).algo == ckl.ALGO_UMMA_1CTA_N128
    assert ckl.plan_gemm(2048, 2048, 2048).algo == ckl.ALGO_UMMA_1CTA
    assert ckl.plan_gemm(256, 256, 256, a_align=2).algo == ckl.ALGO_SIMT
    with pytest.raises(ckl.CklError) as e:
        ckl.plan_gemm(129, 257, 193, algo=ckl.ALGO_UMMA_1CTA)
    assert e.value.status == ckl.ERR_UNSUPPORTED
    # large problems: CTA pairs, 256x256 tile, 128 k per stage
    p = ckl.plan_gemm(8192, 8192, 8192)
    assert p.algo == ckl.ALGO_UMMA_2CTA_WIDE
    assert (p.tile_m, p.tile_n, p.tile_k) == (256, 512, 64)
    assert (p.tiles_m, p.tiles_n, p.k_blocks, p.grid, p.units) == (32, 16, 128, 148, 74)
    p = ckl.plan_gemm(8192, 8192, 8192, algo=ckl.ALGO_UMMA_2CTA)
    assert (p.tile_m, p.tile_n, p.tile_k) == (256, 256, 128)
    assert (p.tiles_m, p.tiles_n, p.k_blocks, p.grid, p.units) == (32, 32, 64, 148, 74)
    p = ckl.plan_gemm(8192, 8192, 8192, algo=ckl.ALGO_UMMA_1CTA)
    assert (p.tile_m, p.tile_n, p.tile_k) == (128, 256, 64)
    assert (p.tiles_m, p.tiles_n, p.k_blocks, p.grid) == (64, 32, 128, 148)
    # the skinny stream-K stress shape splits by default: 16 pair tiles, each cut at the same k
    # offsets over 4 of the 74 pairs; forcing the split works anywhere
    p = ckl.plan_gemm(1024, 1024, 32768)
    assert p.algo == ckl.ALGO_UMMA_2CTA_SK and p.sk_tiles == 16 and p.workspace_bytes > 0
    assert p.units == 64 and p.dp_tiles == 0
    assert [ckl.plan_sk_range(p, u)[0] % p.k_blocks for u in range(8)] == [0, 64, 128, 192] * 2
    # with a short k per unit the single-CTA kernel keeps the job, on 128x128 tiles because
    # 128x256 ones would fill at most half of the SMs (64 tiles x 2 CTAs)
    p = ckl.plan_gemm(1024, 1024, 8192)
    assert p.algo == ckl.ALGO_UMMA_1CTA_N128_SK and p.units == 128 and p.tile_n == 128
    # a last wave that is at most 60 % full is split too, behind whole tiles (44 tiles left for
    # 74 pairs), but only from k = 4096 on: below that the parked partials cost more than the
    # idle SMs; a remainder too thin to give every pair 2048 k of split work takes a whole
    # wave with it when two or more exist (4 + 74 tiles), and is left alone otherwise
    p = ckl.plan_gemm(4000, 3000, 5000)
    assert p.algo == ckl.ALGO_UMMA_2CTA_SK and (p.dp_tiles, p.sk_tiles, p.units) == (148, 44, 74)
    p = ckl.plan_gemm(16384, 1792, 4096)
    assert p.algo == ckl.ALGO_UMMA_2CTA_SK and (p.dp_tiles, p.sk_tiles, p.units) == (370, 78, 74)
    assert ckl.plan_gemm(2048, 2816, 4096).sk_tiles == 0
    # between k = 4096 and 8192 the wide tile needs nearly full waves (or at most two)
    assert ckl.plan_gemm(5120, 5120, 5120).algo == ckl.ALGO_UMMA_2CTA_SK
    assert ckl.plan_gemm(6144, 6144, 6144).algo == ckl.ALGO_UMMA_2CTA_WIDE
    # unaligned row pitches: the wide tile from shorter k on, when its waves fill
    assert ckl.plan_gemm(3000, 3000, 3000).algo == ckl.ALGO_UMMA_2CTA_WIDE
    assert ckl.plan_gemm(3072, 3072, 3072).algo == ckl.ALGO_UMMA_2CTA
    p = ckl.plan_gemm(4096, 4096, 2048)
    assert p.algo == ckl.ALGO_UMMA_2CTA and p.sk_tiles == 0
    # a remainder too thin to occupy the units is not folded into the only full wave
    assert ckl.plan_gemm(2048, 2816, 2048).sk_tiles == 0
    # fewer tiles than units: cut every tile only when the cut saves more than the fix-up pass costs
    assert ckl.plan_gemm(1536, 1536, 1536).sk_tiles == 0
    # whole 128x256 tiles that would fill at most half of the SMs become 128x128 ones
    p = ckl.plan_gemm(1536, 1536, 1536)
    assert p.algo == ckl.ALGO_UMMA_1CTA_N128 and (p.tile_m, p.tile_n, p.tiles_m * p.tiles_n) == (128, 128, 144)
    assert ckl.plan_gemm(1024, 1024, 1024).algo == ckl.ALGO_UMMA_1CTA_N128
    assert ckl.plan_gemm(2048, 2048, 2048).algo == ckl.ALGO_UMMA_1CTA          # 128 tiles: enough
    assert ckl.plan_gemm(512, 128, 512).algo == ckl.ALGO_UMMA_1CTA             # one tile column either way
    p = ckl.plan_gemm(256, 8192, 8192)
    assert p.sk_tiles == 32 and p.units == 64
    # from k = 4096 on the 256x512 tile takes over where its waves fill as well
    assert ckl.plan_gemm(4096, 4096, 4096).algo == ckl.ALGO_UMMA_2CTA_WIDE
    # a nearly full last wave is not
    assert ckl.plan_gemm(3072, 3072, 3072).sk_tiles == 0
    for algo in (ckl.ALGO_UMMA_SK, ckl.ALGO_UMMA_2CTA_SK, ckl.ALGO_UMMA_2CTA_WIDE_SK):
        p = ckl.plan_gemm(4000, 3000, 5000, algo=algo)
        assert p.sk_tiles > 0 and p.workspace_bytes > 0


def test_plan_sees_the_output_type_and_the_pair_count(ckl):
    """ckl_plan_gemm_ex takes what the dispatcher takes: an FP32 C that is read and written
    keeps the 256x256 tile up to k = 8192 (the 16-bit plan switches to the wide tile at 4096),
    and a device that keeps fewer CTA pairs resident gets a schedule for that many."""
    wide = ckl.plan_gemm_ex(16384, 14336, 4096, c_dtype=ckl.BF16, c_is_read=True)
    assert wide.algo == ckl.plan_gemm(16384, 14336, 4096).algo == ckl.ALGO_UMMA_2CTA_WIDE
    f32 = ckl.plan_gemm_ex(16384, 14336, 4096, c_dtype=ckl.F32, c_is_read=True)
    assert f32.algo in (ckl.ALGO_UMMA_2CTA, ckl.ALGO_UMMA_2CTA_SK) and f32.tile_n == 256
    assert ckl.plan_gemm_ex(16384, 14336, 4096, c_dtype=ckl.F32, c_is_read=False).algo == wide.algo
    assert ckl.plan_gemm_ex(16384, 14336, 8192, c_dtype=ckl.F32, c_is_read=True).tile_n == 512
    fewer = ckl.plan_gemm_ex(8192, 8192, 8192, max_pairs=66)
    assert fewer.units == 66 and fewer.grid == 132
    with pytest.raises(ckl.CklError):
        ckl.plan_gemm_ex(256, 256, 256, c_dtype=7)
    assert ckl.debug_counter("no such counter") == 2 ** 64 - 1
    assert ckl.debug_counter("tensor_map_encodes") == 0      # nothing was launched here


def test_large_unaligned_shapes_are_repacked_onto_the_tensor_path(ckl):
    """An odd leading dimension or base keeps a SMALL problem on the general kernel (one launch);
    from m*n*k = 2^28 on AUTO copies the operand to an aligned pitch and takes the tensor-core
    kernel.  Forcing a tensor-core kernel on such a shape is still refused."""
    small = ckl.plan_gemm(129, 257, 193)
    assert small.algo == ckl.ALGO_SIMT and small.repack == 0
    big = ckl.plan_gemm(4097, 4097, 4097)
    assert big.algo != ckl.ALGO_SIMT and big.repack == 1 and big.tile_m in (128, 256)
    assert ckl.plan_gemm(4096, 4096, 4096, a_align=2).repack == 1          # base off by one element
    assert ckl.plan_gemm(4096, 4096, 4096).repack == 0
    edge = ckl.plan_gemm(1000, 1001, 1003)
    assert edge.repack == 1 and edge.algo != ckl.ALGO_SIMT
    assert ckl.plan_gemm(640, 641, 643).algo == ckl.ALGO_SIMT              # 2.6e8 < 2^28
    with pytest.raises(ckl.CklError) as e:
        ckl.plan_gemm(4097, 4097, 4097, algo=ckl.ALGO_UMMA_2CTA)
    assert e.value.status == ckl.ERR_UNSUPPORTED


SHAPES = [(128, 256, 64), (256, 256, 256), (4000, 3000, 5000), (1024, 1024, 32768),
          (8192, 8192, 8192), (8192, 1024, 8192), (16384, 1792, 4096), (200, 264, 72),
          (2304, 4096, 1024), (1000, 776, 520), (128, 256, 6400), (100000, 256, 64)]
ALGOS = ["ALGO_UMMA_1CTA", "ALGO_UMMA_SK", "ALGO_UMMA_2CTA", "ALGO_UMMA_2CTA_SK",
         "ALGO_UMMA_2CTA_WIDE", "ALGO_UMMA_2CTA_WIDE_SK", "ALGO_UMMA_1CTA_N128",
         "ALGO_UMMA_1CTA_N128_SK"]


@pytest.mark.parametrize("sm_count", [148, 132, 8])
@pytest.mark.parametrize("algo_name", ALGOS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_schedule_covers_every_k_block_once(ckl, shape, algo_name, sm_count):
    m, n, k = shape
    plan = ckl.plan_gemm(m, n, k, algo=getattr(ckl, algo_name), sm_count=sm_count)
    tiles = plan.tiles_m * plan.tiles_n
    assert plan.tiles_m == -(-m // plan.tile_m) and plan.tiles_n == -(-n // plan.tile_n)
    assert plan.k_blocks == -(-k // plan.tile_k)
    assert plan.dp_tiles + plan.sk_tiles == tiles
    pair = plan.tile_m == 256
    assert plan.tile_n == (512 if "WIDE" in algo_name else 128 if "N128" in algo_name else 256)
    assert plan.grid == plan.units * (2 if pair else 1)
    assert plan.units <= (sm_count // 2 if pair else sm_count)

    covered = {}                      # tile -> list of (kb0, kb1, unit, slot)
    coords = {}
    slots_used = set()
    per_unit_iters = []
    for u in range(plan.units):
        segs = ckl.plan_unit_segments(plan, u)
        iters = 0
        partial_positions = []
        for idx, (tile, tm, tn, kb0, kb1, slot) in enumerate(segs):
            assert 0 <= tile < tiles and 0 <= kb0 < kb1 <= plan.k_blocks
            assert 0 <= tm < plan.tiles_m and 0 <= tn < plan.tiles_n
            coords.setdefault(tile, (tm, tn))
            assert coords[tile] == (tm, tn)
            whole = kb0 == 0 and kb1 == plan.k_blocks
            assert (slot == -1) == whole
            if slot >= 0:
                assert slot // 2 == u and slot not in slots_used
                assert slot * plan.tile_m * max(plan.tile_n, 256) * 4 < plan.workspace_bytes
                slots_used.add(slot)
                partial_positions.append(idx)
            covered.setdefault(tile, []).append((kb0, kb1, u, slot))
            iters += kb1 - kb0
        # partial accumulators only at the two ends of a unit's stream-K range
        sk_segs = [i for i, s in enumerate(segs) if s[0] >= plan.dp_tiles]
        for pos in partial_positions:
            assert pos in (sk_segs[0], sk_segs[-1])
        per_unit_iters.append(iters)

    assert sorted(covered) == list(range(tiles))
    assert len(set(coords.values())) == tiles          # the raster is a bijection
    for tile, parts in covered.items():
        parts.sort()
        assert parts[0][0] == 0 and parts[-1][1] == plan.k_blocks
        for (a0, a1, _, _), (b0, _, _, _) in zip(parts, parts[1:]):
            assert a1 == b0
        if tile < plan.dp_tiles:
            assert len(parts) == 1
    # balance: split work differs by at most one k block between units
    if plan.sk_tiles:
        sk = []
        for u in range(plan.units):
            b, e = ckl.plan_sk_range(plan, u)
            sk.append(e - b)
        assert sum(sk) == plan.sk_iters == plan.sk_tiles * plan.k_blocks
        assert max(sk) - min(sk) <= 1
    # fix-up lists name exactly the partial slots of each split tile, in unit order
    for t in range(plan.sk_tiles):
        expect = [slot for (_, _, _, slot) in covered[plan.dp_tiles + t] if slot >= 0]
        assert ckl.plan_fixup_slots(plan, t) == expect
        assert len(expect) != 1


def test_raster_groups_keep_a_wave_compact(ckl):
    plan = ckl.plan_gemm(8192, 8192, 8192, algo=ckl.ALGO_UMMA_1CTA)
    first_wave = [ckl.plan_unit_segments(plan, u)[0] for u in range(plan.units)]
    rows = {s[1] for s in first_wave}
    cols = {s[2] for s in first_wave}
    # 148 tiles in flight touch 16 tile rows and 10 tile columns, not a 1 x 148 strip
    assert len(rows) == plan.group_m == 16 and len(cols) <= 10


def test_cpp_headers_compile_and_link_against_the_library(tmp_path):
    """include/ckl/gemm.hpp (the reference's names as inline shims plus the additions: 16-bit C,
    leading dimensions, the N-sharded wrappers) and include/ckl/trsm.hpp compile as C++17 and
    link against libckl_gemm.so; a program that only takes addresses runs without a GPU."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = tmp_path / "use_headers.cu"
    src.write_text(r'''
#include <cstdio>
#include "ckl/gemm.hpp"
#include "ckl/trsm.hpp"
int main() {
    // instantiate every wrapper; none is called (no GPU needed)
    void (*f16)(const __half*, const __half*, float*, int, int, int, float, float, cudaStream_t) = ckl::gemm_mma_opt;
    void (*bf16)(const __nv_bfloat16*, const __nv_bfloat16*, float*, int, int, int, float, float, cudaStream_t) = ckl::gemm_wmma_bf16;
    void (*tensor)(const __nv_bfloat16*, const __nv_bfloat16*, __nv_bfloat16*, int, int, int, int, int, int, float, float,
                   cudaStream_t, int) = ckl::gemm_tensor<__nv_bfloat16, __nv_bfloat16>;
    auto host = &ckl::gemm_tensor_host_sharded<__nv_bfloat16, __nv_bfloat16>;
    auto gathered = &ckl::gemm_tensor_gathered<__half, float>;
    int col0 = -1, width = -1;
    const int rc = ckl_column_shard(14336, 8, 3, 8, &col0, &width);
    std::printf("%d %d %d %d\n", rc, col0, width, (f16 && bf16 && tensor && host && gathered) ? 1 : 0);
    return 0;
}
''')
    exe = tmp_path / "use_headers"
    pkg = os.path.join(ROOT, "cuda-kernel-library_b200")
    out = subprocess.run([nvcc, "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", os.path.join(ROOT, "include"),
                          "-o", str(exe), str(src), "-L", pkg, "-lckl_gemm", "-Xlinker", "-rpath", "-Xlinker", pkg],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and run.stdout.split() == ["0", "5376", "1792", "1"], run.stdout + run.stderr
