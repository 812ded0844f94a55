"""Launch one GEMM configuration a few times so Nsight Compute can capture it.

Counterpart of the reference's benchmarks/ncu_driver.cpp:41-97 (run one variant N times and
let `ncu --launch-skip` pick a warm launch).  Example, the capture behind the summaries in
profiles/:

    ncu --set full --clock-control none -k regex:umma_gemm_kernel -s 2 -c 1 -o prof \
        python cuda-kernel-library_b200/ncu_driver.py --m 8192 --n 8192 --k 8192 \
        --in bf16 --out bf16 --beta 0.5 --algo umma_1cta --iters 4

Prints the CUDA-event time of the last launch (never quote a time taken under ncu).
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--in", dest="in_dtype", choices=["f16", "bf16"], default="bf16")
    ap.add_argument("--out", dest="out_dtype", choices=["f32", "f16", "bf16"], default="bf16")
    ap.add_argument("--alpha", type=float, default=1.0)
    ap.add_argument("--beta", type=float, default=0.0)
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--iters", type=int, default=4)
    args = ap.parse_args()

    import torch
    spec = importlib.util.spec_from_file_location("ckl_b200", os.path.join(HERE, "__init__.py"),
                                                  submodule_search_locations=[HERE])
    ckl = importlib.util.module_from_spec(spec)
    sys.modules["ckl_b200"] = ckl
    spec.loader.exec_module(ckl)

    if args.algo == "sgemm":
        # the FP32 CUDA-core kernel behind the reference's FP32 rungs (operands are FP32)
        m, n, k = args.m, args.n, args.k
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(k, n, device="cuda")
        c = torch.randn(m, n, device="cuda")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(args.iters):
            e0.record()
            ckl.sgemm(a, b, c, m, n, k, alpha=args.alpha, beta=args.beta)
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        print(f"sgemm {m}x{n}x{k} fp32 beta={args.beta}: {ms:.4f} ms, "
              f"{2.0 * m * n * k / ms / 1e9:.2f} TFLOP/s (last of {args.iters} launches)")
        return
    if args.algo == "helpers":
        # the memory-bound helper kernels, one launch each per iteration, on matrices larger
        # than L2: m x n FP32 / BF16 with n taken from --n (bias+ReLU pass, C = beta*C, the
        # post-gather interleave, the column-block scatter to 4 local matrices, the copy to an
        # aligned pitch, the bandwidth probe)
        m, n = args.m, args.n
        c32 = torch.randn(m, n, device="cuda")
        bias = torch.randn(n, device="cuda")
        c16 = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        parts = 4
        blocks = torch.randn(parts, m, n // parts, device="cuda").to(torch.bfloat16)
        full = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        dsts = [torch.empty(m, n, device="cuda", dtype=torch.bfloat16) for _ in range(parts)]
        odd = torch.randn(m, n - 1, device="cuda").to(torch.bfloat16)          # pitch not 16-byte aligned
        even = torch.randn(n - 1, n, device="cuda").to(torch.bfloat16)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.iters):
            ckl.gemm_bias_relu(c32, bias, m, n)
            ckl.gemm_ex(ckl.BF16, c16, c16, c16, ckl.BF16, m, n, 0, 8, n, n, 1.0, 0.5)      # k = 0: C = beta*C
            ckl.assemble_column_blocks(full, blocks, 2, m, n // parts, parts)
            ckl.scatter_column_block(dsts, blocks[1], 2, m, n // parts, n, n // parts)
            ckl.gemm_ex(ckl.BF16, odd, even, out, ckl.BF16, m, n, n - 1, n - 1, n, n, 1.0, 0.0)  # copies A first
            ckl.stream_copy(full, c16, m * n * 2)
        torch.cuda.synchronize()
        ckl.device_status()
        print(f"helpers on {m} x {n}: bias_relu, scale_c, assemble_column_blocks, scatter_column_block, "
              f"copy_rows, stream_copy launched {args.iters} times each")
        return
    if args.algo == "trsm":
        # the blocked triangular solve: m x m lower triangle, n right-hand sides (k is ignored)
        m, n = args.m, args.n
        l = torch.tril(torch.randn(m, m, device="cuda")) + 4.0 * torch.eye(m, device="cuda")
        b0 = torch.randn(m, n, device="cuda")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(args.iters):
            b = b0.clone()
            e0.record()
            ckl.strsm_lower(l, b, m, n, alpha=args.alpha)
            e1.record()
        torch.cuda.synchronize()
        print(f"trsm {m}x{m}, {n} right-hand sides: {e0.elapsed_time(e1):.4f} ms "
              f"(last of {args.iters} solves)")
        return
    algos = {ckl.algo_name(i): i for i in range(ckl.NUM_ALGOS)}
    if args.algo not in algos:
        raise SystemExit(f"--algo must be one of {sorted(algos) + ['sgemm', 'trsm', 'helpers']}")
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
    cdt = {"f16": ckl.F16, "bf16": ckl.BF16, "f32": ckl.F32}
    m, n, k = args.m, args.n, args.k
    g = torch.Generator(device="cuda").manual_seed(7)
    a = (torch.randn(m, k, device="cuda", generator=g) * 0.02).to(tdt[args.in_dtype])
    b = (torch.randn(k, n, device="cuda", generator=g) * 0.02).to(tdt[args.in_dtype])
    c = (torch.randn(m, n, device="cuda", generator=g) * 0.02).to(tdt[args.out_dtype])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.iters):
        e0.record()
        ckl.gemm_ex(cdt[args.in_dtype], a, b, c, cdt[args.out_dtype], m, n, k, k, n, n, args.alpha,
                    args.beta, algos[args.algo])
        e1.record()
    torch.cuda.synchronize()
    ckl.device_status()
    ms = e0.elapsed_time(e1)
    print(f"{args.algo} {m}x{n}x{k} in={args.in_dtype} out={args.out_dtype} beta={args.beta}: "
          f"{ms:.4f} ms, {2.0 * m * n * k / ms / 1e9:.1f} TFLOP/s (last of {args.iters} launches)")


if __name__ == "__main__":
    main()
