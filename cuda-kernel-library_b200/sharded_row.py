"""One row of the sweep for an N-sharded GEMM on several GPUs (run under torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        cuda-kernel-library_b200/sharded_row.py <variant> <dtype> <m> <n> <k> [commit]

The single-GPU rows come from the C++ tool bench_all; the reference has no multi-GPU row
(it never leaves one device), so this one follows the same protocol
(include/ckl/event_timer.hpp:28-71 of the reference: 5 warm-ups, 20 launches timed one by one
with CUDA events, median and inter-quartile range) on every rank, for the rank's column block
(B and C sharded by columns, A replicated, no collective), and takes the maximum over ranks
per launch.  Rank 0 prints the row; `gpus` is the world size and the rate is the whole job's.
dtype is fp16 | bf16 (FP32 C) or fp16_c16 | bf16_c16, as in bench_all.
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def load(name: str, path: str, search=None):
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=search)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    if len(sys.argv) < 6:
        raise SystemExit("usage: sharded_row.py <variant> <dtype> <m> <n> <k> [commit]")
    variant, dtype = sys.argv[1], sys.argv[2]
    m, n, k = (int(x) for x in sys.argv[3:6])
    commit = sys.argv[6] if len(sys.argv) > 6 else "unknown"
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ckl = load("ckl_b200", os.path.join(HERE, "__init__.py"), [HERE])
    sharded = load("ckl_b200_sharded", os.path.join(HERE, "sharded.py"))
    algos = {ckl.algo_name(i): i for i in range(ckl.NUM_ALGOS)}
    bf16 = dtype.startswith("bf16")
    if variant not in algos or not (bf16 or dtype.startswith("fp16")):
        raise SystemExit(f"unknown variant {variant} or dtype {dtype}")
    in_t, in_c = (torch.bfloat16, ckl.BF16) if bf16 else (torch.float16, ckl.F16)
    out_t, out_c = (in_t, in_c) if dtype.endswith("_c16") else (torch.float32, ckl.F32)
    op = sharded.ShardedGemm(ckl, m, n, k, in_c, out_c, world, rank)
    w = op.shard.width
    g = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(in_t)
    b = (torch.rand(k, max(w, 1), device="cuda", generator=g) * 2 - 1).to(in_t)
    c = torch.zeros(m, max(w, 1), device="cuda", dtype=out_t)
    stream = torch.cuda.current_stream()
    for _ in range(5):
        op.run(a, b, c, 1.0, 0.0, algo=algos[variant], stream=stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(20)]
    for e0, e1 in events:
        e0.record(stream)
        op.run(a, b, c, 1.0, 0.0, algo=algos[variant], stream=stream)
        e1.record(stream)
    torch.cuda.synchronize()
    ckl.device_status()
    times = torch.tensor([e0.elapsed_time(e1) for e0, e1 in events], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ts = sorted(times.tolist())
    median = 0.5 * (ts[9] + ts[10])
    iqr = ts[15] - ts[5]
    gflops = 2.0 * m * n * k / (median * 1e6)
    if rank == 0:
        print(json.dumps({"family": "gemm", "variant": variant, "dtype": dtype, "m": m, "n": n, "k": k,
                          "gpus": world, "median_ms": median, "iqr_ms": iqr, "gflops": gflops,
                          "tflops": gflops / 1000.0,
                          "pct_peak_datasheet": 100.0 * gflops / (2.25e6 * world),
                          "baseline_gflops": 0.0, "pct_baseline": 0.0, "commit": commit}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
