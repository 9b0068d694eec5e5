"""Reduced-shard interface benchmark: 64 buckets of 32 MiB bf16 gradients, compressed
reduce-scatter (shard output) + compressed all-gather, flat versus hierarchical 2x4 grouping.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 benchmarks/sharded_rs_ag.py [--buckets 64 --mib 32 --iters 100]

Values N(0, 1e-3), int8 group 64 with error feedback (this rank's own quantization
error on the scatter stage).  One timed iteration = all buckets through
reduce-scatter then all-gather; timed on the device with CUDA events, max over
ranks.  The working set (64 x 32 MiB = 2 GiB per rank) is far larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--buckets", type=int, default=64)
    ap.add_argument("--mib", type=int, default=32)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--local-group", type=int, default=4)
    ap.add_argument("--out", default="bench_out/sharded_rs_ag.json")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.communicator import Communicator
    from lowbit_comm_b200.parallel.fused import FusedWorkspace, geometry

    cfg = CompressionConfig()
    n = args.mib * 1024 * 1024 // 2
    arena = FusedWorkspace.required_bytes(world, "bf16", cfg, 1 << (n - 1).bit_length(), True) + (128 << 20)
    comm = Communicator(None, arena_bytes=arena)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    buckets = [(torch.randn(n, generator=gen, device=dev) * 1e-3).to(torch.bfloat16) for _ in range(args.buckets)]
    residuals = [torch.zeros_like(b) for b in buckets]
    geo = geometry(n, world, "bf16", cfg)
    shards = [torch.empty(geo.shard_numel, dtype=torch.bfloat16, device=dev) for _ in range(args.buckets)]
    gathered = [[torch.empty(geo.shard_numel, dtype=torch.bfloat16, device=dev) for _ in range(world)]
                for _ in range(2)]

    def flat_step() -> None:
        ws = comm.workspace(buckets[0], cfg, "bf16")
        for i, (b, r, s) in enumerate(zip(buckets, residuals, shards)):
            ws.reduce_scatter(b, s, residual=r, op="mean")
            ws.all_gather(s, gathered[i & 1])

    def hierarchical_step() -> None:
        for b in buckets:
            comm.hierarchical_all_reduce(b, config=cfg, op="mean", local_group_size=args.local_group, out=b)

    def nccl_step() -> None:
        for b, s in zip(buckets, shards):
            dist.reduce_scatter_tensor(s[: n // world], b, op=dist.ReduceOp.AVG)
            dist.all_gather_into_tensor(b, s[: n // world])

    def measure(fn, iters: int) -> dict:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        samples = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            samples.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(samples), sum(samples) / len(samples)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return {"median_ms": float(t[0]), "mean_ms": float(t[1]), "iters": iters}

    total_bytes = args.buckets * n * 2
    rows = []
    arms = [("ours_flat_rs_ag", flat_step), ("nccl_bf16_rs_ag", nccl_step)]
    if world % args.local_group == 0 and world > args.local_group:
        arms.insert(1, (f"ours_hierarchical_{world // args.local_group}x{args.local_group}", hierarchical_step))
    for name, fn in arms:
        iters = args.iters if name != arms[1][0] or len(arms) == 2 else max(5, args.iters // 5)
        t = measure(fn, iters)
        comm.check_status()
        rows.append({"impl": name, "world": world, "buckets": args.buckets, "bucket_mib": args.mib, **t,
                     "algbw_gbs": total_bytes / (t["median_ms"] * 1e-3) / 1e9,
                     "per_bucket_us": t["median_ms"] * 1e3 / args.buckets})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump(rows, open(args.out, "w"), indent=1)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
