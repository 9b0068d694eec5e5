"""Reduced-shard interface benchmark: 64 buckets of 32 MiB bf16 gradients, compressed
reduce-scatter (shard output) + compressed all-gather, flat versus hierarchical 2x4 grouping.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 benchmarks/sharded_rs_ag.py [--buckets 64 --mib 32 --iters 100]

Values N(0, 1e-3), int8 group 64 with error feedback (this rank's own quantization
error on the scatter stage).  One timed iteration = all buckets through
reduce-scatter then all-gather; timed on the device with CUDA events, max over
ranks.  The working set (64 x 32 MiB = 2 GiB per rank) is far larger than L2.
Arms: this library flat (reduce-scatter shard + all-gather of the shards) and hierarchical
(2 x 4: the three-stage chain), NCCL bf16 reduce-scatter + all-gather, and with
`--with-reference` the unmodified reference: its `compressed_reduce_scatter_shard` followed by
its `compressed_all_gather` of the shard, and its `compressed_hierarchical_all_reduce`.
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
    ap.add_argument("--with-reference", action="store_true")
    ap.add_argument("--ref-iters", type=int, default=10)
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

    ref_arms = []
    if args.with_reference:
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import reference_env

            reference_env.activate(need_cuda_extension=True)
            from ccdl_comm.collectives import compressed_all_gather as ref_gather
            from ccdl_comm.collectives import compressed_hierarchical_all_reduce as ref_hier
            from ccdl_comm.collectives import compressed_reduce_scatter_shard as ref_shard
            from ccdl_comm.config import CompressionConfig as RefConfig

            rcfg = RefConfig(bit=8, group_size=64, topk=0)

            def ref_flat_step() -> None:
                for b in buckets:
                    shard = ref_shard(b, config=rcfg, op="mean")
                    ref_gather(shard.shard, config=rcfg)

            def ref_hier_step() -> None:
                os.environ.setdefault("CCDL_LOCAL_GROUP_SIZE", str(args.local_group))
                for b in buckets:
                    ref_hier(b, config=rcfg, op="mean")

            ref_arms = [("reference_rs_shard_ag", ref_flat_step), ("reference_hierarchical", ref_hier_step)]
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}), flush=True)

    total_bytes = args.buckets * n * 2
    rows = []
    arms = [("ours_flat_rs_ag", flat_step), ("nccl_bf16_rs_ag", nccl_step)]
    if world % args.local_group == 0 and world > args.local_group:
        arms.insert(1, (f"ours_hierarchical_{world // args.local_group}x{args.local_group}", hierarchical_step))
    for name, fn in arms + ref_arms:
        iters = args.ref_iters if name.startswith("reference") else args.iters
        try:
            t = measure(fn, iters)
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": name, "error": f"{type(exc).__name__}: {exc}"[:300]}), flush=True)
            continue
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
