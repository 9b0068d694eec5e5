"""Synthetic-MLP DDP throughput (samples/s): the shape of the reference's own end-to-end benchmark.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/mlp_ddp.py --impl ours|nccl|reference|fsdp [--steps 20 --warmup 5]

Model and schedule follow the reference's published run (fp16 MLP 2048 -> 4096 x 4 -> 1024, 62.9 M parameters,
batch 16 per rank, SGD, 20 timed steps after 5 warm-up steps; its numbers are for 2 x RTX A6000:
tests/benchmarks/reports/a6000_scale_20260804).  Timing: CUDA events around the timed steps, bracketed by a
barrier and a device synchronise, maximum over ranks.  Every step copies its batch from pinned host memory and
reads the loss back, so the figure is end to end.  A step touches the 126 MB of parameters and as much again
of gradients, more than the L2, so nothing is flushed between steps.  One JSON line on rank 0.
`--impl fsdp` wraps the same model in torch's FullyShardedDataParallel instead of DDP: the baseline mode of the
reference's comparison script (tests/distributed/synthetic_ddp_compare.py:100-105), uncompressed, GPU only.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

WIDTHS = (2048, 4096, 4096, 4096, 4096, 1024)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("ours", "nccl", "reference", "fsdp"), default="ours")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=3,
                    help="timed regions of --steps steps each; the median is reported, every sample is kept")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--dtype", choices=("fp16", "bf16", "fp32"), default="fp16")
    ap.add_argument("--strategy", default="auto")
    ap.add_argument("--max-blocks", type=int, default=0, help="grid cap of the hook's kernels (0 = library default)")
    ap.add_argument("--out", default="bench_out/mlp_ddp.json")
    ap.add_argument("--cpu", action="store_true",
                    help="dry run on CPU ranks (gloo, host timer, narrow model): checks the script, measures nothing useful")
    args = ap.parse_args()
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from lowbit_comm_b200.models.mlp import SyntheticMLP

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    widths = WIDTHS
    if args.cpu:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        args.dtype, widths = "fp32", tuple(w // 16 for w in WIDTHS)
    else:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[args.dtype]

    torch.manual_seed(1234)
    model = SyntheticMLP(widths, dtype=dtype, bias=False).to(device)      # 62 914 560 weights, as published
    if args.impl == "fsdp":
        if args.cpu:
            if rank == 0:
                print(json.dumps({"impl": "fsdp", "unavailable": "the FSDP baseline arm runs on CUDA ranks only"}), flush=True)
            dist.destroy_process_group()
            return
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

        ddp = FSDP(model, device_id=local_rank, use_orig_params=True)
        note = "none (torch FullyShardedDataParallel, full shard, uncompressed)"
    else:
        ddp = DDP(model, device_ids=None if args.cpu else [local_rank], bucket_cap_mb=25, gradient_as_bucket_view=True)
        note = "none (NCCL all-reduce)"
    hook = None
    if args.impl == "ours":
        from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook

        cfg = CompressionConfig(bit=8, group_size=64, error_feedback=True, target="ddp_gradient_bucket")
        hook = create_ddp_comm_hook(cfg, strategy=args.strategy, reduce="mean", module=ddp.module,
                                    max_blocks=args.max_blocks)
        ddp.register_comm_hook(state=None, hook=hook)
        note = f"lowbit_comm_b200 int8 g64 EF strategy={args.strategy}" + (
            f" max_blocks={args.max_blocks}" if args.max_blocks else "")
    elif args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_env

        ok, why = reference_env.reference_available()
        if not ok:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            dist.destroy_process_group()
            return
        reference_env.activate(need_cuda_extension=True)
        from ccdl_comm.communication import create_ddp_comm_hook as ref_factory
        from ccdl_comm.config import CompressionConfig as RefConfig

        rcfg = RefConfig(bit=8, group_size=64, error_feedback=True, target="ddp_gradient_bucket")
        ddp.register_comm_hook(state=None, hook=ref_factory(rcfg, dtype="auto", strategy="all_gather", reduce="mean",
                                                            async_gather=True, async_error_feedback=True))
        note = "ccdl_comm hook strategy=all_gather async_gather async_error_feedback"

    opt = torch.optim.SGD(ddp.parameters(), lr=0.01)
    total = args.warmup + args.steps
    gen = torch.Generator().manual_seed(100 + rank)
    xs = torch.randn(total, args.batch, widths[0], generator=gen).to(dtype)
    ys = torch.randn(total, args.batch, widths[-1], generator=gen).to(dtype)
    if not args.cpu:
        xs, ys = xs.pin_memory(), ys.pin_memory()

    def step(i: int) -> float:
        x, y = xs[i].to(device, non_blocking=True), ys[i].to(device, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(ddp(x).float(), y.float())
        loss.backward()
        opt.step()
        return loss.item()

    for i in range(args.warmup):
        step(i)
    last, peak_mib = 0.0, 0.0
    samples: list[float] = []
    launches_before = hook.gpu_launches() if hook is not None else 0
    # A region of 20 steps lasts some tens of milliseconds, so one stall doubles it: several regions, the median
    # reported, every sample kept (the reference's script reports the median of three runs as well,
    # tests/distributed/synthetic_ddp_compare.py:157-249).
    for _ in range(max(1, args.repeats)):
        dist.barrier()
        if args.cpu:
            import time

            began = time.perf_counter()
            for i in range(args.warmup, total):
                last = step(i)
            elapsed_ms = (time.perf_counter() - began) * 1e3
        else:
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(args.warmup, total):
                last = step(i)
            stop.record()
            torch.cuda.synchronize()
            elapsed_ms = start.elapsed_time(stop)
            peak_mib = max(peak_mib, torch.cuda.max_memory_allocated() / 2**20)
        region = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(region, op=dist.ReduceOp.MAX)
        samples.append(float(region.item()))
    dist.barrier()
    import statistics

    ms = torch.tensor([statistics.median(samples)], dtype=torch.float64, device=device)
    launches = ((hook.gpu_launches() - launches_before) // max(1, args.repeats)) if hook is not None else 0
    if rank == 0:
        line = {"metric": "synthetic MLP DDP training throughput", "value": args.batch * world * args.steps / (ms.item() * 1e-3),
                "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms.item() / args.steps, "higher_is_better": True, "scaling": "weak", "dtype": args.dtype,
                "impl": args.impl, "data": "synthetic (normal inputs and targets, random-init weights)",
                "config": {"model": "mlp " + "-".join(map(str, widths)), "params": sum(p.numel() for p in model.parameters()),
                           "micro_batch_per_gpu": args.batch, "optimizer": "SGD lr 0.01", "bucket_cap_mb": 25, "hook": note,
                           "l2": "a step touches more than 126 MB; no explicit flush"},
                "e2e": {"h2d_bytes_per_step": int(xs[0].numel() + ys[0].numel()) * xs.element_size(), "d2h_bytes_per_step": 4},
                "peak_memory_mib": peak_mib, "ms_per_step_samples": [round(m / args.steps, 4) for m in samples],
                "gpu_launches": launches, "final_loss": last}
        print(json.dumps(line), flush=True)
        os.makedirs(os.path.dirname(os.path.join(ROOT, args.out)), exist_ok=True)
        with open(os.path.join(ROOT, args.out), "w") as fh:
            json.dump(line, fh)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
