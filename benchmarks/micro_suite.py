"""The smaller latency figures the reference publishes, measured here through the public API on N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/micro_suite.py [--sizes-mib 1 16 64] [--iters 10] [--out bench_out/micro_suite.json]

Cases (each row names the call that is timed):
  reduced_shard      compressed_reduce_scatter_shard (ReducedShard output) vs NCCL reduce_scatter_tensor and vs NCCL's
                     full all-reduce, the baseline the reference quotes its shard numbers against
  async_vs_sync      compressed_all_reduce(async_op=True) + wait() vs the synchronous call
  dynamic_gather     compressed_all_gather_dynamic with metadata_protocol tensor_v1 vs object_v1 (ragged sizes)
  p2p                qsend / qrecv of one tensor between ranks 0 and 1: time and relative L2 error
  dispatch_overhead  host time per call (no synchronisation inside the loop) of a compiled plan's `run()`, of the
                     public `compressed_all_reduce` and of the workspace's own `all_reduce`, against the device time
                     of the collective: what planning and dispatch add (the reference requires < 1 % for its
                     compiled dispatch, tests/distributed/executor_overhead_perf.py)

Timing: CUDA events on the launching stream, 3 warm-up calls, median of `--iters`, a 256 MiB write between calls
to flush the 126 MB L2, a barrier before every call, maximum over ranks.  fp16 sources, int8 codes, 64-element
groups, error feedback off (single calls, as in the reference's tables).
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
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=[1, 16, 64])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cases", nargs="+",
                    default=["reduced_shard", "async_vs_sync", "dynamic_gather", "p2p", "dispatch_overhead"])
    ap.add_argument("--out", default="bench_out/micro_suite.json")
    ap.add_argument("--cpu", action="store_true",
                    help="dry run on CPU ranks (gloo, host timer, no L2 flush): checks the script, measures nothing useful")
    args = ap.parse_args()
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

    import torch
    import torch.distributed as dist

    import lowbit_comm_b200 as lbc
    from lowbit_comm_b200.utils.timing import L2Flusher

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    if args.cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
        flush = lambda: None                                                        # noqa: E731
    else:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        flush = L2Flusher(dev)
    cfg = lbc.CompressionConfig(error_feedback=False)

    def measure(fn) -> float:
        """Median milliseconds of `fn()`, maximum over ranks."""

        import time

        times = []
        for i in range(args.warmup + args.iters):
            flush()
            dist.barrier()
            if args.cpu:
                began = time.perf_counter()
                fn()
                elapsed = (time.perf_counter() - began) * 1e3
            else:
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                fn()
                stop.record()
                torch.cuda.synchronize()
                elapsed = start.elapsed_time(stop)
            if i >= args.warmup:
                times.append(elapsed)
        t = torch.tensor([statistics.median(times)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows: list[dict] = []

    def record(**row) -> None:
        row.update(world=world, dtype="fp16")
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    def rel_l2(got, exact) -> float:
        return ((got.float() - exact.float()).norm() / exact.float().norm()).item()

    for mib in args.sizes_mib:
        n = int(mib * (1 << 20)) // 2
        n -= n % (64 * 8 * world)                       # whole groups per shard: the reference's shard path needs it too
        gen = torch.Generator(device=dev).manual_seed(7 + rank)
        x = (torch.randn(n, generator=gen, device=dev) * 1e-2).half()
        exact = x.float().clone()
        dist.all_reduce(exact)
        exact /= world

        if "reduced_shard" in args.cases and world > 1:
            shard_out = torch.empty(n // world, dtype=torch.float16, device=dev)
            probe = lbc.compressed_reduce_scatter_shard(x, config=cfg, op="mean")
            own_out = torch.empty(probe.shard_numel, dtype=torch.float16, device=dev)
            t_ours = measure(lambda: lbc.compressed_reduce_scatter_shard(x, config=cfg, op="mean", out=own_out))
            lo = probe.shard_index * probe.shard_numel
            err = rel_l2(own_out[: max(0, min(n - lo, probe.shard_numel))], exact[lo:lo + probe.shard_numel])
            full = x.clone()
            if args.cpu:                                   # gloo has neither reduce_scatter_tensor nor AVG
                t_rs = float("nan")
                t_full = measure(lambda: dist.all_reduce(full))
            else:
                t_rs = measure(lambda: dist.reduce_scatter_tensor(shard_out, x, op=dist.ReduceOp.AVG))
                t_full = measure(lambda: dist.all_reduce(full, op=dist.ReduceOp.AVG))
            record(case="reduced_shard", mib=mib, ours_ms=t_ours, nccl_reduce_scatter_ms=t_rs, nccl_all_reduce_ms=t_full,
                   speedup_vs_nccl_full=t_full / t_ours, speedup_vs_nccl_reduce_scatter=t_rs / t_ours, rel_l2=err,
                   transport=probe.transport)

        if "dispatch_overhead" in args.cases and not args.cpu:
            import time

            from lowbit_comm_b200.parallel.backend_cuda import compile_cuda_shortcut
            from lowbit_comm_b200.parallel.communicator import get_communicator

            comm = get_communicator(None)
            ws = comm.workspace(x, cfg, "fp16")
            work, scratch = x.clone(), x.clone()           # the compiled shortcut reduces in place: not into x
            compiled = compile_cuda_shortcut(scratch, collective="all_reduce", strategy="auto", output_layout="full",
                                             config=cfg, reduce_op="mean")

            def host_us(fn, calls=200) -> float:
                fn()
                torch.cuda.synchronize()
                dist.barrier()
                t0 = time.perf_counter()
                for _ in range(calls):
                    fn()
                dt = time.perf_counter() - t0
                torch.cuda.synchronize()
                return dt / calls * 1e6

            direct = host_us(lambda: ws.all_reduce(x, work))
            public = host_us(lambda: lbc.compressed_all_reduce(x, config=cfg, op="mean", strategy="auto", out=work))
            planned = host_us(lambda: compiled.run(scratch))
            device = measure(lambda: ws.all_reduce(x, work)) * 1e3
            # a call returns as soon as its kernels are enqueued, so host time only shows in the step time when it
            # exceeds the device time of the collective; back-to-back device time per call says whether it does
            t_direct = measure(lambda: [ws.all_reduce(x, work) for _ in range(20)]) * 1e3 / 20
            t_planned = measure(lambda: [compiled.run(scratch) for _ in range(20)]) * 1e3 / 20
            record(case="dispatch_overhead", mib=mib, direct_host_us=direct, public_api_host_us=public,
                   compiled_run_host_us=planned, device_us=device, back_to_back_direct_us=t_direct,
                   back_to_back_compiled_us=t_planned,
                   compiled_over_direct_pct=100.0 * (t_planned - t_direct) / t_direct,
                   host_bound=bool(planned > device))

        if "async_vs_sync" in args.cases:
            work = x.clone()
            t_sync = measure(lambda: lbc.compressed_all_reduce(x, config=cfg, op="mean", strategy="auto", out=work))
            t_async = measure(lambda: lbc.compressed_all_reduce(x, config=cfg, op="mean", strategy="auto", out=work,
                                                                async_op=True).wait())
            record(case="async_vs_sync", mib=mib, sync_ms=t_sync, async_launch_wait_ms=t_async, rel_l2=rel_l2(work, exact))

        if "dynamic_gather" in args.cases:
            mine = x[: max(64, n - rank * 1024)].contiguous()      # every rank a different length
            for protocol in ("tensor_v1", "object_v1"):
                t = measure(lambda p=protocol: lbc.compressed_all_gather_dynamic(mine, config=cfg, metadata_protocol=p))
                record(case="dynamic_gather", mib=mib, metadata_protocol=protocol, ms=t)

        if "p2p" in args.cases and world > 1:
            recv = torch.empty_like(x)

            def exchange():
                if rank == 0:
                    lbc.qsend(x, 1, config=cfg)
                elif rank == 1:
                    lbc.qrecv(recv, 0, config=cfg)

            t = measure(exchange)
            err = torch.zeros(1, device=dev)
            if rank == 1:
                gen0 = torch.Generator(device=dev).manual_seed(7)                 # rank 0's tensor, from its seed
                sent = (torch.randn(n, generator=gen0, device=dev) * 1e-2).half()
                err[0] = rel_l2(recv, sent)
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
            record(case="p2p", mib=mib, ms=t, rel_l2=float(err.item()))
        del x, exact
        if not args.cpu:
            torch.cuda.empty_cache()

    if rank == 0:
        os.makedirs(os.path.dirname(os.path.join(ROOT, args.out)) or ".", exist_ok=True)
        with open(os.path.join(ROOT, args.out), "w") as fh:
            json.dump(rows, fh, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
