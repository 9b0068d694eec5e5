"""Compressed all-reduce sweep (algBW vs size) on 2/4/8 GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/allreduce_sweep.py [--min-mib 1 --max-mib 1024] [--with-reference]

One bf16 gradient tensor per size (x2 steps), values N(0, 1e-3) with 0.1 %
outliers x100, int8 group-64 payload with error feedback.  Arms: this library
(the default choice, and the one-stage and two-stage paths forced), NCCL bf16
all-reduce, and optionally the unmodified reference from baseline/_ref: its
`compressed_all_reduce` with strategy all_gather and with strategy topology (its
compiled pipelined ring) and its `compressed_reduce_scatter_shard`.  Every sample
is timed on the device with CUDA events after an L2 flush and a barrier; the
reported time is the max over ranks of each rank's median.  algBW = tensor bytes /
time.  The roofline of a fused path (`lowbit_comm_b200.utils.roofline`) is the
slower of its HBM traffic at the measured copy bandwidth and its NVLink traffic at
770 GB/s per direction (the measured peer-copy rate of this pool; 900 nominal).
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
    ap.add_argument("--min-mib", type=float, default=1)
    ap.add_argument("--max-mib", type=float, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--with-reference", action="store_true")
    ap.add_argument("--ref-arms", default="all_gather,topology,shard",
                    help="reference paths to time: all_gather, topology (compiled ring), shard (reduce-scatter shard)")
    ap.add_argument("--ref-max-mib", type=float, default=1024)
    ap.add_argument("--engine", choices=("auto", "pipe", "legacy"), default="auto",
                    help="pipe: one persistent kernel per all-reduce; legacy: the K1/K2/K3 kernel sequence; "
                         "auto: the library's choice by size")
    ap.add_argument("--arms", default="auto,1,2", help="paths of this library to time: auto, 1 (one stage), 2 (two stages)")
    ap.add_argument("--topk", default="", help="also time top-k profiles (e.g. 1,2) through the fused general kernels")
    ap.add_argument("--topk-max-mib", type=float, default=64, help="largest tensor of the top-k arms")
    ap.add_argument("--ring", type=int, default=None, help="pipelined engine: rows in flight per block (2..4)")
    ap.add_argument("--no-ef", action="store_true", help="time the collectives without error feedback")
    ap.add_argument("--chunk-mib", type=float, default=None, help="pipeline chunk size (0 = no pipelining)")
    ap.add_argument("--variants", action="store_true", help="time every push/reduce kernel variant")
    ap.add_argument("--phases", action="store_true", help="also time K1/K2/K3 separately (Python launch path)")
    ap.add_argument("--gather", choices=("pull", "push"), default=None,
                    help="two-stage gather: peer loads by the decode kernel (pull) or peer stores by the reduce kernel")
    ap.add_argument("--gather-order", type=int, choices=(0, 1), default=None,
                    help="pull gather: 1 = tiles round-robin over the owners (default), 0 = linear sweep")
    ap.add_argument("--gather-prefetch", type=int, choices=(0, 2, 4), default=None,
                    help="decode stage: tiles of peer loads in flight per thread (0 = general reduce kernel)")
    ap.add_argument("--kernel-names", action="store_true",
                    help="record which CUDA kernels one (untimed) call launches, from torch.profiler")
    ap.add_argument("--multicast", action="store_true",
                    help="arenas from the symmetric-memory allocator: broadcasts use multimem stores")
    ap.add_argument("--out", default="bench_out/allreduce_sweep.json")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.communicator import Communicator
    from lowbit_comm_b200.utils.roofline import MEASURED_LINK_GBS, fused_all_reduce_roofline, measured_hbm_gbs
    from lowbit_comm_b200.utils.timing import L2Flusher

    cfg = CompressionConfig()
    hbm_gbs, peak_kind = measured_hbm_gbs(ROOT)
    os.environ["LBC_ENGINE"] = args.engine
    flush = L2Flusher(dev)
    max_numel = int(args.max_mib * 1024 * 1024 // 2)
    from lowbit_comm_b200.parallel.fused import FusedWorkspace

    arena = FusedWorkspace.required_bytes(world, "bf16", cfg, 1 << (max_numel - 1).bit_length(), True) + (256 << 20)
    topks = [int(k) for k in args.topk.split(",") if k]
    topk_cfgs = {k: CompressionConfig(topk=k, allow_experimental=True) for k in topks}
    topk_numel = int(min(args.topk_max_mib, args.max_mib) * 1024 * 1024 // 2)
    if topks:
        from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

        arena += sum(GeneralPeerWorkspace.required_bytes(world, "bf16", c, topk_numel) for c in topk_cfgs.values())
    if args.multicast:
        os.environ["LBC_MULTICAST"] = "1"
    comm = Communicator(None, arena_bytes=arena)
    big = comm.workspace(torch.empty(max_numel, dtype=torch.bfloat16, device=dev), cfg, "bf16")  # largest first
    if args.gather_order is not None:
        from lowbit_comm_b200.ops.loader import require_extension as _req

        _req().set_gather_order(args.gather_order)
    if args.gather_prefetch is not None:
        from lowbit_comm_b200.ops.loader import require_extension as _req

        _req().set_gather_prefetch(args.gather_prefetch)
    if args.gather is not None:
        big.set_gather_mode(args.gather)
    if args.engine != "legacy" and args.ring is not None:
        big._pipe.set_ring_depth(args.ring)
    if args.chunk_mib is not None:
        big.set_chunking(int(max(args.chunk_mib, 1e-3) * (1 << 20)), 1 if args.chunk_mib == 0 else 8)

    ref = None
    if args.with_reference:
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import reference_env

            reference_env.activate(need_cuda_extension=True)
            from ccdl_comm.collectives import compressed_all_reduce as ref_all_reduce
            from ccdl_comm.collectives import compressed_reduce_scatter_shard as ref_shard
            from ccdl_comm.config import CompressionConfig as RefConfig

            ref = (ref_all_reduce, ref_shard, RefConfig(bit=8, group_size=64, topk=0))
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))

    def measure(fn) -> float:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        samples = []
        for _ in range(args.iters):
            flush()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            samples.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(samples)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    multicast_on = bool(comm.peer_group is not None and comm.peer_group.multicast_ptr)
    if rank == 0:
        print(json.dumps({"multicast_arena": multicast_on, "engine": args.engine, "link_gbs": MEASURED_LINK_GBS,
                          "hbm_gbs": hbm_gbs, "peak_kind": peak_kind}), flush=True)
    rows = []
    mib = args.min_mib
    while mib <= args.max_mib:
        n = int(mib * 1024 * 1024 // 2)
        gen = torch.Generator(device=dev).manual_seed(1000 + rank)
        x = torch.randn(n, generator=gen, device=dev) * 1e-3
        mask = torch.rand(n, generator=gen, device=dev) < 1e-3
        x = torch.where(mask, x * 100, x).to(torch.bfloat16)
        exact = x.float().clone()
        dist.all_reduce(exact)
        exact /= world
        nbytes = n * 2
        residual = None if args.no_ef else torch.zeros_like(x)
        work = x.clone()

        def ours(stages):
            strategy = {0: "auto", 1: "all_gather", 2: "reduce_scatter"}[stages]

            def run():
                comm.all_reduce(x, out=work, config=cfg, op="mean", strategy=strategy, residual=residual)
            return run

        from lowbit_comm_b200.ops.loader import require_extension

        ext = require_extension()
        combos = [(1, True, 0)]
        if args.variants:
            combos = [(0, True, 0), (1, True, 0), (2, True, 0), (1, False, 0), (1, False, -1), (1, True, -1),
                      (1, True, 592)]
        arms = [{"auto": 0, "1": 1, "2": 2}[a] for a in args.arms.split(",") if a]
        for stages, (push_variant, reduce_bulk, k2_blocks) in [(s, c) for s in arms for c in combos]:
            if stages == 1 and (not reduce_bulk or k2_blocks):
                continue
            ext.set_push_variant(push_variant, reduce_bulk, k2_blocks)
            if residual is not None:
                residual.zero_()
            t = measure(ours(stages))
            comm.check_status()
            if residual is not None:
                residual.zero_()
            ours(stages)()
            torch.cuda.synchronize()
            rel = ((work.float() - exact).norm() / exact.norm()).item()
            ran = stages or comm.workspace(x, cfg, "bf16").route(n, 2)[1]
            roof = fused_all_reduce_roofline(nbytes, world, stages=ran, error_feedback=residual is not None,
                                             hbm_gbs=hbm_gbs)
            phases = None
            if args.phases and args.engine == "legacy":
                from lowbit_comm_b200.utils.tracing import PhaseTimer

                ws = comm.workspace(x, cfg, "bf16")
                ws.phase_timer = PhaseTimer()
                for _ in range(5):
                    flush()
                    dist.barrier()
                    ours(stages)()
                phases = ws.phase_timer.summary()
                ws.phase_timer = None
            launched = None
            if args.kernel_names:                       # a separate call after the timed ones: evidence only
                from lowbit_comm_b200.utils.tracing import kernel_names

                launched = kernel_names(ours(stages))
            tag = f"_p{push_variant}r{int(reduce_bulk)}b{k2_blocks}" if args.variants else ""
            rows.append({"impl": ("ours_auto" if stages == 0 else f"ours_{stages}stage") + tag, "stages_run": ran,
                         "engine": args.engine, "error_feedback": residual is not None,
                         "mib": mib, "world": world, "ms": t,
                         "algbw_gbs": nbytes / (t * 1e-3) / 1e9, "rel_l2": rel, **roof,
                         "roofline_frac": roof["roofline_us"] / (t * 1e3), "peak_kind": peak_kind,
                         "phases_ms": phases, "multicast": multicast_on, "chunk_mib": args.chunk_mib,
                         "gather": "pull" if big.pull_gather else "push",
                         "gather_prefetch": ext.get_gather_prefetch(), "kernels": launched})
        ext.set_push_variant(1, True, 0)
        for k, kcfg in topk_cfgs.items():
            if n > topk_numel:
                continue
            if mib == args.min_mib:                      # the largest size first, so that the workspace fits them all
                comm.general_workspace(torch.empty(topk_numel, dtype=torch.bfloat16, device=dev), kcfg, "bf16")

            def general():
                comm.all_reduce(x, out=work, config=kcfg, op="mean", residual=residual)

            if residual is not None:
                residual.zero_()
            t = measure(general)
            comm.check_status()
            if residual is not None:
                residual.zero_()
            general()
            torch.cuda.synchronize()
            rows.append({"impl": f"ours_topk{k}", "mib": mib, "world": world, "ms": t, "error_feedback": residual is not None,
                         "algbw_gbs": nbytes / (t * 1e-3) / 1e9,
                         "rel_l2": ((work.float() - exact).norm() / exact.norm()).item()})
        nccl_buf = x.clone()

        def nccl():
            dist.all_reduce(nccl_buf, op=dist.ReduceOp.AVG)

        t = measure(nccl)
        rows.append({"impl": "nccl_bf16", "mib": mib, "world": world, "ms": t,
                     "algbw_gbs": nbytes / (t * 1e-3) / 1e9})
        if ref is not None and mib <= args.ref_max_mib:
            ref_all, ref_shard_fn, ref_cfg = ref
            ref_calls = {
                "all_gather": lambda: ref_all(x, config=ref_cfg, op="mean", strategy="all_gather"),
                "topology": lambda: ref_all(x, config=ref_cfg, op="mean", strategy="topology"),
                "shard": lambda: ref_shard_fn(x, config=ref_cfg, op="mean"),
            }
            for arm in [a for a in args.ref_arms.split(",") if a in ref_calls]:
                name = {"all_gather": "reference_all_gather", "topology": "reference_topology_ring",
                        "shard": "reference_reduce_scatter_shard"}[arm]
                try:
                    t = measure(ref_calls[arm])
                    out = ref_calls[arm]()
                    torch.cuda.synchronize()
                    row = {"impl": name, "mib": mib, "world": world, "ms": t, "algbw_gbs": nbytes / (t * 1e-3) / 1e9}
                    if arm != "shard":
                        row["rel_l2"] = ((out.float() - exact).norm() / exact.norm()).item()
                    rows.append(row)
                except Exception as exc:  # noqa: BLE001
                    rows.append({"impl": name, "mib": mib, "world": world, "error": f"{type(exc).__name__}: {exc}"[:200]})
        if rank == 0:
            for r in rows[-16:]:
                if r["mib"] == mib:
                    print(json.dumps(r), flush=True)
        del x, work, residual, nccl_buf, exact, mask
        torch.cuda.empty_cache()
        mib *= 2
    if rank == 0:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump(rows, open(args.out, "w"), indent=1)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
