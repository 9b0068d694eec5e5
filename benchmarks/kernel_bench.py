"""Single-GPU microbenchmark of the codec and fused kernels (HBM roofline check).

Usage: python benchmarks/kernel_bench.py [--mib 64 256] [--worlds 1 2 8] [--with-reference] [--topk K] [--profile] [--out FILE]
Every kernel is timed with CUDA events after warm-up with an L2 flush between
iterations; bandwidth = algorithmic bytes / median time, reported as a fraction
of the measured copy bandwidth in MEASURED_PEAKS.json (fallback 6650 GB/s).
`--with-reference` also times the unmodified reference's own kernels (its extension
built for sm_100 under baseline/_ref, loaded into the same process) on the same
tensors: `inplace_quantize_pack`, `inplace_dequantize_reduce_mean` and
`inplace_dequantize_reduce_mean_update_error_feedback`
(ccdl_comm/quantization/codec.py:161-217, 355-466).
`--topk K` also times the general-profile all-reduce (K outliers per group kept verbatim) on the emulated ranks,
in its one-stage and its two-stage form.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lowbit_comm_b200.config import CompressionConfig  # noqa: E402
from lowbit_comm_b200.ops import codec  # noqa: E402
from lowbit_comm_b200.parallel.fused import FusedWorkspace, run_loopback  # noqa: E402
from lowbit_comm_b200.parallel.peer_memory import PeerGroup  # noqa: E402
from lowbit_comm_b200.utils.timing import L2Flusher, time_cuda  # noqa: E402


def peak_gbs() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, nargs="+", default=[64, 256])
    ap.add_argument("--worlds", type=int, nargs="*", default=[1, 2, 8])
    ap.add_argument("--profile", action="store_true", help="one warm-up + one timed launch per kernel (for ncu)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--with-reference", action="store_true")
    ap.add_argument("--engine", choices=("auto", "pipe", "legacy"), default="auto",
                    help="all-reduce engine of the emulated-rank part: single persistent kernel or kernel sequence")
    ap.add_argument("--skip-codec", action="store_true", help="only the all-reduce on emulated ranks (for captures)")
    ap.add_argument("--topk", type=int, default=0, choices=(0, 1, 2),
                    help="also time the general-profile (top-k) all-reduce on the emulated ranks, one and two stages")
    ap.add_argument("--out", default="bench_out/kernel_bench.json")
    args = ap.parse_args()
    ref = None
    if args.with_reference:
        try:
            sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
            import reference_env

            _, ref_status = reference_env.activate(need_cuda_extension=True)
            from ccdl_comm.config import CompressionConfig as RefConfig
            from ccdl_comm.quantization import codec as ref_codec

            ref = (ref_codec, RefConfig(bit=8, group_size=64, topk=0), ref_status)
        except Exception as exc:  # noqa: BLE001
            print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}), flush=True)
    cfg = CompressionConfig()
    peak, peak_kind = peak_gbs()
    flush = None if args.profile else L2Flusher()
    warm = 1 if args.profile else 3
    if args.profile:
        args.iters = 1
    rows = []

    def record(name, mib, nbytes, t, **extra):
        gbs = nbytes / (t["median_ms"] * 1e-3) / 1e9
        row = {"kernel": name, "mib": mib, "bytes": nbytes, **t, "gbs": gbs, "frac_of_peak": gbs / peak,
               "peak_gbs": peak, "peak_kind": peak_kind, **extra}
        rows.append(row)
        print(json.dumps(row), flush=True)

    for mib in args.mib:
        n = mib * 1024 * 1024 // 2
        x = (torch.randn(n, device="cuda") * 1e-3).to(torch.bfloat16)
        res = torch.zeros_like(x)
        out = codec.allocate_quantized_buffer(x, cfg)
        pb = out.numel()
        if not args.skip_codec:
            t = time_cuda(lambda: codec.quantize_tensor(x, cfg, output=out), iters=args.iters, flush=flush, warmup=warm)
            record("quant_push(local)", mib, 2 * n + pb, t)
            t = time_cuda(lambda: codec.quantize_tensor(x, cfg, output=out, residual=res, prepared_out=res),
                          iters=args.iters, flush=flush, warmup=warm)
            record("quant_push(local,+EF in place)", mib, 6 * n + pb, t)
            y = torch.empty_like(x)
            t = time_cuda(lambda: codec.dequantize_tensor(out, x.shape, cfg, dtype="bf16", output=y),
                          iters=args.iters, flush=flush, warmup=warm)
            record("reduce(1 payload)", mib, 2 * n + pb, t)
            t = time_cuda(lambda: codec.inplace_dequantize_reduce_mean_update_error_feedback(
                [out], res, y, res, cfg, reduce="mean"), iters=args.iters, flush=flush, warmup=warm)
            record("reduce(1 payload,+EF in place)", mib, 6 * n + pb, t)
            bufs = [out] + [out.clone() for _ in range(7)]
            t = time_cuda(lambda: codec.inplace_dequantize_reduce_mean(bufs, y, cfg, reduce="mean"),
                          iters=args.iters, flush=flush, warmup=warm)
            record("reduce(8 payloads)", mib, 2 * n + 8 * pb, t)
            z = torch.empty_like(x)
            t = time_cuda(lambda: z.copy_(x), iters=args.iters, flush=flush, warmup=warm)
            record("torch copy_ (reference point)", mib, 4 * n, t)
            if ref is not None:
                rc, rcfg, rstatus = ref
                try:
                    rout = rc.allocate_quantized_buffer(x, rcfg, dtype="bf16").reshape(-1)
                    # the default (planar) profile: what the reference's hook and transports run per bucket
                    t = time_cuda(lambda: rc.quantize_tensor(x, rcfg, extension_status=rstatus, output=rout),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("reference quantize_tensor(output=)", mib, 2 * n + pb, t)
                    t = time_cuda(lambda: rc.quantize_tensor(x, rcfg, extension_status=rstatus, output=rout, residual=res),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("reference quantize_tensor(output=, residual=)", mib, 4 * n + pb, t)
                    # its fused quantize-and-pack kernel serves compact payloads only (it answers False otherwise)
                    from dataclasses import replace as _replace

                    rcompact, ccompact = _replace(rcfg, compact=True), CompressionConfig(compact=True)
                    ok = rc.inplace_quantize_pack(x, rout, res, rcompact, extension_status=rstatus)
                    t = time_cuda(lambda: rc.inplace_quantize_pack(x, rout, res, rcompact, extension_status=rstatus),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("reference inplace_quantize_pack(compact,+residual)", mib, 4 * n + pb, t, fused=bool(ok))
                    t = time_cuda(lambda: codec.quantize_tensor(x, ccompact, output=out, residual=res),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("quant_push(local,compact,+residual)", mib, 4 * n + pb, t)
                    rbufs = [rout] + [rout.clone() for _ in range(7)]
                    t = time_cuda(lambda: rc.inplace_dequantize_reduce_mean(rbufs[:1], y, rcfg, extension_status=rstatus,
                                                                            reduce="mean"),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("reference inplace_dequantize_reduce_mean(1 payload)", mib, 2 * n + pb, t)
                    t = time_cuda(lambda: rc.inplace_dequantize_reduce_mean(rbufs, y, rcfg, extension_status=rstatus,
                                                                            reduce="mean"),
                                  iters=args.iters, flush=flush, warmup=warm)
                    record("reference inplace_dequantize_reduce_mean(8 payloads)", mib, 2 * n + 8 * pb, t)
                    prep, restored = x.clone(), torch.empty_like(x)
                    t = time_cuda(lambda: rc.inplace_dequantize_reduce_mean_update_error_feedback(
                        rbufs[:1], prep, restored, res, rcfg, extension_status=rstatus, reduce="mean"),
                        iters=args.iters, flush=flush, warmup=warm)
                    record("reference inplace_dequantize_reduce_mean_update_error_feedback(1 payload)", mib,
                           6 * n + pb, t)
                    del rbufs, prep, restored
                except Exception as exc:  # noqa: BLE001
                    print(json.dumps({"impl": "reference", "mib": mib, "error": f"{type(exc).__name__}: {exc}"[:300]}),
                          flush=True)
            del bufs, y, z
        for world in args.worlds:
            need = FusedWorkspace.required_bytes(world, "bf16", cfg, n, world <= 2) + (1 << 20)
            if need * world > 60 * (1 << 30):
                continue
            groups = PeerGroup.loopback(world, need)
            wss = [FusedWorkspace(g, dtype="bf16", config=cfg, max_numel=n, engine=args.engine) for g in groups]
            xs = [x] + [x.clone() for _ in range(world - 1)]
            rs = [torch.zeros_like(x) for _ in range(world)]

            def step():
                run_loopback(wss, "all_reduce", [(xs[r],) for r in range(world)],
                             [{"residual": rs[r]} for r in range(world)])

            t = time_cuda(step, iters=max(3, args.iters // 2), flush=flush)
            # all emulated ranks share one GPU: per-rank time = total / world
            per_rank_ms = t["median_ms"] / world
            stages = 1 if world <= 2 else 2
            c = pb / n
            hbm = (6 * n + c * n) + (stages == 2) * (2 * c * n) + (c * n * (world if stages == 1 else 1) + 6 * n)
            rows.append({"kernel": f"all_reduce loopback W={world} ({stages}-stage, EF, engine {wss[0].engine})", "mib": mib,
                         "per_rank_ms": per_rank_ms, "hbm_bytes_model": hbm,
                         "gbs": hbm / (per_rank_ms * 1e-3) / 1e9, "frac_of_peak": hbm / (per_rank_ms * 1e-3) / 1e9 / peak,
                         "launches_per_rank": wss[0].launches // max(1, (3 + max(3, args.iters // 2)))})
            print(json.dumps(rows[-1]), flush=True)
            torch.cuda.synchronize()
            groups[0].check_status()
            PeerGroup.close_loopback(groups)
            del wss, xs, rs
            if args.topk and world > 1:
                from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

                kcfg = CompressionConfig(topk=args.topk, allow_experimental=True)
                need = GeneralPeerWorkspace.required_bytes(world, "bf16", kcfg, n) + (1 << 20)
                if need * world <= 60 * (1 << 30):
                    groups = PeerGroup.loopback(world, need)
                    gws = [GeneralPeerWorkspace(g, dtype="bf16", config=kcfg, max_numel=n) for g in groups]
                    xs = [x] + [x.clone() for _ in range(world - 1)]
                    rs = [torch.zeros_like(x) for _ in range(world)]
                    for stages in (1, 2):
                        def general_step(stages=stages):
                            run_loopback(gws, "all_reduce", [(xs[r],) for r in range(world)],
                                         [{"residual": rs[r]} for r in range(world)], stages=stages)

                        t = time_cuda(general_step, iters=max(3, args.iters // 2), flush=flush)
                        rows.append({"kernel": f"top-k {args.topk} all_reduce loopback W={world} ({stages}-stage, EF)",
                                     "mib": mib, "per_rank_ms": t["median_ms"] / world})
                        print(json.dumps(rows[-1]), flush=True)
                    torch.cuda.synchronize()
                    groups[0].check_status()
                    PeerGroup.close_loopback(groups)
                    del gws, xs, rs
        del x, res, out
        torch.cuda.empty_cache()
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    json.dump(rows, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
