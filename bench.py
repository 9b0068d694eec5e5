"""Headline benchmark: GPT-2 small DDP training throughput (tokens/s) with the
compressed int8 group-64 gradient hook and error feedback.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # unmodified reference (baseline/_ref)
    python bench.py --impl nccl --gpus N ...                 # plain NCCL bf16 DDP, no hook

For N > 1 launch with `python -m torch.distributed.run --nnodes=1 --nproc-per-node N
--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...`.

Configuration (fixed by the benchmark definition): 12 layers, d_model 768,
12 heads, sequence 1024, vocabulary 50257, random initialisation, uniform random
token ids, micro-batch 8 per GPU, AdamW lr 6e-4, bf16 parameters and gradients,
25 MB DDP buckets.  Weak scaling: per-GPU work is fixed.

After the W warm-up steps an untimed settle phase runs until three consecutive steps
agree within 2 % and at least 3 s have passed (a GPU of a fresh lease idles at a few
hundred MHz and needs seconds, not steps, to reach its working clocks); its length is
reported as `settle_steps`.  Then two kinds of region, K steps each, are timed
alternately three times (value, e2e, value, e2e, value, e2e); every region is bracketed
by a barrier and a device synchronise and timed with CUDA events, max over ranks, and
the reported numbers are the medians of the three samples (all samples are printed):
  value : inputs already on the device, no host read-back inside the loop
  e2e   : every step copies its token batch from pinned host memory and reads the
          loss back to the host
A training step touches far more than the 126 MB L2 (248 MB of parameters alone),
so no explicit L2 flush is needed between steps.

All three arms train the same model classes (`baseline/plain_models.py`, stock torch
modules that import nothing from either library), so the arms differ in the gradient
hook only.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """`nvidia-smi -lms 200` in the background; summarised after the timed region."""

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = os.path.join(ROOT, "bench_out", f"clocks_{os.getpid()}.csv")

    def start(self) -> None:
        try:
            os.makedirs(os.path.dirname(self.path), exist_ok=True)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            cols = [c.strip() for c in line.split(",")]
            if len(cols) < 9 or cols[0] != str(self.gpu_index):
                continue
            try:
                sm.append(float(cols[1]))
                sm_max.append(float(cols[2]))
                power.append(float(cols[3]))
            except ValueError:
                continue
            for name, val in zip(names, cols[5:9]):
                if val == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(sm_max), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference", "nccl"), default="ours")
    ap.add_argument("--model", choices=("gpt2-small", "gpt2-tiny", "llama-3b", "llama-tiny"), default="gpt2-small")
    ap.add_argument("--batch", type=int, default=None, help="micro-batch per GPU (default: 8, llama-3b: 2)")
    ap.add_argument("--strategy", default="auto", help="hook strategy of this library")
    ap.add_argument("--ef-mode", choices=("reference", "local"), default="reference")
    ap.add_argument("--ref-strategy", default="all_gather")
    ap.add_argument("--bucket-mb", type=int, default=None)
    ap.add_argument("--repeats", type=int, default=3, help="timed samples of each region (the median is reported)")
    ap.add_argument("--settle-s", type=float, default=3.0,
                    help="minimum length of the untimed settle phase after the warm-up (0 = none)")
    ap.add_argument("--gc-mode", choices=("default", "between"), default="default",
                    help="default: Python's cyclic collector runs when it wants; between: it is switched off inside "
                         "the timed regions and a full collection runs, untimed, between them (diagnostic: tells a "
                         "collector pause from a stall of the library)")
    ap.add_argument("--hook-max-blocks", type=int, default=0,
                    help="grid cap of the hook's kernels (0 = library default: the full persistent grid)")
    return ap.parse_args()


def build_model(name: str):
    """(model, vocabulary, sequence length): the same stock-torch classes for every arm."""

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from plain_models import PlainGPT2, PlainLlama

    if name == "gpt2-tiny":
        return PlainGPT2(2, 2, 64, 257, 32), 257, 32
    if name == "gpt2-small":
        return PlainGPT2(), 50257, 1024
    if name == "llama-tiny":
        return PlainLlama(2, 64, 4, 2, 128, 257, 32), 257, 32
    return PlainLlama(), 128256, 2048


def main() -> None:
    args = parse_args()
    # NCCL writes its version banner and warnings to stdout by default; the only stdout line of this
    # program is the JSON result, so NCCL's log goes to stderr.
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":   # NCCL honours the log file only above VERSION
        os.environ["NCCL_DEBUG"] = "WARN"
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_env

        ok, why = reference_env.reference_available()
        if not ok:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(free_port()))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    batch = args.batch or (2 if args.model == "llama-3b" else 8)
    bucket_mb = args.bucket_mb or (50 if args.model == "llama-3b" else 25)

    torch.manual_seed(1234)
    model, vocab, seq = build_model(args.model)
    model = model.to(device=device, dtype=torch.bfloat16)
    n_params = sum(p.numel() for p in model.parameters())
    ddp = DDP(model, device_ids=[local_rank], bucket_cap_mb=bucket_mb, gradient_as_bucket_view=True)

    hook = None
    ref_note = None
    if args.impl == "ours":
        from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook

        cfg = CompressionConfig(bit=8, group_size=64, topk=0, error_feedback=True, target="ddp_gradient_bucket")
        hook = create_ddp_comm_hook(cfg, strategy=args.strategy, reduce="mean", ef_mode=args.ef_mode,
                                    max_blocks=args.hook_max_blocks)
        ddp.register_comm_hook(state=None, hook=hook)
    elif args.impl == "reference":
        try:
            _, status = reference_env.activate(need_cuda_extension=True)
            from ccdl_comm.communication import create_ddp_comm_hook as ref_hook_factory
            from ccdl_comm.config import CompressionConfig as RefConfig

            rcfg = RefConfig(bit=8, group_size=64, topk=0, error_feedback=True, target="ddp_gradient_bucket")
            rhook = ref_hook_factory(rcfg, dtype="auto", strategy=args.ref_strategy, reduce="mean",
                                     async_gather=True, async_error_feedback=True)
            ddp.register_comm_hook(state=None, hook=rhook)
            ref_note = f"ccdl_comm hook strategy={args.ref_strategy} async_gather async_error_feedback"
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
            dist.destroy_process_group()
            return

    opt = torch.optim.AdamW(ddp.parameters(), lr=6e-4, fused=True)
    repeats = max(1, args.repeats)
    gen = torch.Generator().manual_seed(99 + rank)
    pool = args.warmup + 2 * args.steps            # distinct batches; regions draw from the pool in turn
    host_tokens = torch.randint(0, vocab, (pool, batch, seq + 1), generator=gen, dtype=torch.int64).pin_memory()

    def train_step(tok: "torch.Tensor"):
        loss = ddp(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    last = None
    for i in range(args.warmup):  # warm-up, end-to-end style
        last = train_step(host_tokens[i].to(device, non_blocking=True)).item()

    # settle: untimed for the result, timed only to decide when the clocks and the caches have settled
    settle_steps, settle_s = 0, 0.0
    if args.settle_s > 0:
        recent: list[float] = []
        t_start = time.perf_counter()
        while settle_steps < 2000:
            t0 = time.perf_counter()
            last = train_step(host_tokens[settle_steps % pool].to(device, non_blocking=True)).item()
            recent = (recent + [time.perf_counter() - t0])[-3:]
            settle_steps += 1
            elapsed = time.perf_counter() - t_start
            steady = len(recent) == 3 and max(recent) <= 1.02 * min(recent)
            flag = torch.tensor([1.0 if (steady and elapsed >= args.settle_s) or elapsed >= 10 * args.settle_s else 0.0],
                                device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)      # every rank leaves in the same step
            if flag.item() > 0:
                break
        settle_s = time.perf_counter() - t_start

    import gc

    def timed(fn) -> float:
        if args.gc_mode == "between":
            gc.collect()
            gc.disable()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        dist.barrier()
        if args.gc_mode == "between":
            gc.enable()
        ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    staged = [host_tokens[args.warmup + i].to(device) for i in range(args.steps)]
    losses: list[float] = []

    def device_region():     # device-resident inputs, no host read-back
        for tok in staged:
            train_step(tok)

    step_marks: list[list[float]] = []      # host clock after every read-back of an end-to-end region (diagnostic)

    def e2e_region():        # through the public API: H2D of the inputs and D2H of the loss, every step
        marks = [time.perf_counter()]
        for i in range(args.steps):
            tok = host_tokens[args.warmup + args.steps + i].to(device, non_blocking=True)
            losses.append(train_step(tok).item())
            marks.append(time.perf_counter())
        step_marks.append([round((b - a) * 1e3, 3) for a, b in zip(marks, marks[1:])])

    device_samples, e2e_samples, launches = [], [], 0
    for _ in range(repeats):
        launches_before = hook.gpu_launches() if hook is not None else 0
        device_samples.append(timed(device_region))
        launches = (hook.gpu_launches() - launches_before) if hook is not None else 0
        e2e_samples.append(timed(e2e_region))
    clocks = sampler.stop() if rank == 0 else None
    device_ms, e2e_ms = statistics.median(device_samples), statistics.median(e2e_samples)
    if hook is not None and hasattr(hook, "check_status"):
        hook.check_status()

    tokens_per_step = batch * seq * world
    value = tokens_per_step * args.steps / (device_ms * 1e-3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms * 1e-3)
    if rank == 0:
        line = {
            "metric": "GPT-2 DDP training throughput" if args.model.startswith("gpt2") else "Llama-style DDP training throughput",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "impl": args.impl,
            "config": {"model": args.model, "params": n_params, "global_batch": batch * world,
                       "micro_batch_per_gpu": batch, "seq_len": seq, "parallelism": f"dp{world}",
                       "optimizer": "AdamW lr 6e-4 (fused)", "bucket_cap_mb": bucket_mb,
                       "model_class": type(model).__name__ + " (baseline/plain_models.py)",
                       "hook": (f"lowbit_comm_b200 int8 g64 EF({args.ef_mode}) strategy={args.strategy} "
                                f"effective={getattr(hook, '_ccdl_effective_strategy', None)}") if args.impl == "ours"
                       else (ref_note or "none (NCCL bf16 all-reduce)"),
                       "l2": "inputs larger than L2 (a step touches >126 MB); no explicit flush"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": batch * (seq + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "timing": {"settle_steps": settle_steps, "settle_s": round(settle_s, 2), "repeats": repeats,
                       "value_ms_per_step_samples": [round(m / args.steps, 4) for m in device_samples],
                       "e2e_ms_per_step_samples": [round(m / args.steps, 4) for m in e2e_samples],
                       "e2e_host_ms_of_every_step": step_marks, "gc_mode": args.gc_mode,
                       "reported": "median of the samples; regions alternate value, e2e"},
            "clocks": clocks,
            "final_loss": losses[-1] if losses else last,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
