"""Loss-curve comparison: the same GPT-2 DDP run with plain NCCL bf16 gradients and with the
int8 group-64 hook (both error-feedback rules), same seeds, same synthetic data.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29531 benchmarks/loss_curve.py [--model gpt2-small --steps 60 --batch 8]

Two controls put the gap in context: `nccl_bf16_noise` multiplies every gradient element by
(1 + 0.017 * N(0, 1)) before the NCCL all-reduce (the relative error of int8 group-64 payloads,
without its structure), and `reference_hook` registers the unmodified reference's own hook
(`--with-reference`, needs baseline/_ref) on the same model.

The data is learnable (token t+1 = (a * token t + b) mod V with 10 % noise), so the loss falls
during the run and a broken gradient path shows up as a diverging curve.  The reference compares
20-50-step synthetic training losses against DDP the same way
(tests/benchmarks/reports/full_compare_20260728/README.md:36-43).  Output: one JSON line per arm
with the loss every 5 steps, then a summary line with the largest gap to the NCCL arm.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def make_tokens(torch, steps: int, batch: int, seq: int, vocab: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    first = torch.randint(0, vocab, (steps, batch, 1), generator=gen)
    noise = torch.rand(steps, batch, seq + 1, generator=gen) < 0.1
    rand = torch.randint(0, vocab, (steps, batch, seq + 1), generator=gen)
    tok = torch.empty(steps, batch, seq + 1, dtype=torch.int64)
    tok[:, :, :1] = first
    for t in range(1, seq + 1):
        nxt = (tok[:, :, t - 1] * 31 + 7) % vocab
        tok[:, :, t] = torch.where(noise[:, :, t], rand[:, :, t], nxt)
    return tok


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=("gpt2-small", "gpt2-tiny"), default="gpt2-small")
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--with-reference", action="store_true")
    ap.add_argument("--out", default="bench_out/loss_curve.json")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29532")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook
    from lowbit_comm_b200.models import GPT2, GPT2Config

    mcfg = GPT2Config() if args.model == "gpt2-small" else GPT2Config.tiny()
    tokens = make_tokens(torch, args.steps, args.batch, mcfg.seq_len, mcfg.vocab_size, 4242 + rank).pin_memory()

    def run(arm: str) -> list[float]:
        torch.manual_seed(1234)
        model = GPT2(mcfg).to(device=dev, dtype=torch.bfloat16)
        ddp = DDP(model, device_ids=[local], bucket_cap_mb=25, gradient_as_bucket_view=True)
        hook = None
        if arm == "nccl_bf16_noise":
            def noisy(state, bucket):
                buf = bucket.buffer()
                buf.mul_(1 + 0.017 * torch.randn_like(buf))
                fut = dist.all_reduce(buf, op=dist.ReduceOp.AVG, async_op=True).get_future()
                return fut.then(lambda f: f.value()[0])

            ddp.register_comm_hook(state=None, hook=noisy)
        elif arm == "reference_hook":
            from ccdl_comm.communication import create_ddp_comm_hook as ref_factory
            from ccdl_comm.config import CompressionConfig as RefConfig

            rcfg = RefConfig(bit=8, group_size=64, topk=0, error_feedback=True, target="ddp_gradient_bucket")
            ddp.register_comm_hook(state=None, hook=ref_factory(rcfg, dtype="auto", strategy="all_gather",
                                                                reduce="mean", async_gather=True,
                                                                async_error_feedback=True))
        elif arm != "nccl_bf16":
            cfg = CompressionConfig(bit=8, group_size=64, topk=0, error_feedback=True, target="ddp_gradient_bucket")
            hook = create_ddp_comm_hook(cfg, strategy="auto", reduce="mean", ef_mode=arm.split(":")[1])
            ddp.register_comm_hook(state=None, hook=hook)
        opt = torch.optim.AdamW(ddp.parameters(), lr=args.lr, fused=True)
        losses = []
        for i in range(args.steps):
            tok = tokens[i].to(dev, non_blocking=True)
            loss = ddp(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            t = loss.detach().float().clone()
            dist.all_reduce(t, op=dist.ReduceOp.AVG)
            losses.append(float(t.item()))
        del ddp, opt, model
        torch.cuda.empty_cache()
        return losses

    arms = ["nccl_bf16", "nccl_bf16_noise", "int8_g64:reference", "int8_g64:local"]
    if args.with_reference:
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import reference_env

            reference_env.activate(need_cuda_extension=True)
            arms.append("reference_hook")
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"arm": "reference_hook", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
    curves = {}
    for arm in arms:
        curves[arm] = run(arm)
        if rank == 0:
            print(json.dumps({"arm": arm, "world": world, "model": args.model,
                              "loss_every_5": [round(v, 4) for v in curves[arm][::5]],
                              "final": curves[arm][-1]}), flush=True)
    if rank == 0:
        base = curves["nccl_bf16"]
        summary = {"summary": True, "world": world, "steps": args.steps}
        for arm, c in curves.items():
            if arm == "nccl_bf16":
                continue
            gaps = [abs(a - b) for a, b in zip(c, base)]
            tail = max(1, args.steps // 6)
            summary[arm] = {"max_abs_gap": max(gaps), "mean_gap_last_steps": sum(gaps[-tail:]) / tail,
                            "final_rel_gap": abs(c[-1] - base[-1]) / abs(base[-1])}
        print(json.dumps(summary), flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump({"curves": curves, "summary": summary}, open(args.out, "w"), indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
