"""DDP with the compressed gradient hook on CPU ranks (gloo): no GPU needed.

    python examples/cpu_gloo_mlp.py [--ranks 2] [--steps 50] [--strategy all_gather]

Trains the synthetic MLP of the reference's CPU smoke configuration (1024 -> 4096 -> 4096 -> 1024, GELU, fp32,
batch 32 per rank, MSE loss, SGD) three times from the same seed -- plain DDP, the hook with the wire-format
codec (C++ on CPU), the hook with the simple torch-fallback codec -- and prints the loss curves side by side
with the time per step.  The hook keeps error-feedback residuals; its state is saved and reloaded half way
through the second run to show checkpointing.
"""

from __future__ import annotations

import argparse
import os
import socket
import sys
import tempfile
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODES = ("plain", "wire_codec", "fallback_codec")


def worker(rank: int, world: int, port: int, steps: int, strategy: str, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from torch.nn.parallel import DistributedDataParallel as DDP

    from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook
    from lowbit_comm_b200.models.mlp import SyntheticMLP
    from lowbit_comm_b200.ops.torch_fallback import dequantize_tensor_fallback, quantize_tensor_fallback
    from lowbit_comm_b200.parallel.payload_packing import make_payload_all_gather
    from lowbit_comm_b200.parallel.torch_transport import make_torch_all_gather

    cfg = CompressionConfig(bit=8, group_size=64, error_feedback=True, target="ddp_gradient_bucket")
    curves, times = {}, {}
    for mode in MODES:
        torch.manual_seed(1234)
        ddp = DDP(SyntheticMLP((1024, 4096, 4096, 1024)), bucket_cap_mb=25)
        hook = None
        if mode == "wire_codec":
            hook = create_ddp_comm_hook(cfg, strategy=strategy, module=ddp.module)
        elif mode == "fallback_codec":
            hook = create_ddp_comm_hook(cfg, strategy="all_gather", quantize=quantize_tensor_fallback,
                                        dequantize=dequantize_tensor_fallback,
                                        all_gather=make_payload_all_gather(make_torch_all_gather()))
        if hook is not None:
            ddp.register_comm_hook(state=None, hook=hook)
        opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
        gen = torch.Generator().manual_seed(100 + rank)
        losses = []
        dist.barrier()
        start = time.perf_counter()
        for step in range(steps):
            x, y = torch.randn(32, 1024, generator=gen), torch.randn(32, 1024, generator=gen)
            opt.zero_grad(set_to_none=True)
            loss = torch.nn.functional.mse_loss(ddp(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
            if mode == "wire_codec" and step == steps // 2:      # checkpoint round trip of the residuals
                path = os.path.join(out_dir, f"ef_{rank}.pt")
                torch.save(hook.state_dict(), path)
                hook.load_state_dict(torch.load(path))
        dist.barrier()
        curves[mode], times[mode] = losses, (time.perf_counter() - start) / steps
    if rank == 0:
        print(f"{world} gloo ranks, {steps} steps, hook strategy {strategy}")
        print("step  " + "  ".join(f"{m:>15s}" for m in MODES))
        for step in sorted({0, 1, 2, steps // 4, steps // 2, 3 * steps // 4, steps - 1}):
            print(f"{step:4d}  " + "  ".join(f"{curves[m][step]:15.6f}" for m in MODES))
        print("ms/step" + "".join(f"{times[m] * 1e3:17.1f}" for m in MODES))
        worst = max(abs(curves[m][-1] - curves["plain"][-1]) / abs(curves["plain"][-1]) for m in MODES[1:])
        print(f"largest relative difference of the final loss from plain DDP: {worst:.4%}")
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--strategy", default="all_gather", choices=("all_gather", "reduce_scatter", "hierarchical", "auto"))
    args = ap.parse_args()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as out_dir:
        mp.start_processes(worker, args=(args.ranks, port, args.steps, args.strategy, out_dir), nprocs=args.ranks,
                           start_method="spawn")


if __name__ == "__main__":
    main()
