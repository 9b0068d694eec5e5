"""Two real gloo ranks on CPU: DDP + compressed hook vs an uncompressed run.

This is the CPU/gloo configuration of the benchmark list: MLP
1024->4096->4096->1024 (GELU, fp32), batch 32, MSE loss, int8 group-64 hook
with error feedback, torch-fallback codec, 25 MB buckets.  A shorter run keeps
the test fast; `examples/cpu_gloo_mlp.py` runs the full 50 steps.
"""

import os
import sys

import pytest
import torch
import torch.distributed as dist
from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, mode: str, steps: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook
        from lowbit_comm_b200.models.mlp import SyntheticMLP
        from lowbit_comm_b200.ops.torch_fallback import dequantize_tensor_fallback, quantize_tensor_fallback
        from lowbit_comm_b200.parallel.payload_packing import make_payload_all_gather
        from lowbit_comm_b200.parallel.torch_transport import make_torch_all_gather

        torch.manual_seed(1234)
        model = SyntheticMLP((256, 512, 512, 256))
        ddp = DDP(model, bucket_cap_mb=25)
        cfg = CompressionConfig(bit=8, group_size=64, topk=0, error_feedback=True, target="ddp_gradient_bucket")
        hook = None
        if mode == "fallback_codec":
            hook = create_ddp_comm_hook(cfg, strategy="all_gather", quantize=quantize_tensor_fallback,
                                        dequantize=dequantize_tensor_fallback,
                                        all_gather=make_payload_all_gather(make_torch_all_gather()))
        elif mode == "wire_codec":
            hook = create_ddp_comm_hook(cfg, strategy="all_gather")
        elif mode == "wire_codec_rs":
            hook = create_ddp_comm_hook(cfg, strategy="reduce_scatter")
        if hook is not None:
            ddp.register_comm_hook(state=None, hook=hook)
        opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
        gen = torch.Generator().manual_seed(100 + rank)
        losses, grads = [], None
        for _ in range(steps):
            x = torch.randn(32, 256, generator=gen)
            y = torch.randn(32, 256, generator=gen)
            opt.zero_grad(set_to_none=True)
            loss = torch.nn.functional.mse_loss(ddp(x), y)
            loss.backward()
            if grads is None:
                grads = torch.cat([p.grad.reshape(-1) for p in ddp.parameters()]).clone()
            opt.step()
            losses.append(loss.item())
        torch.save({"losses": losses, "grads": grads,
                    "params": torch.cat([p.detach().reshape(-1) for p in ddp.parameters()])},
                   os.path.join(out_dir, f"{mode}_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(mode: str, steps: int, out_dir: str) -> None:
    spawn_ranks(_worker, lambda port: (2, port, mode, steps, out_dir), 2)


@pytest.mark.timeout(600)
def test_compressed_hook_tracks_uncompressed_ddp(tmp_path):
    out = str(tmp_path)
    steps = 12
    for mode in ("plain", "fallback_codec", "wire_codec", "wire_codec_rs"):
        _run(mode, steps, out)
    plain = torch.load(os.path.join(out, "plain_0.pt"))
    for mode in ("fallback_codec", "wire_codec", "wire_codec_rs"):
        got0 = torch.load(os.path.join(out, f"{mode}_0.pt"))
        got1 = torch.load(os.path.join(out, f"{mode}_1.pt"))
        # both ranks hold the same averaged gradient and the same parameters
        assert torch.equal(got0["grads"], got1["grads"]), mode
        assert torch.equal(got0["params"], got1["params"]), mode
        rel = ((got0["grads"] - plain["grads"]).norm() / plain["grads"].norm()).item()
        assert rel < 0.02, (mode, rel)  # int8 group-64 quantisation tolerance (two stages for rs)
        assert abs(got0["losses"][-1] - plain["losses"][-1]) < 0.02 * abs(plain["losses"][-1]) + 1e-3, mode
        drift = ((got0["params"] - plain["params"]).norm() / plain["params"].norm()).item()
        assert drift < 5e-3, (mode, drift)
