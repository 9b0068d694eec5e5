"""DDP hook strategies that the two-rank test does not reach, on four gloo ranks: hierarchical (2 x 2),
uncompressed pass-through, a hop-by-hop schedule injected as the topology transport, and resuming the
error-feedback state from a checkpoint."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLD = 4


def _worker(rank: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        import lowbit_comm_b200 as lbc
        from lowbit_comm_b200.models.mlp import SyntheticMLP

        cfg = lbc.CompressionConfig(target="ddp_gradient_bucket")

        def make_hook(mode):
            if mode == "hierarchical":
                return lbc.create_ddp_comm_hook(cfg, strategy="hierarchical", local_group_size=2)
            if mode == "native":
                return lbc.create_ddp_comm_hook(cfg, strategy="native_nccl")
            if mode == "p2p_hops":
                return lbc.create_ddp_comm_hook(cfg, strategy="topology",
                                                topology_all_reduce=lbc.make_schedule_all_reduce(method="p2p"))
            return None

        def train(mode, steps, resume_from=None, stop_at=None):
            torch.manual_seed(77)
            ddp = DDP(SyntheticMLP((64, 128, 64)), bucket_cap_mb=25)
            hook = make_hook(mode)
            if hook is not None:
                hook.bind_module(ddp.module)                   # parameter names: residuals survive bucket re-ordering
                ddp.register_comm_hook(state=None, hook=hook)
            opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
            gen = torch.Generator().manual_seed(500 + rank)
            saved = None
            for step in range(steps):
                x, y = torch.randn(16, 64, generator=gen), torch.randn(16, 64, generator=gen)
                if resume_from is not None and step == resume_from[0]:
                    hook.load_state_dict(resume_from[1])
                    with torch.no_grad():
                        for p, v in zip(ddp.parameters(), resume_from[2]):
                            p.copy_(v)
                if resume_from is not None and step < resume_from[0]:
                    continue                                   # data of the skipped steps was drawn above
                opt.zero_grad(set_to_none=True)
                torch.nn.functional.mse_loss(ddp(x), y).backward()
                opt.step()
                if stop_at is not None and step + 1 == stop_at:
                    saved = (stop_at, hook.state_dict(), [p.detach().clone() for p in ddp.parameters()])
            return torch.cat([p.detach().reshape(-1) for p in ddp.parameters()]), hook, saved

        plain, _, _ = train("plain", 4)
        results = {}
        for mode in ("hierarchical", "native", "p2p_hops"):
            params, hook, _ = train(mode, 4)
            gathered = [torch.empty_like(params) for _ in range(WORLD)]
            dist.all_gather(gathered, params)
            assert all(torch.equal(gathered[0], other) for other in gathered), mode      # ranks stay in lockstep
            drift = ((params - plain).norm() / plain.norm()).item()
            assert drift < (1e-6 if mode == "native" else 5e-3), (mode, drift)
            results[mode] = drift
            assert hook._ccdl_effective_strategy == {"hierarchical": "hierarchical", "native": "native_nccl",
                                                     "p2p_hops": "topology"}[mode]

        # checkpoint after 2 of 4 steps, resume in a fresh hook: same parameters as the uninterrupted run
        full, hook, saved = train("hierarchical", 4, stop_at=2)
        state = saved[1]
        assert state["feedback"] and any(v.abs().max() > 0 for v in state["feedback"]["residuals"].values())
        names = {name for name, _ in SyntheticMLP((64, 128, 64)).named_parameters()}
        assert set(state["residual_by_parameter"]) == names
        resumed, _, _ = train("hierarchical", 4, resume_from=saved)
        # the resumed process starts in DDP's first-iteration bucket order, the checkpoint was taken in the
        # rebuilt order: the per-parameter residuals make the continuation identical anyway
        assert torch.equal(resumed, full)
        if rank == 0:
            torch.save(results, os.path.join(out_dir, "drift.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(900)
def test_hook_strategies_and_resume_on_four_ranks(tmp_path):
    spawn_ranks(_worker, lambda port: (port, str(tmp_path)), WORLD)
    drift = torch.load(os.path.join(str(tmp_path), "drift.pt"))
    assert set(drift) == {"hierarchical", "native", "p2p_hops"}
