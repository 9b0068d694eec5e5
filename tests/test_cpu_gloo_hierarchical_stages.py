"""A hierarchical plan that spells out its three stages, compiled and run on four gloo ranks as 2 x 2."""

import os
import sys

import pytest
import torch
import torch.distributed as dist

from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import lowbit_comm_b200 as lbc
        from lowbit_comm_b200.core.hierarchy import canonical_hierarchical_stages
        from lowbit_comm_b200.parallel.backend_cuda import compile_cuda_plan

        cfg = lbc.CompressionConfig()
        n = 64 * 23 + 9
        g = torch.Generator().manual_seed(0)
        xs = [(torch.randn(n, generator=g) * 0.01 * (r + 1)).to(torch.bfloat16) for r in range(world)]
        exact = torch.stack([x.float() for x in xs]).mean(0)
        ctx = lbc.CompileContext(rank=rank, world_size=world, device="cpu", shape=(n,), dtype="bf16",
                                 local_rank=rank % 2, local_world_size=2, node_id=rank // 2, node_count=2)
        for gather in ("native_nccl", "compressed"):
            plan = lbc.CommunicationPlan(collective="all_reduce", strategy="hierarchical", compression=cfg,
                                         async_op=False,
                                         stages=canonical_hierarchical_stages(cfg, gather_strategy=gather))
            executor = compile_cuda_plan(plan, ctx, allow_cpu=True)
            assert executor.execution_info.stage_names == ("local_reduce_scatter", "inter_all_reduce", "local_all_gather")
            got = executor.run(xs[rank].clone()).wait()
            assert got.shape == (n,) and got.dtype == torch.bfloat16
            rel = ((got.float() - exact).norm() / exact.norm()).item()
            assert rel < 0.03, (gather, rel)
            everyone = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(everyone, got)
            assert all(torch.equal(e, everyone[0]) for e in everyone), gather      # one result on all four ranks
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_staged_hierarchical_plan_on_two_by_two():
    spawn_ranks(_worker, lambda port: (4, port), 4)
