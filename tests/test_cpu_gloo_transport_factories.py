"""The reference's transport factories (names and calling convention), injected into the public
collectives and into the DDP hook, on real gloo ranks."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(world, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * 0.01 * (r + 1)).to(torch.bfloat16) for r in range(world)]


def _worker(rank: int, world: int, port: int) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import lowbit_comm_b200 as lbc
        from lowbit_comm_b200.exceptions import UnsupportedCollective
        from lowbit_comm_b200.ops import oracle
        from lowbit_comm_b200.parallel.fused import geometry

        cfg = lbc.CompressionConfig()
        n = 64 * 41 + 3
        xs = _inputs(world, n)
        payloads = [oracle.encode(x, cfg) for x in xs]
        one, _ = oracle.reduce_mean(payloads, n, cfg, "bf16")
        two = oracle.decode(oracle.encode(one, cfg), n, cfg, "bf16")
        exact = torch.stack([x.float() for x in xs]).mean(0)

        shard_t = lbc.make_torch_compressed_reduce_scatter_shard()
        full_t = lbc.make_torch_compressed_reduce_scatter_all_gather()
        ring_t = lbc.make_native_topology_all_reduce(method="ring")
        gather_t = lbc.make_native_topology_all_reduce(method="overlap-gather")
        topo_shard_t = lbc.make_native_topology_reduce_scatter_shard(method="p2p")

        geo = geometry(n, world, "bf16", cfg)
        padded = torch.zeros(geo.shard_numel * world, dtype=torch.bfloat16)
        padded[:n] = one
        want_shard = padded[rank * geo.shard_numel:(rank + 1) * geo.shard_numel]
        for transport in (shard_t, topo_shard_t):
            shard = lbc.compressed_reduce_scatter_shard(xs[rank].clone(), config=cfg, reduce_scatter_shard=transport)
            assert shard.shard_index == rank and torch.equal(shard.shard.view(torch.uint8), want_shard.view(torch.uint8))
        got = lbc.compressed_reduce_scatter(xs[rank].clone(), config=cfg, reduce_scatter=full_t)
        assert torch.equal(got.view(torch.uint8), two.view(torch.uint8))
        got = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy="topology", topology_all_reduce=ring_t)
        assert torch.equal(got.view(torch.uint8), two.view(torch.uint8))
        got = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy="topology", topology_all_reduce=gather_t)
        assert torch.equal(got.view(torch.uint8), one.view(torch.uint8))
        work = ring_t(xs[rank].clone(), config=cfg, op="mean", async_op=True, dtype="bf16", extension_status=None)
        assert torch.equal(work.wait().view(torch.uint8), two.view(torch.uint8))
        if world % 2 == 0 and world >= 4:
            hier_t = lbc.make_torch_hierarchical_all_reduce(local_group_size=2)
            got = lbc.compressed_hierarchical_all_reduce(xs[rank].clone(), config=cfg, hierarchical_all_reduce=hier_t)
            rel = ((got.float() - exact).norm() / exact.norm()).item()
            assert rel < 0.03, rel
        with pytest.raises(UnsupportedCollective):
            lbc.make_native_topology_all_reduce(method="carrier-pigeon")
        with pytest.raises(UnsupportedCollective):
            ring_t(xs[rank], config=cfg, op="max", async_op=False, dtype="bf16", extension_status=None)

        # the DDP hook with an injected topology transport
        from torch.nn.parallel import DistributedDataParallel as DDP

        torch.manual_seed(0)
        model = torch.nn.Linear(64, 32)
        ddp = DDP(model)
        hook = lbc.create_ddp_comm_hook(lbc.CompressionConfig(error_feedback=False), strategy="topology",
                                        topology_all_reduce=ring_t)
        ddp.register_comm_hook(None, hook)
        x = torch.randn(8, 64, generator=torch.Generator().manual_seed(10 + rank))
        ddp(x).square().mean().backward()
        grads = [torch.zeros_like(model.weight.grad) for _ in range(world)]
        dist.all_gather(grads, model.weight.grad)
        assert all(torch.equal(g, grads[0]) for g in grads)          # every rank holds the same reduced gradient
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", (2, 4))
def test_transport_factories_over_gloo(world):
    spawn_ranks(_worker, lambda port: (world, port), world)
