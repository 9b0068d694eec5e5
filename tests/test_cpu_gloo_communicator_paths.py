"""Corners of the `Communicator`'s torch.distributed path on gloo ranks: error feedback with a residual,
caller-owned outputs, the uncompressed pass-through, and argument validation."""

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
        from lowbit_comm_b200.exceptions import UnsupportedCollective
        from lowbit_comm_b200.ops import oracle
        from lowbit_comm_b200.parallel.communicator import Communicator, get_communicator

        cfg = lbc.CompressionConfig()
        n = 64 * 11 + 9
        g = torch.Generator().manual_seed(7)
        xs = [(torch.randn(n, generator=g) * 0.02 * (r + 1)).to(torch.bfloat16) for r in range(world)]
        rs = [(torch.randn(n, generator=g) * 0.002).to(torch.bfloat16) for r in range(world)]
        comm = get_communicator(None)
        assert get_communicator(None) is comm and isinstance(comm, Communicator)

        # one stage with error feedback: residual = prepared - fp32 mean (the reference's rule), result into `out`
        prepared = [oracle.prepare(x, r) for x, r in zip(xs, rs)]
        payloads = [oracle.encode(p, cfg) for p in prepared]
        y, y32 = oracle.reduce_mean(payloads, n, cfg, "bf16")
        x, residual, out = xs[rank].clone(), rs[rank].clone(), torch.empty(n, dtype=torch.bfloat16)
        got = comm.all_reduce(x, config=cfg, op="mean", strategy="all_gather", out=out, residual=residual)
        assert got is out and torch.equal(out.view(torch.uint8), y.view(torch.uint8)) and torch.equal(x, xs[rank])
        assert torch.equal(residual.view(torch.uint8),
                           oracle.residual_update_from_restored(prepared[rank], y).view(torch.uint8))
        kept = rs[rank].clone()
        comm.all_reduce(xs[rank].clone(), config=cfg, strategy="all_gather", residual=kept, update_residual=False)
        assert torch.equal(kept, rs[rank])

        # uncompressed pass-through and asynchronous form
        exact = torch.stack([v.float() for v in xs]).mean(0)
        plain = comm.all_reduce(xs[rank].clone().float(), config=cfg, op="mean", strategy="native_nccl")
        assert torch.allclose(plain, exact, atol=1e-6)
        work = comm.all_reduce(xs[rank].clone(), config=cfg, op="sum", strategy="native_nccl", async_op=True)
        assert torch.allclose(work.wait().float(), exact * world, atol=0.05)

        with pytest.raises(UnsupportedCollective, match="unknown strategy"):
            comm.all_reduce(xs[rank].clone(), config=cfg, strategy="gossip")
        with pytest.raises(UnsupportedCollective, match="only op="):
            comm.all_reduce(xs[rank].clone(), config=cfg, op="max")
        with pytest.raises(UnsupportedCollective, match="only op="):
            comm.reduce_scatter_shard(xs[rank].clone(), config=cfg, op="min")

        # caller-owned shard output: shape, dtype, contiguity and aliasing are checked before anything is sent
        shard = comm.reduce_scatter_shard(xs[rank].clone(), config=cfg, op="mean")
        mine = torch.empty(shard.shard_numel, dtype=torch.bfloat16)
        again = comm.reduce_scatter_shard(xs[rank].clone(), config=cfg, op="mean", out=mine)
        assert again.shard.data_ptr() == mine.data_ptr() and again.metadata["caller_owned_output"]
        assert torch.equal(mine.view(torch.uint8), shard.shard.view(torch.uint8))
        check = Communicator._validated_out
        src = xs[rank].clone()
        with pytest.raises(ValueError, match="shape"):
            check(torch.empty(shard.shard_numel + 1, dtype=torch.bfloat16), src, shard.shard_numel)
        with pytest.raises(TypeError, match="dtype"):
            check(torch.empty(shard.shard_numel, dtype=torch.float32), src, shard.shard_numel)
        with pytest.raises(ValueError, match="contiguous"):
            check(torch.empty(2 * shard.shard_numel, dtype=torch.bfloat16)[::2], src, shard.shard_numel)
        with pytest.raises(ValueError, match="alias"):
            check(src[: shard.shard_numel], src, shard.shard_numel)
        assert check(None, src, 5).shape == (5,)
        with pytest.raises(UnsupportedCollective, match="multiple of the local group size"):
            comm.hierarchical_all_reduce(xs[rank].clone(), config=cfg, local_group_size=world + 1)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 3))
def test_communicator_torch_path_corners(world):
    spawn_ranks(_worker, lambda port: (world, port), world)
