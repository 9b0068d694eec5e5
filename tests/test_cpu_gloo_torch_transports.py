"""The plain `torch.distributed` transports (payload all-gather / all-reduce, tensor all-reduce, their
asynchronous forms) on gloo ranks, and their behaviour without an initialised process group."""

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
        from lowbit_comm_b200.parallel.payload import CompressedPayload, GatheredPayloads
        from lowbit_comm_b200.parallel.torch_transport import (AsyncAllGatherWork, make_torch_all_gather,
                                                               make_torch_all_reduce, make_torch_async_all_gather,
                                                               make_torch_async_all_reduce,
                                                               make_torch_tensor_all_reduce)

        mine = torch.full((8,), rank + 1, dtype=torch.uint8)
        gathered = make_torch_all_gather()(mine)
        assert isinstance(gathered, GatheredPayloads) and gathered.world_size == world
        assert [int(p[0]) for p in gathered.payloads] == list(range(1, world + 1))
        work = make_torch_async_all_gather()(CompressedPayload(mine.clone(), (8,), "bf16"))
        assert isinstance(work, AsyncAllGatherWork)
        later = work.wait()
        assert work.is_completed() and [int(p[0]) for p in later.payloads] == list(range(1, world + 1))
        future = work.get_future()
        assert future is None or hasattr(future, "wait")

        total = world * (world + 1) // 2
        payload = CompressedPayload(mine.clone(), (8,), "bf16")
        assert make_torch_all_reduce()(payload, "sum") is payload and int(payload.buffer[0]) == total
        payload = CompressedPayload(mine.clone(), (8,), "bf16")
        handle = make_torch_async_all_reduce()(payload, "sum")
        assert handle.wait() is payload and int(payload.buffer[3]) == total

        plain = make_torch_tensor_all_reduce()
        x = torch.full((5,), float(rank + 1))
        assert plain(x, "mean") is x and torch.allclose(x, torch.full((5,), total / world))
        assert torch.equal(plain(torch.full((5,), float(rank + 1)), "max"), torch.full((5,), float(world)))
        with pytest.raises(ValueError, match="unsupported torch.distributed reduce op"):
            plain(torch.zeros(1), "median")
        if world >= 4:
            pair = dist.new_group([0, 2], backend="gloo")
            if rank in (0, 2):
                y = torch.full((3,), float(rank))
                assert torch.equal(make_torch_tensor_all_reduce(group=pair)(y, "mean"), torch.full((3,), 1.0))
                assert make_torch_all_gather(group=pair)(mine).world_size == 2
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 4))
def test_torch_transports_over_gloo(world):
    spawn_ranks(_worker, lambda port: (world, port), world)


def test_transports_say_when_there_is_no_process_group():
    from lowbit_comm_b200.exceptions import TorchDistributedUnavailableError
    from lowbit_comm_b200.parallel.torch_transport import make_torch_all_gather, make_torch_tensor_all_reduce

    assert not dist.is_initialized()
    with pytest.raises(TorchDistributedUnavailableError, match="not initialized"):
        make_torch_all_gather()(torch.zeros(4, dtype=torch.uint8))

    def no_torch(name):
        raise ImportError(name)

    with pytest.raises(TorchDistributedUnavailableError, match="not available"):
        make_torch_tensor_all_reduce(import_module=no_torch)(torch.zeros(1), "sum")
