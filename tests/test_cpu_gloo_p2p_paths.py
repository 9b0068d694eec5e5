"""Quantized point-to-point over torch.distributed on gloo ranks: compiled endpoints reused across messages,
blocking and non-blocking forms, endpoint validation, and what `transport=` accepts without a mailbox."""

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
        from lowbit_comm_b200.exceptions import CCDLError
        from lowbit_comm_b200.ops import codec, oracle

        cfg = lbc.CompressionConfig(error_feedback=False, target="p2p")
        n = 64 * 7 + 5
        g = torch.Generator().manual_seed(11)
        messages = [(torch.randn(n, generator=g) * 0.03).to(torch.bfloat16) for _ in range(3)]
        want = [oracle.decode(oracle.encode(m, cfg), n, cfg, "bf16") for m in messages]
        if rank == 0:
            endpoint = lbc.compile_qsend(messages[0], 1, config=cfg, tag=3)
            for m in messages:                                   # one compiled endpoint, many messages
                lbc.qsend(m, 1, config=cfg, compiled_executor=endpoint)
            assert endpoint.execution_counters.snapshot().run_calls == 3
            assert endpoint.execution_info.compressed_bytes == codec.quantize_tensor(messages[0], cfg).numel()
            with pytest.raises(ValueError, match="does not match compiled shape"):
                endpoint.run(torch.zeros(n + 1, dtype=torch.bfloat16))
            with pytest.raises(TypeError, match="does not match compiled dtype"):
                endpoint.run(torch.zeros(n, dtype=torch.float32))
            assert endpoint.execution_counters.snapshot().failed_runs == 2
            lbc.qsend(messages[0], 1, config=cfg, transport="auto")      # no mailbox on CPU tensors: torch send
        elif rank == 1:
            endpoint = lbc.compile_qrecv(torch.empty(n, dtype=torch.bfloat16), 0, config=cfg, tag=3)
            for w in want:
                got = lbc.qrecv(torch.empty(n, dtype=torch.bfloat16), 0, config=cfg, compiled_executor=endpoint)
                assert torch.equal(got.view(torch.uint8), w.view(torch.uint8))
            got = lbc.qrecv(torch.empty(n, dtype=torch.bfloat16), None, config=cfg)      # from whoever sends
            assert torch.equal(got.view(torch.uint8), want[0].view(torch.uint8))
        with pytest.raises(CCDLError):
            lbc.iqsend(messages[0], (rank + 1) % world, config=cfg, transport="peer")   # CPU tensors have no mailbox
        with pytest.raises(ValueError, match="transport must be"):
            lbc.iqsend(messages[0], (rank + 1) % world, config=cfg, transport="carrier-pigeon")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_quantized_p2p_over_gloo():
    spawn_ranks(_worker, lambda port: (2, port), 2)


def test_endpoint_arguments_are_validated_without_a_process_group():
    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.p2p import CudaP2PExecutor, compile_p2p_executor

    x, cfg = torch.zeros(64, dtype=torch.bfloat16), CompressionConfig()
    for bad in (dict(direction="both", peer=0), dict(direction="send", peer=None), dict(direction="recv", peer=-1),
                dict(direction="recv", peer=True), dict(direction="send", peer=1, tag=-1)):
        with pytest.raises(ValueError):
            CudaP2PExecutor(tensor=x, config=cfg, **bad)
    with pytest.raises(TypeError):
        CudaP2PExecutor(direction="send", peer=1, tensor=x, config={"bit": 8})
    endpoint = compile_p2p_executor(direction="recv", peer=None, tensor=x, config=cfg)
    assert isinstance(endpoint, CudaP2PExecutor) and endpoint.execution_info.backend == "cuda"
