"""Real gloo ranks on CPU through the public collectives: the transports' host-side logic end to end."""

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
        from lowbit_comm_b200.ops import oracle
        from lowbit_comm_b200.parallel.backend_cuda import compile_cuda_shortcut

        cfg = lbc.CompressionConfig()
        n = 64 * 37 + 11
        xs = _inputs(world, n)
        payloads = [oracle.encode(x, cfg) for x in xs]
        one, _ = oracle.reduce_mean(payloads, n, cfg, "bf16")
        got = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy="all_gather")
        assert torch.equal(got.view(torch.uint8), one.view(torch.uint8))
        exact = torch.stack([x.float() for x in xs]).mean(0)
        for strategy in ("reduce_scatter", "topology", "auto", "hierarchical"):
            if strategy == "hierarchical" and world < 4:
                continue
            got = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy=strategy)
            assert ((got.float() - exact).norm() / exact.norm()).item() < 0.03, strategy
        # general profiles: one stage = the codec's in-dtype sum of the payloads, two stages = that result quantized
        # once more; the peer-memory kernels are held to the same two values on GPUs
        from lowbit_comm_b200.ops import codec

        for k in (1, 2):
            kcfg = lbc.CompressionConfig(topk=k, allow_experimental=True)
            packed = [codec.quantize_tensor(x, kcfg) for x in xs]
            y = codec.dequantize_reduce_tensors(packed, (n,), kcfg, dtype="bf16", reduce="mean")
            twice = codec.dequantize_tensor(codec.quantize_tensor(y, kcfg), (n,), kcfg, dtype="bf16")
            got = lbc.compressed_all_reduce(xs[rank].clone(), config=kcfg, strategy="all_gather")
            assert torch.equal(got.view(torch.uint8), y.view(torch.uint8)), k
            got = lbc.compressed_all_reduce(xs[rank].clone(), config=kcfg, strategy="reduce_scatter")
            assert torch.equal(got.view(torch.uint8), twice.view(torch.uint8)), k
        work = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy="all_gather", async_op=True)
        assert torch.equal(work.wait().view(torch.uint8), one.view(torch.uint8)) and work.query()
        summed = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, op="sum")
        assert ((summed.float() - exact * world).norm() / (exact * world).norm()).item() < 0.03

        shard = lbc.compressed_reduce_scatter_shard(xs[rank], config=cfg)
        assert shard.shard_index == rank and shard.world_size == world and shard.original_numel == n
        lo, valid = shard.shard_offset, shard.valid_numel
        assert valid == 0 or (shard.shard[:valid].float() - exact[lo:lo + valid]).abs().max() < 2e-3
        assert shard.shard[valid:].abs().sum() == 0 and shard.is_padding_only == (valid == 0)  # padding is zero
        out = torch.empty(shard.shard_numel, dtype=torch.bfloat16)
        again = lbc.compressed_reduce_scatter_shard(xs[rank], config=cfg, out=out)
        assert again.shard.data_ptr() == out.data_ptr() and again.metadata["caller_owned_output"]
        with pytest.raises(ValueError):
            lbc.compressed_reduce_scatter_shard(xs[rank], config=cfg, out=torch.empty(3, dtype=torch.bfloat16))
        full = lbc.compressed_reduce_scatter(xs[rank], config=cfg)
        assert ((full.float() - exact).norm() / exact.norm()).item() < 0.03

        parts = lbc.compressed_all_gather(xs[rank], config=cfg)
        for r in range(world):
            assert torch.equal(parts[r], oracle.decode(payloads[r], n, cfg, "bf16"))
        topk = lbc.CompressionConfig(topk=2)
        parts = lbc.compressed_all_gather(xs[rank], config=topk)
        assert torch.equal(parts[(rank + 1) % world], oracle.decode(oracle.encode(xs[(rank + 1) % world], topk), n, topk, "bf16"))

        ragged = torch.full((rank + 1, 3), float(rank), dtype=torch.float32)
        for protocol in ("object_v1", "tensor_v1"):
            got = lbc.compressed_all_gather_dynamic(ragged, config=cfg, metadata_protocol=protocol)
            assert [tuple(t.shape) for t in got] == [(r + 1, 3) for r in range(world)]
            assert all(torch.allclose(t, torch.full_like(t, float(r)), atol=0.02) for r, t in enumerate(got))
        empty = lbc.compressed_all_gather_dynamic(torch.empty(0, 4) if rank == 0 else ragged, config=cfg)
        assert tuple(empty[0].shape) == (0, 4)

        peer = (rank + 1) % world
        src = (rank - 1) % world
        recv = torch.empty(n, dtype=torch.bfloat16)
        w_recv = lbc.iqrecv(recv, src, config=cfg)
        lbc.qsend(xs[rank], peer, config=cfg)
        assert torch.equal(w_recv.wait(), oracle.decode(payloads[src], n, cfg, "bf16"))
        assert w_recv.execution_info.fast_path == "cuda_compiled_recv"

        t = torch.full((4,), float(rank + 1))
        assert lbc.all_reduce(t, op="sum").wait().tolist() == [world * (world + 1) / 2] * 4
        gathered = lbc.all_gather(torch.tensor([float(rank)])).wait()
        assert [g.item() for g in gathered] == list(range(world))
        b = torch.tensor([float(rank)])
        lbc.broadcast(b, src=1).wait()
        assert b.item() == 1.0
        lbc.barrier().wait()
        assert lbc.native_collectives()[0] == "all_reduce" and len(lbc.native_collectives()) == 9
        compiled = lbc.compile_collective(t, collective="all_reduce", op="max")
        assert compiled.execution_info.fast_path == "cuda_native_nccl"
        assert compiled.run(torch.tensor([float(rank)])).wait().item() == world - 1

        plan = compile_cuda_shortcut(xs[rank], collective="reduce_scatter", strategy="compressed", output_layout="shard",
                                     config=cfg)
        assert compile_cuda_shortcut(xs[rank], collective="reduce_scatter", strategy="compressed", output_layout="shard",
                                     config=cfg) is plan
        lease = plan.executor.acquire_output()
        work = plan.run(xs[rank], out=lease)
        result = work.wait()
        assert result.shard.data_ptr() == lease.buffer.data_ptr() and work.execution_info.fast_path == "torch_fallback"
        lease.release_after(result.shard)
        assert plan.executor.workspace_stats.in_flight_bytes == 0
        # the registry-free entry point with the reference's name
        from lowbit_comm_b200.parallel.backend_cuda import compile_cuda_plan, default_operation_factories

        assert ("all_reduce", "all_gather", "full") in default_operation_factories()
        direct = compile_cuda_plan(lbc.CommunicationPlan(collective="all_reduce", strategy="all_gather", compression=cfg,
                                                         async_op=False),
                                   lbc.CompileContext(rank=rank, world_size=world, device="cpu", shape=(n,), dtype="bf16"),
                                   allow_cpu=True)
        assert torch.equal(direct.run(xs[rank].clone()).wait().view(torch.uint8), one.view(torch.uint8))
        # payloads that are already gathered (the hook's path): fused decode + mean + residual, or payload by payload
        from lowbit_comm_b200.ops import codec, oracle
        from lowbit_comm_b200.parallel.backend_cuda import (FusedReducedShardCapability, PrecollectedPayloadExecution,
                                                            fused_reduced_shard_capability)

        payloads = [codec.quantize_tensor(x, cfg) for x in xs]
        out, residual = torch.empty_like(xs[rank]), torch.zeros_like(xs[rank])
        got = direct.run_precollected_payloads(payloads, xs[rank], out, residual).wait()
        y, y32 = oracle.reduce_mean(payloads, n, cfg, "bf16")
        assert got is out and torch.equal(out.view(torch.uint8), y.view(torch.uint8))
        assert torch.equal(residual.view(torch.uint8), oracle.residual_update(xs[rank], y32).view(torch.uint8))
        assert direct.last_execution_info.fast_path == "cuda_fused_dequant_reduce_mean_ef"
        topk = lbc.CompressionConfig(topk=1)
        general = compile_cuda_plan(lbc.CommunicationPlan(collective="all_reduce", strategy="all_gather", compression=topk),
                                    lbc.CompileContext(rank=rank, world_size=world, device="cpu", shape=(n,), dtype="bf16"),
                                    allow_cpu=True)
        payloads = [codec.quantize_tensor(x, topk) for x in xs]
        out2, residual2 = torch.empty_like(xs[rank]), torch.zeros_like(xs[rank])
        general.run_precollected_payloads(payloads, xs[rank], out2, residual2).wait()
        want = codec.dequantize_reduce_tensors(payloads, (n,), topk, dtype="bf16", reduce="mean")
        assert torch.equal(out2.view(torch.uint8), want.view(torch.uint8)) and residual2.abs().max() > 0
        assert general.last_execution_info.fallback_used and "fused" in general.last_execution_info.fallback_reason
        with pytest.raises(ValueError):
            PrecollectedPayloadExecution(out, False)
        with pytest.raises(ValueError):
            FusedReducedShardCapability(True, "but")
        shard_plan = lbc.CommunicationPlan(collective="reduce_scatter", strategy="compressed", output_layout="shard",
                                           compression=cfg)
        cpu_ctx = lbc.CompileContext(rank=rank, world_size=world, device="cpu", shape=(n,), dtype="bf16")
        gpu_ctx = lbc.CompileContext(rank=rank, world_size=world, device="cuda:0", shape=(n,), dtype="bf16")
        assert not fused_reduced_shard_capability(shard_plan, cpu_ctx, peer_access=True).available
        assert fused_reduced_shard_capability(shard_plan, gpu_ctx, peer_access=True).available
        assert "peer access" in fused_reduced_shard_capability(shard_plan, gpu_ctx, peer_access=False).reason
        auto = compile_cuda_shortcut(xs[rank], collective="all_reduce", strategy="auto", output_layout="full", config=cfg)
        assert auto.execution_info.requested_strategy == "auto"
        assert auto.execution_info.details["strategy_policy_id"] == "b200-nvlink5-v1"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", (2, 4))
def test_public_collectives_over_gloo(world):
    spawn_ranks(_worker, lambda port: (world, port), world)
