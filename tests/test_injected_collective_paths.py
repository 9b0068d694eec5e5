"""The generic compositions behind `compressed_all_reduce` / `compressed_all_gather` when the caller injects
the codec or the transport (the reference's calling convention), with a two-rank world faked in one process."""

import pytest
import torch

import lowbit_comm_b200 as lbc
from lowbit_comm_b200.exceptions import UnsupportedCollective
from lowbit_comm_b200.ops import codec, oracle
from lowbit_comm_b200.parallel.payload import CompressedPayload, GatheredPayloads, payload_buffer

CFG = lbc.CompressionConfig()


def _x(n=64 * 5 + 3, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * 0.05).to(torch.bfloat16)


def _peer_payload(x):
    return CompressedPayload(buffer=codec.quantize_tensor(-x * 0.5, CFG), shape=tuple(x.shape), dtype="bf16",
                             metadata={})


def _fake_gather(x):
    """A two-rank all-gather: this rank's payload plus the payload of a peer that holds -x / 2."""

    def gather(payload):
        return GatheredPayloads(payloads=[payload, _peer_payload(x)], world_size=2)

    return gather


def test_all_gather_reduce_composition_with_default_and_injected_codec():
    x = _x()
    want_parts = [oracle.decode(codec.quantize_tensor(v, CFG), x.numel(), CFG, "bf16") for v in (x, -x * 0.5)]
    got = lbc.compressed_all_reduce(x.clone(), config=CFG, op="mean", all_gather=_fake_gather(x))
    assert torch.equal(got, (want_parts[0] + want_parts[1]) / 2)
    calls = []

    def q(t, cfg):
        calls.append("q")
        return codec.quantize_tensor(t, cfg)

    def dq(payload, shape, cfg, name):
        calls.append("dq")
        return codec.dequantize_tensor(payload_buffer(payload), shape, cfg, dtype=name)

    work = lbc.compressed_all_reduce(x.clone(), config=CFG, op="sum", async_op=True, quantize=q, dequantize=dq,
                                     all_gather=_fake_gather(x))
    assert not calls                                              # the asynchronous form runs when it is waited on
    assert torch.equal(work.wait(), want_parts[0] + want_parts[1]) and calls == ["q", "dq", "dq"]


def test_payload_all_reduce_strategy_needs_and_uses_the_injected_transport():
    x = _x(seed=1)
    with pytest.raises(UnsupportedCollective, match="must be injected"):
        lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="all_reduce", quantize=codec.quantize_tensor)
    seen = []

    def payload_all_reduce(payload, reduce):
        seen.append(reduce)
        return payload                                            # a one-rank world: the sum is the payload itself

    got = lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="all_reduce", op="sum", all_reduce=payload_all_reduce)
    assert seen == ["sum"] and torch.equal(got, oracle.decode(codec.quantize_tensor(x, CFG), x.numel(), CFG, "bf16"))


def test_topology_strategy_routes_to_the_injected_transport_and_validates_names():
    x = _x(seed=2)

    def transport(tensor, *, config, op, async_op, dtype, extension_status):
        return tensor * 2

    assert torch.equal(lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="topology",
                                                 topology_all_reduce=transport), x * 2)
    work = lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="topology", async_op=True,
                                     topology_all_reduce=transport)
    assert torch.equal(work.wait(), x * 2)
    with pytest.raises(UnsupportedCollective, match="no topology transport"):
        lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="topology", quantize=codec.quantize_tensor)
    with pytest.raises(UnsupportedCollective, match="supported strategies"):
        lbc.compressed_all_reduce(x.clone(), config=CFG, strategy="butterfly-ish")
    with pytest.raises(UnsupportedCollective, match="only op="):
        lbc.compressed_all_reduce(x.clone(), config=CFG, op="max")

    class Plan:
        def run(self, tensor):
            return lbc.ImmediateWork(tensor + 1)

    assert torch.equal(lbc.compressed_all_reduce(x.clone(), config=CFG, compiled_plan=Plan()), x + 1)
    assert torch.equal(lbc.compressed_all_reduce(x.clone(), config=CFG, compiled_plan=Plan(), async_op=True).wait(), x + 1)


def test_all_gather_with_injected_transport_and_codec():
    x = _x(seed=3)
    outs = lbc.compressed_all_gather(x.clone(), config=CFG, all_gather=_fake_gather(x))
    assert len(outs) == 2 and torch.equal(outs[0], oracle.decode(codec.quantize_tensor(x, CFG), x.numel(), CFG, "bf16"))
    assert torch.equal(outs[1], oracle.decode(codec.quantize_tensor(-x * 0.5, CFG), x.numel(), CFG, "bf16"))
    marks = []
    work = lbc.compressed_all_gather(
        x.clone(), config=CFG, async_op=True, all_gather=_fake_gather(x),
        quantize=lambda t, cfg: marks.append("q") or codec.quantize_tensor(t, cfg),
        dequantize=lambda p, shape, cfg, name: marks.append("dq") or codec.dequantize_tensor(
            payload_buffer(p), shape, cfg, dtype=name))
    assert [o.shape for o in work.wait()] == [x.shape, x.shape] and marks == ["q", "dq", "dq"]


def test_gathered_payloads_accepts_and_checks_world_size():
    assert GatheredPayloads([1, 2]).world_size == 2 and GatheredPayloads(payloads=[1], world_size=1).payloads == (1,)
    with pytest.raises(ValueError, match="does not match"):
        GatheredPayloads(payloads=[1, 2], world_size=3)


def test_shard_workspace_cache_byte_budget_and_allocators():
    from lowbit_comm_b200.parallel.workspace import ShardCommunicationWorkspaceCache

    made = []

    def quantized(tensor, config, dtype):
        made.append(("q", dtype))
        return torch.empty(100, dtype=torch.uint8)

    def reduced(tensor, shape, config):
        made.append(("r", shape))
        return torch.empty(shape, dtype=tensor.dtype)

    cache = ShardCommunicationWorkspaceCache(quantized_allocator=quantized, reduced_allocator=reduced,
                                             max_cached_bytes=250)
    x = torch.zeros(64, dtype=torch.bfloat16)
    a = cache.get_quantized_chunk("b0", 0, x, CFG, dtype="bf16", world_size=2)
    b = cache.get_quantized_chunk("b0", 1, x, CFG, dtype="bf16", world_size=2)
    assert cache.get_quantized_chunk("b0", 0, x, CFG, dtype="bf16", world_size=2) is a and cache.cached_bytes == 200
    r = cache.get_reduced_shard("b0", x, (32,), CFG, dtype="bf16", world_size=2, rank=1)      # 64 bytes: over budget
    assert len(cache) == 2 and cache.cached_bytes == 164                                        # chunk 1 was least recent
    assert cache.get_quantized_chunk("b0", 0, x, CFG, dtype="bf16", world_size=2) is a
    assert cache.get_quantized_chunk("b0", 1, x, CFG, dtype="bf16", world_size=2) is not b
    assert made.count(("q", "bf16")) == 3 and made.count(("r", (32,))) == 1 and r.shape == (32,)
    huge = ShardCommunicationWorkspaceCache(max_cached_bytes=10)
    assert huge.get_quantized_chunk("k", 0, x, CFG, dtype="bf16", world_size=2).numel() > 10 and len(huge) == 0
    cache.clear()
    assert len(cache) == 0 and cache.cached_bytes == 0
    with pytest.raises(ValueError):
        ShardCommunicationWorkspaceCache(max_entries=0)
    with pytest.raises(ValueError):
        ShardCommunicationWorkspaceCache(max_cached_bytes=-1)
