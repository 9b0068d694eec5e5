"""Dynamic-shape compressed all-gather with a fabricated torch.distributed: one simulated rank, the other
ranks' metadata and payloads are produced by the fake (the reference's test style for transports,
tests/test_dynamic_all_gather.py)."""

import importlib

import pytest
import torch

from lowbit_comm_b200 import CompressionConfig
from lowbit_comm_b200.ops import codec, oracle
from lowbit_comm_b200.parallel.collectives.dynamic_all_gather import (CudaDynamicGatherExecutor,
                                                                      compressed_all_gather_dynamic)
from lowbit_comm_b200.parallel.metadata_packet import PACKET_WORDS, MetadataPacket


class FakeDist:
    """Rank 0 of 3.  Ranks 1 and 2 hold tensors of other shapes (one of them empty)."""

    class ReduceOp:
        MAX = "MAX"

    def __init__(self, cfg, others):
        self.cfg, self.others, self.calls = cfg, others, []

    def get_world_size(self, **kw):
        return 1 + len(self.others)

    def all_reduce(self, t, op=None, **kw):
        self.calls.append("all_reduce")
        t[0] = max([int(t[0])] + [o.numel() for o in self.others])

    def _packets(self, capacity_bytes):
        out = []
        for o in self.others:
            n = o.numel()
            nbytes = 0 if n == 0 else oracle.encode(o, self.cfg).numel()
            out.append(MetadataPacket(tuple(o.shape), "bf16", nbytes, 1 if n == 0 else 0))
        return out

    def all_gather_object(self, objs, mine, **kw):
        self.calls.append("all_gather_object")
        objs[0] = mine
        for i, p in enumerate(self._packets(None)):
            objs[i + 1] = {"shape": p.shape, "dtype": p.dtype, "payload_numel": p.payload_numel, "flags": p.flags}

    def all_gather_into_tensor(self, gathered, words, **kw):
        self.calls.append("all_gather_into_tensor")
        gathered[:PACKET_WORDS] = words
        for i, p in enumerate(self._packets(None)):
            gathered[(i + 1) * PACKET_WORDS:(i + 2) * PACKET_WORDS] = torch.tensor(p.encode(), dtype=torch.int64)

    def all_gather(self, slots, send, **kw):
        self.calls.append("all_gather")
        slots[0].copy_(send)
        for slot, o in zip(slots[1:], self.others):
            slot.zero_()
            if o.numel():
                payload = oracle.encode(o, self.cfg)
                slot[:payload.numel()] = payload


def _importer(fake):
    def load(name):
        return fake if name == "torch.distributed" else importlib.import_module(name)

    return load


@pytest.mark.parametrize("protocol", ("object_v1", "tensor_v1", "auto"))
def test_ragged_and_empty_contributions(protocol):
    cfg = CompressionConfig()
    g = torch.Generator().manual_seed(5)
    mine = (torch.randn(7, 33, generator=g) * 0.1).to(torch.bfloat16)
    others = [(torch.randn(500, generator=g) * 0.1).to(torch.bfloat16), torch.empty(0, 4, dtype=torch.bfloat16)]
    fake = FakeDist(cfg, others)
    seen = []

    def recording_quantize(t, config, **kw):
        seen.append(("quantize", t.numel()))
        return codec.quantize_tensor(t, config, **kw)

    outs = compressed_all_gather_dynamic(mine, config=cfg, metadata_protocol=protocol, import_module_fn=_importer(fake),
                                         quantize=recording_quantize)
    assert [tuple(o.shape) for o in outs] == [(7, 33), (500,), (0, 4)]
    assert torch.equal(outs[0], oracle.decode(oracle.encode(mine, cfg), mine.numel(), cfg, "bf16").reshape(7, 33))
    assert torch.equal(outs[1], oracle.decode(oracle.encode(others[0], cfg), 500, cfg, "bf16"))
    assert outs[2].numel() == 0
    assert seen == [("quantize", 231)]
    # capacity agreement first, then metadata, then one payload all-gather: three collectives, in this order
    meta_call = "all_gather_object" if protocol == "object_v1" else "all_gather_into_tensor"
    assert fake.calls == ["all_reduce", meta_call, "all_gather"]


def test_compiled_executor_rejects_what_does_not_fit():
    cfg = CompressionConfig()
    fake = FakeDist(cfg, [torch.zeros(10, dtype=torch.bfloat16)])
    ex = CudaDynamicGatherExecutor(shape_class=(64,), config=cfg, dtype="bf16", import_module_fn=_importer(fake))
    with pytest.raises(ValueError):
        ex.run(torch.zeros(65, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        ex.run(torch.zeros(8, dtype=torch.float16))
    snap = ex.execution_counters.snapshot()
    assert snap.run_calls == 2 and snap.failed_runs == 2 and fake.calls == []
    outs = ex.run(torch.ones(64, dtype=torch.bfloat16))
    assert len(outs) == 2 and ex.execution_counters.snapshot().completed_runs == 1


def test_executor_keeps_its_send_and_receive_slots_between_runs():
    cfg = CompressionConfig()
    fake = FakeDist(cfg, [torch.full((40,), 0.25, dtype=torch.bfloat16)])
    seen = []
    plain = fake.all_gather

    def watching(slots, send, **kw):
        seen.append((send.data_ptr(), tuple(s.data_ptr() for s in slots)))
        plain(slots, send, **kw)

    fake.all_gather = watching
    ex = CudaDynamicGatherExecutor(shape_class=(128,), config=cfg, dtype="bf16", metadata_protocol="tensor_v1",
                                   import_module_fn=_importer(fake))
    first = ex.run(torch.full((128,), 0.5, dtype=torch.bfloat16))
    second = ex.run(torch.full((3, 5), -0.5, dtype=torch.bfloat16))     # a smaller tensor of the same shape class
    assert ex.slot_allocations == 1 and seen[0] == seen[1] and ex.host_sync_count == 2
    assert seen[0][1][1] - seen[0][1][0] == ex.capacity_bytes           # slots are rows of one receive buffer
    assert tuple(first[0].shape) == (128,) and tuple(second[0].shape) == (3, 5)
    assert torch.equal(second[0], torch.full((3, 5), -0.5, dtype=torch.bfloat16))
    assert torch.equal(first[1], second[1]) and first[1].data_ptr() != second[1].data_ptr()   # results own their memory
