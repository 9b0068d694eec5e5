"""Workspace pool and leases (fake events), payload packing, metadata packet, result schema and gates,
architecture contract."""

import ast
import pathlib

import pytest
import torch

from lowbit_comm_b200.parallel.metadata_packet import PACKET_WORDS, MetadataPacket, decode_all
from lowbit_comm_b200.parallel.payload import CompressedPayload, GatheredPayloads
from lowbit_comm_b200.parallel.payload_packing import (FusedPayloadPacker, make_fused_payload_all_gather,
                                                        make_payload_all_gather, should_fuse_payload)
from lowbit_comm_b200.parallel.workspace import (CudaOutputLease, CudaWorkspacePool, DequantizedWorkspaceCache,
                                                  ShardCommunicationWorkspaceCache, WorkspaceKey)
from lowbit_comm_b200.utils import perf_gate, result_schema, roofline


class FakeEvent:
    def __init__(self, ready=False):
        self.ready, self.log = ready, []

    def query(self):
        return self.ready

    def wait_stream(self, stream):
        self.log.append(("wait_stream", stream))


class FakeManager:
    def __init__(self):
        self.events = []

    def record_for(self, value, stream=None):
        ev = FakeEvent(ready=True)
        self.events.append((value, stream))
        return ev


def key(kind="recv", n=64):
    return WorkspaceKey(backend="cuda", collective="reduce_scatter", strategy="compressed", shape_class=(n,),
                        dtype="bf16", world_size=4, bit=8, group_size=64, chunk_config=(n,), workspace_kind=kind)


def pool(**kw):
    made = []

    def alloc(k, stream):
        made.append(k)
        return torch.empty(k.shape_class, dtype=torch.bfloat16)

    return CudaWorkspacePool(allocator=alloc, **kw), made


def test_pool_reuses_only_finished_buffers():
    p, made = pool()
    a = p.acquire(key(), "s0")
    pending = FakeEvent(ready=False)
    a.release(completion=pending)
    assert p.stats.in_flight_bytes == 0 and p.stats.cached_bytes == 128
    b = p.acquire(key(), "s1")            # same key, previous use not finished: handed over after a stream wait
    assert b.buffer is a.buffer and pending.log == [("wait_stream", "s1")] and p.stats.hits == 1
    c = p.acquire(key(), "s1")
    assert c.buffer is not b.buffer and len(made) == 2 and p.stats.misses == 2
    b.release(completion=FakeEvent(ready=True))
    assert p.acquire(key(), "s2").buffer is b.buffer
    with pytest.raises(RuntimeError):
        b.release(completion=None)
    with pytest.raises(TypeError):
        p.acquire("key", None)
    with pytest.raises(TypeError):
        c.release(completion=object())
    assert not c.released  # a failed release leaves the lease usable
    c.release(completion=None)


def test_pool_budgets_and_stats():
    p, _ = pool(max_entries=1)
    leases = [p.acquire(key(n=64 * (i + 1)), None) for i in range(3)]
    for lease in leases:
        lease.release(completion=FakeEvent(ready=True))
    st = p.stats
    assert st.evictions == 2 and st.cached_bytes == leases[-1].size_bytes
    q, _ = pool(max_cached_bytes=0)
    q.acquire(key(), None).release(completion=None)
    assert q.stats.cached_bytes == 0 and q.stats.evictions == 1
    with pytest.raises(ValueError):
        CudaWorkspacePool(allocator=lambda k, s: None, max_entries=0)
    with pytest.raises(ValueError):
        WorkspaceKey(**{**key().__dict__, "world_size": 0})


def test_output_lease_state_machine():
    p, _ = pool()
    token, manager = object(), FakeManager()
    lease = CudaOutputLease(p.acquire(key("reduced_output"), "s"), owner_token=token, completion_manager=manager,
                            acquisition_stream="s")
    with pytest.raises(RuntimeError):
        lease.release_after("x")                    # not used yet
    with pytest.raises(RuntimeError):
        lease.mark_used(object())                   # someone else's executor
    buf = lease.mark_used(token)
    assert buf is lease.buffer and lease.state == "SUBMITTING"
    with pytest.raises(RuntimeError):
        lease.mark_used(token)
    lease.abort_use(token)
    lease.mark_used(token)

    class Work:
        done = False

        def query(self):
            return self.done

    work = Work()
    lease.bind_work(token, work)
    with pytest.raises(RuntimeError):
        lease.release_after(buf)                    # work still running
    work.done = True
    lease.release_after(buf)
    assert lease.state == "RELEASED" and p.stats.in_flight_bytes == 0
    with pytest.raises(RuntimeError):
        lease.release_unused()
    fresh = CudaOutputLease(p.acquire(key("reduced_output"), "s"), owner_token=token, completion_manager=manager,
                            acquisition_stream="s9")
    fresh.release_unused()
    assert manager.events[-1][1] == "s9"


def test_legacy_caches():
    cache = DequantizedWorkspaceCache(allocator=lambda like, shape, cfg: torch.empty(shape, dtype=like.dtype), max_entries=1)
    like = torch.zeros(4)
    a = cache.get("b0", like, (4,), None)
    assert cache.get("b0", like, (4,), None) is a and cache.hits == 1
    cache.get("b1", like, (4,), None)
    assert cache.get("b0", like, (4,), None) is not a
    shard = ShardCommunicationWorkspaceCache(max_entries=2)
    s0 = shard.get("b", "send", 0, lambda: [0])
    assert shard.get("b", "send", 0, lambda: [1]) is s0
    with pytest.raises(ValueError):
        shard.get("b", "scratch", 0, list)


def fake_gather(world=3):
    def gather(t):
        return GatheredPayloads(tuple(t + r for r in range(world)))
    return gather


def test_payload_all_gather_variants():
    payload = CompressedPayload(torch.arange(8, dtype=torch.int8), (8,), "fp32",
                                {"scales": torch.ones(2), "original_numel": 8})
    for make in (make_payload_all_gather, make_fused_payload_all_gather):
        out = make(fake_gather())(payload)
        assert len(out.payloads) == 3 and all(isinstance(p, CompressedPayload) for p in out.payloads)
        assert out.payloads[0].metadata["original_numel"] == 8
        assert torch.equal(out.payloads[0].buffer, payload.buffer)
        assert out.payloads[0].metadata["scales"].shape == (2,)
    packer = FusedPayloadPacker()
    packed = packer.pack(payload)
    assert packed.dtype == torch.uint8 and packed.numel() == 8 + 8
    back = packer.unpack(packed, payload)
    assert torch.equal(back.buffer, payload.buffer) and torch.equal(back.metadata["scales"], payload.metadata["scales"])
    assert should_fuse_payload(torch.zeros(10), enabled=True, min_numel=10)
    assert not should_fuse_payload(torch.zeros(10), enabled=False, min_numel=1)
    raw = make_payload_all_gather(fake_gather(2))(torch.zeros(3))
    assert len(raw.payloads) == 2


def test_metadata_packet_round_trip():
    pkt = MetadataPacket((3, 5, 7), "bf16", 1234)
    words = pkt.encode()
    assert len(words) == PACKET_WORDS and words[:5] == [1, 3, 2, 1234, 0] and words[8:11] == [3, 5, 7]
    assert MetadataPacket.decode(words) == pkt and pkt.numel == 105
    both = decode_all(words + MetadataPacket((), "fp32", 0, flags=1).encode(), 2)
    assert both[1].shape == () and both[1].flags == 1
    for bad in ([2] + words[1:], words[:5] + [9] + words[6:], words[:-1] + [4], words[:2] + [7] + words[3:]):
        with pytest.raises(ValueError):
            MetadataPacket.decode(bad)
    with pytest.raises(ValueError):
        MetadataPacket(tuple(range(9)), "bf16", 0)


def record(**kw):
    base = dict(commit="abc123", hostname="h", gpu_name="NVIDIA B200", cuda_version="12.9", torch_version="2.11",
                world_size=8, dtype="bf16", numel=1 << 25, strategy="reduce_scatter", latency_ms=0.12,
                effective_gbps=500.0, peak_memory_bytes=1, relative_l2=0.006, max_abs_error=0.01, rmse=0.001,
                non_finite=False)
    base.update(kw)
    return base


def test_result_schema_and_gates(monkeypatch):
    assert result_schema.BenchmarkResult(**record()).to_dict()["schema_version"] == result_schema.SCHEMA_VERSION
    for bad in (dict(commit="unknown"), dict(latency_ms=0.0), dict(relative_l2=-1), dict(world_size=0)):
        with pytest.raises(ValueError):
            result_schema.validate_result(record(**bad))
    with pytest.raises(ValueError):
        result_schema.validate_result({"commit": "x"})
    monkeypatch.setenv("CCDL_BENCHMARK_COMMIT", "deadbeef")
    monkeypatch.setenv("CCDL_BENCHMARK_HOSTNAME", "box7")
    assert result_schema.benchmark_identity() == {"commit": "deadbeef", "hostname": "box7"}
    assert abs(result_schema.effective_gbps(1 << 30, 2, 2.0) - 1073.741824) < 1e-6
    perf_gate.assert_performance_gate([record()], [record(latency_ms=0.121)])
    with pytest.raises(AssertionError):
        perf_gate.assert_performance_gate([record()], [record(latency_ms=0.13)])
    with pytest.raises(ValueError):
        perf_gate.compare_results([record()], [record(world_size=4)])
    runs = [dict(run_id=i, fused_launches_per_rank=1, steady_state_allocated_bytes=0, relative_l2=0.006) for i in range(5)]
    assert perf_gate.evaluate_fused_gate(runs, launches_per_rank=1)["passed"]
    assert not perf_gate.evaluate_fused_gate(runs[:3], launches_per_rank=1)["passed"]
    assert not perf_gate.evaluate_fused_gate(runs + [dict(run_id=9, fused_launches_per_rank=2)], launches_per_rank=1)["passed"]
    rows = [dict(mib=64, roofline_frac=0.7), dict(mib=64, roofline_frac=0.5), dict(mib=1, roofline_frac=0.1)]
    assert perf_gate.roofline_gate(rows) == [rows[1]]
    model = roofline.fused_all_reduce_roofline(64 << 20, 8, stages=2, hbm_gbs=6552.3)
    assert model["bound"] == "hbm" and 80 < model["roofline_us"] < 85 and 78 < model["t_link_us"] < 79
    assert roofline.fused_all_reduce_roofline(64 << 20, 8, stages=1, hbm_gbs=6552.3)["bound"] == "nvlink"


def test_control_plane_never_imports_torch_or_backends():
    """Architecture contract: `core/` and the top-level policy modules stay torch-free and backend-free."""

    root = pathlib.Path(__file__).resolve().parents[1] / "lowbit_comm_b200"
    pure = list((root / "core").glob("*.py")) + [root / n for n in ("config.py", "plugin.py", "exceptions.py", "abi.py")]
    pure += [root / "parallel" / n for n in ("strategy.py", "bucket_fusion.py", "metadata_packet.py")]
    assert len(pure) >= 15
    for path in pure:
        for node in ast.walk(ast.parse(path.read_text())):
            names = []
            if isinstance(node, ast.Import):
                names = [a.name for a in node.names]
            elif isinstance(node, ast.ImportFrom):
                names = [("." * node.level) + (node.module or "")]
            for name in names:
                assert not name.startswith("torch"), (path.name, name)
                assert "ops" not in name.split(".") and "csrc" not in name, (path.name, name)
                if path.parent.name == "core":
                    assert "parallel" not in name.split("."), (path.name, name)


def test_fused_payload_packer_schema_round_trip():
    import torch

    from lowbit_comm_b200.parallel.payload import CompressedPayload, GatheredPayloads
    from lowbit_comm_b200.parallel.payload_packing import (FusedPayloadAllGather, FusedPayloadPacker, TensorFieldSchema,
                                                          make_fused_payload_all_gather)

    payload = CompressedPayload(torch.arange(128, dtype=torch.int8), (2, 64), "bf16",
                                {"scales": torch.tensor([0.5, 2.0]), "original_numel": 128, "zeros": torch.zeros(3, dtype=torch.int16)})
    packer = FusedPayloadPacker.from_payload(payload)
    assert isinstance(packer.buffer_schema, TensorFieldSchema)
    assert packer.buffer_schema.byte_count == 128 and packer.buffer_schema.offset == 0
    assert [(f.name, f.offset, f.byte_count) for f in packer.metadata_schemas] == [("scales", 128, 8), ("zeros", 136, 6)]
    assert packer.scalar_metadata == {"original_numel": 128} and packer.packed_bytes == 142
    packed = packer.pack(payload)
    assert packed.dtype == torch.uint8 and packed.numel() == 142
    back = packer.unpack(packed, shape=(2, 64), dtype="bf16")
    assert torch.equal(back.buffer, payload.buffer) and torch.equal(back.metadata["scales"], payload.metadata["scales"])
    assert back.metadata["original_numel"] == 128 and back.shape == (2, 64) and back.dtype == "bf16"
    with pytest.raises(ValueError):
        packer.unpack(packed[:-1], shape=(2, 64), dtype="bf16")
    with pytest.raises(ValueError):
        packer.pack(payload.with_buffer(torch.zeros(64, dtype=torch.int8)))      # another buffer shape: schema mismatch
    assert payload.with_buffer(packed).metadata["original_numel"] == 128

    calls = []

    def byte_all_gather(t):
        calls.append(t.numel())
        return GatheredPayloads((t, t.clone()))

    fused = FusedPayloadAllGather(byte_all_gather, packer, (2, 64), "bf16")
    got = fused(payload)
    assert got.world_size == 2 and calls == [142] and torch.equal(got.payloads[1].metadata["scales"], payload.metadata["scales"])
    transport = make_fused_payload_all_gather(byte_all_gather)
    assert transport(payload).world_size == 2 and transport(payload).world_size == 2 and calls == [142, 142, 142]


def test_metadata_packet_function_interface():
    import torch

    from lowbit_comm_b200.parallel import metadata_packet as mp

    packet = mp.encode_metadata_packet(shape=(3, 0, 5), dtype="bf16", payload_numel=99, torch=torch, device="cpu", flags=1)
    assert packet.dtype == torch.int64 and packet.numel() == mp.METADATA_PACKET_NUMEL == 16
    assert packet.tolist() == [1, 3, 2, 99, 1, 0, 0, 0, 3, 0, 5, 0, 0, 0, 0, 0]       # bf16 is code 2 on the wire
    assert mp.decode_metadata_packet(packet) == {"protocol_version": 1, "shape": (3, 0, 5), "dtype": "bf16",
                                                 "payload_numel": 99, "flags": 1}
    reused = torch.zeros(16, dtype=torch.int64)
    assert mp.write_metadata_packet(reused, shape=(7,), dtype="fp32", payload_numel=0) is reused
    both = torch.cat([packet, reused])
    decoded = mp.decode_metadata_packets(both, world_size=2)
    assert [d["shape"] for d in decoded] == [(3, 0, 5), (7,)] and decoded[1]["dtype"] == "fp32"
    bad = packet.clone()
    bad[6] = 4                                            # a reserved word
    with pytest.raises(RuntimeError):
        mp.decode_metadata_packet(bad)
    with pytest.raises(RuntimeError):
        mp.decode_metadata_packets(both[:-1], world_size=2)
    with pytest.raises(ValueError):
        mp.write_metadata_packet(reused, shape=(1,) * 9, dtype="fp16", payload_numel=0)
    with pytest.raises(TypeError):
        mp.write_metadata_packet(reused, shape=(1.5,), dtype="fp16", payload_numel=0)
    with pytest.raises(ValueError):
        mp.write_metadata_packet(torch.zeros(8, dtype=torch.int64), shape=(1,), dtype="fp16", payload_numel=0)


def test_shard_workspace_cache_accessors_and_torch_pool():
    import types

    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.completion import native_work_available
    from lowbit_comm_b200.parallel.workspace import (ShardCommunicationWorkspaceCache, WorkspaceKey,
                                                     create_torch_workspace_pool)

    cfg = CompressionConfig()
    cache = ShardCommunicationWorkspaceCache()
    chunk = torch.zeros(640, dtype=torch.bfloat16)
    a = cache.get_quantized_chunk("bucket0", 1, chunk, cfg, dtype="bf16", world_size=4)
    assert a.dtype == torch.uint8 and a.numel() == 660
    assert cache.get_quantized_chunk("bucket0", 1, chunk, cfg, dtype="bf16", world_size=4) is a        # cached
    assert cache.get_quantized_chunk("bucket0", 2, chunk, cfg, dtype="bf16", world_size=4) is not a    # other chunk
    assert cache.get_quantized_chunk("bucket0", 1, chunk[:320], cfg, dtype="bf16", world_size=4) is not a  # new shape
    r = cache.get_received_payload("bucket0", a, 3, world_size=4, config=cfg)
    assert r.shape == a.shape and r is cache.get_received_payload("bucket0", a, 3, world_size=4, config=cfg)
    s = cache.get_reduced_shard("bucket0", chunk, (160,), cfg, dtype="bf16", world_size=4, rank=2)
    assert s.shape == (160,) and s.dtype == torch.bfloat16
    cache.clear("bucket0")
    assert cache.get_reduced_shard("bucket0", chunk, (160,), cfg, dtype="bf16", world_size=4, rank=2) is not s

    pool = create_torch_workspace_pool(max_entries=2)
    key = WorkspaceKey("cuda", "reduce_scatter", "compressed", (128,), "uint8", 4, 8, 64, (), "send", device="cpu")
    lease = pool.acquire(key, None)
    assert lease.buffer.dtype == torch.uint8 and lease.buffer.numel() == 128

    assert not native_work_available(types.SimpleNamespace(available=False, module=None))
    fake = types.SimpleNamespace(create_cuda_executor=lambda: None, NATIVE_WORK_ABI_VERSION=1)
    assert native_work_available(types.SimpleNamespace(available=True, module=fake))
    fake.NATIVE_WORK_ABI_VERSION = 2
    assert not native_work_available(types.SimpleNamespace(available=True, module=fake))


def test_shard_workspace_session_leases_and_release():
    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.workspace import CudaShardWorkspaceProvider, create_torch_workspace_pool

    class Completion:
        def __init__(self, ready):
            self.ready = ready

        def query(self):
            return self.ready

    cfg = CompressionConfig()
    pool = create_torch_workspace_pool()
    provider = CudaShardWorkspaceProvider(pool, backend="cuda", collective="reduce_scatter", strategy="compressed",
                                          device="cpu")
    with pytest.raises(TypeError):
        CudaShardWorkspaceProvider(object(), backend="cuda", collective="reduce_scatter", strategy="compressed", device="cpu")
    chunk = torch.zeros(640, dtype=torch.bfloat16)
    session = provider.begin(stream=None)
    send = session.get_quantized_chunk("b0", 0, chunk, cfg, dtype="bf16", world_size=4)
    recv = session.get_received_payload("b0", send, 2, world_size=4, config=cfg)
    recv2 = session.get_received_tensor_payload("b0", 3, chunk, cfg, dtype="bf16", world_size=4)
    reduced = session.get_reduced_shard("b0", chunk, (150,), cfg, dtype="bf16", world_size=4, rank=1)
    assert send.dtype == torch.uint8 and send.numel() == 660 and recv.shape == send.shape and recv2.numel() == 660
    assert reduced.dtype == torch.bfloat16 and reduced.numel() == 192            # padded to whole groups of 64
    assert len(session.leases) == 4 and pool.stats.in_flight_bytes > 0
    # a second session running at the same time gets other buffers
    other = provider.begin(stream=None)
    assert other.get_quantized_chunk("b0", 0, chunk, cfg, dtype="bf16", world_size=4).data_ptr() != send.data_ptr()
    other.release(completion=Completion(True))
    pending = Completion(False)
    session.release(completion=pending)
    assert session.leases == ()
    third = provider.begin(stream=None)
    again = third.get_quantized_chunk("b0", 0, chunk, cfg, dtype="bf16", world_size=4)
    assert again.data_ptr() != send.data_ptr()           # not reusable while its completion is pending
    pending.ready = True
    fourth = provider.begin(stream=None)
    reused = fourth.get_quantized_chunk("b0", 0, chunk, cfg, dtype="bf16", world_size=4)
    assert reused.data_ptr() == send.data_ptr()          # its completion is ready now: the buffer comes back
    no_out = CudaShardWorkspaceProvider(pool, backend="cuda", collective="reduce_scatter", strategy="compressed",
                                        device="cpu", pool_reduced_output=False)
    assert no_out.begin(stream=None).get_reduced_shard("b0", chunk, (150,), cfg, dtype="bf16", world_size=4, rank=0) is None
