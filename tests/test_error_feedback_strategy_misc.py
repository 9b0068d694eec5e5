"""Error-feedback state/policies, DDP strategy planner, B200 strategy table, bucket fusion, plugin, capability."""

import pytest
import torch

from lowbit_comm_b200 import (CCDLCommunicationPlugin, CapabilityReport, CommunicationPlan, CompileContext,
                              CompressionConfig, UnsupportedCollective, detect)
from lowbit_comm_b200.ops.error_feedback import ErrorFeedbackPolicy, ErrorFeedbackState
from lowbit_comm_b200.parallel.bucket_fusion import BucketDescriptor, plan_bucket_fusion
from lowbit_comm_b200.parallel.strategy import CollectiveCapabilities, TopologyInfo, plan_ddp_compression_strategy
from lowbit_comm_b200.parallel.strategy_table import CudaStrategyRule, CudaStrategyTable


def test_error_feedback_state():
    st = ErrorFeedbackState()
    g = torch.ones(4)
    assert st.compensate(0, g) is g and st.get(0) is None
    st.update(0, original=g * 3, transmitted=g)
    assert torch.equal(st.compensate(0, g), g * 3)
    assert st.compensate(0, torch.ones(5)).numel() == 5 and st.get(0) is None  # shape change drops the residual
    buf = st.residual_for("k", g)
    assert buf.abs().sum() == 0 and st.residual_for("k", g) is buf and st.residual_for("k", torch.ones(6)) is not buf
    saved = st.state_dict()
    other = ErrorFeedbackState()
    other.load_state_dict(saved)
    assert set(other.keys()) == {"k"}
    st.clear()
    assert st.get("k") is None


def test_error_feedback_policies():
    def run(cfg, numel=100, steps=5):
        pol = ErrorFeedbackPolicy(cfg)
        out = []
        for _ in range(steps):
            d = pol.decide("b", numel=numel)
            out.append((d.apply, d.update))
            pol.advance("b")
        return out, pol

    assert run(CompressionConfig(error_feedback=False))[0] == [(False, False)] * 5
    assert run(CompressionConfig())[0] == [(True, True)] * 5
    big = CompressionConfig(error_feedback_policy="large_bucket_only", error_feedback_min_numel=101)
    assert run(big)[0][0] == (False, False) and run(big, numel=101)[0][0] == (True, True)
    warm = CompressionConfig(error_feedback_policy="warmup_then_enable", error_feedback_warmup_steps=2)
    assert run(warm)[0] == [(False, False)] * 2 + [(True, True)] * 3
    per = CompressionConfig(error_feedback_policy="periodic", error_feedback_period=3)
    seq, pol = run(per, steps=6)
    assert seq == [(True, True), (True, False), (True, False)] * 2
    fresh = ErrorFeedbackPolicy(per)
    fresh.load_state_dict(pol.state_dict())
    assert fresh.decide("b", numel=1).update and "every 3" in fresh.decide("b", numel=1).reason


def test_ddp_strategy_planner():
    caps = CollectiveCapabilities(reduce_scatter=True, hierarchical=True, topology=True)
    plan = plan_ddp_compression_strategy
    assert plan(requested_strategy="auto", world_size=2, capabilities=caps).strategy == "all_gather"
    assert plan(requested_strategy="auto", world_size=8, capabilities=caps).strategy == "reduce_scatter"
    multi = plan(requested_strategy="auto", world_size=16, node_count=2, capabilities=caps)
    assert multi.strategy == "all_gather" and multi.requires_fallback and "process groups" in multi.reason
    topo = TopologyInfo(rank=0, world_size=16, node_count=2, has_process_groups=True)
    assert plan(requested_strategy="auto", world_size=16, topology=topo, capabilities=caps).strategy == "hierarchical"
    none = plan(requested_strategy="auto", world_size=8, capabilities=CollectiveCapabilities())
    assert none.strategy == "all_gather" and none.requires_fallback
    assert plan(requested_strategy=" Topology ", world_size=4, capabilities=caps).strategy == "topology"
    assert plan(requested_strategy="all_reduce", world_size=4).capability_flags["reduce_scatter"] is False
    for wanted in ("hierarchical", "reduce_scatter", "topology"):
        with pytest.raises(UnsupportedCollective):
            plan(requested_strategy=wanted, world_size=4)
    with pytest.raises(UnsupportedCollective):
        plan(requested_strategy="butterfly", world_size=4)


def test_b200_strategy_table():
    table = CudaStrategyTable.for_b200()
    cfg = CompressionConfig()

    def ctx(world, numel, arch="sm_100", dtype="bf16"):
        return CompileContext(rank=0, world_size=world, device="cuda:0", shape=(numel,), dtype=dtype,
                              device_architecture=arch)

    full = CommunicationPlan(collective="all_reduce", strategy="auto", compression=cfg)
    assert table.select(full, ctx(2, 1 << 24)).strategy == "all_gather"
    big = table.select(full, ctx(8, 1 << 25))
    assert big.strategy == "reduce_scatter" and big.benchmark_matched and big.evidence and big.fallback == ("native_nccl",)
    assert table.select(full, ctx(2, 1 << 20)).strategy == "all_gather"
    between = table.select(full, ctx(8, 1 << 24))                    # 32 MiB on 8 GPUs: NCCL was measured faster
    assert between.strategy == "native_nccl" and "crossover" in between.reason and not between.benchmark_matched
    assert table.select(full, ctx(4, 1 << 26)).strategy == "reduce_scatter"
    small = table.select(full, ctx(8, 1000))
    assert small.strategy == "native_nccl" and "small bucket" in small.reason and not small.benchmark_matched
    other = table.select(full, ctx(8, 1 << 24, arch="sm_90"))
    assert other.strategy == "native_nccl" and "device_architecture" in other.reason
    shard = CommunicationPlan(collective="reduce_scatter", strategy="auto", compression=cfg, output_layout="shard")
    picked = table.select(shard, ctx(4, 1 << 24))
    assert picked.strategy == "compressed" and picked.observed_speedup and picked.baseline
    assert table.select(shard, ctx(3, 1 << 24)).strategy == "compressed"
    assert table.select(CommunicationPlan(collective="all_reduce", strategy="auto"), ctx(8, 10)).strategy == "native_nccl"
    with pytest.raises(UnsupportedCollective):
        table.select(CommunicationPlan(collective="all_gather", strategy="auto", compression=cfg), ctx(8, 10))
    rule = table.rules[0]
    with pytest.raises(ValueError):
        CudaStrategyTable((rule, rule))
    with pytest.raises(ValueError):
        CudaStrategyRule(**{**rule.__dict__, "min_numel": 10, "max_numel": 5})
    assert table.as_selector()(full, ctx(2, 1 << 24)).strategy == "all_gather"


def test_bucket_fusion():
    b = [BucketDescriptor(i, n, "bf16") for i, n in enumerate([1_000_000, 2_000_000, 1_500_000, 10, 20])]
    plan = plan_bucket_fusion(b)
    assert [g.bucket_indices for g in plan.groups] == [(0, 1), (2, 3, 4)]
    assert plan.fused_bucket_count == 5 and plan.total_fused_numel == 4_500_030 and plan.group_count == 2
    mixed = plan_bucket_fusion([BucketDescriptor(0, 5, "bf16"), BucketDescriptor(1, 5, "fp32"),
                                BucketDescriptor(2, 5, "fp32", requires_full_bucket=True), BucketDescriptor(3, 5, "fp32")])
    assert [g.fused for g in mixed.groups] == [False, False, False, False]
    assert mixed.groups[2].reason == "requires full-bucket consumer"
    assert plan_bucket_fusion(b, enabled=False).fused_group_count == 0
    assert [len(g.bucket_indices) for g in plan_bucket_fusion(b, max_bucket_count=2).groups] == [2, 2, 1]
    assert plan.to_metadata()["groups"][0]["fused"] is True
    with pytest.raises(ValueError):
        plan_bucket_fusion([BucketDescriptor(0, 0)])
    with pytest.raises(ValueError):
        plan_bucket_fusion(b, max_fused_numel=0)


def test_plugin_and_capability():
    plugin = CCDLCommunicationPlugin()
    cfg = CompressionConfig()
    assert plugin.name == "ccdl" and len(plugin.explain(cfg)) == 3 and "8-bit linear" in plugin.explain(cfg)[1]
    ok = plugin.plan({"training_backend": "native_ddp", "device_type": "cuda"}, cfg)
    assert ok.enabled and ok.fallback is None
    for ctx in ({"training_backend": "fsdp", "device_type": "cuda"}, {"training_backend": "native_ddp", "device_type": "npu"}):
        no = plugin.plan(ctx, cfg)
        assert not no.enabled and no.fallback == "bf16_compress"
    report = detect(import_torch=lambda: (_ for _ in ()).throw(ImportError("no torch")))
    assert not report.available and "torch" in report.reason
    d = CapabilityReport(available=True, cuda=True, torch_version="2.11", cuda_arch="sm_100", quantize=True,
                         compressed_collectives=True, ddp_hook=True).to_dict()
    assert set(d) == {"available", "cuda", "torch_version", "cuda_arch", "ops", "reason", "warnings"}
    assert d["ops"] == {"quantize": True, "compressed_collectives": True, "ddp_hook": True}
    caps = CapabilityReport.unavailable("no gpu").to_backend_capabilities()
    assert not caps.available and caps.reason == "no gpu"
    live = CapabilityReport(available=True, cuda=True, quantize=True, compressed_collectives=True).to_backend_capabilities()
    assert live.available and "reduce_scatter" in live.collectives and 8 in live.bits


def test_p2p_transport_selection_rules():
    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.exceptions import UnsupportedCollective
    from lowbit_comm_b200.parallel.p2p import _mailbox_for

    cfg = CompressionConfig()
    t = torch.zeros(128, dtype=torch.bfloat16)
    assert _mailbox_for(t, 1, cfg, None, 0, "auto", "torch") is None
    assert _mailbox_for(t, 1, cfg, None, 0, "auto", "auto") is None      # CPU tensor: torch.distributed send
    with pytest.raises(UnsupportedCollective):
        _mailbox_for(t, 1, cfg, None, 0, "auto", "peer")                 # insisting on the mailbox fails loudly
    with pytest.raises(ValueError):
        _mailbox_for(t, 1, cfg, None, 0, "auto", "carrier-pigeon")


def test_default_stage_rule():
    from lowbit_comm_b200.parallel.fused import default_stages

    assert default_stages(2, 1 << 30) == 1
    assert default_stages(8, 4 << 20) == 1 and default_stages(8, 8 << 20) == 1 and default_stages(8, 16 << 20) == 2
    assert default_stages(4, 16 << 20) == 1 and default_stages(4, 32 << 20) == 2
    assert default_stages(8, 16 << 20, multicast=True) == 1
