"""Control-plane value types: policy object, wire-size contract, reduced shard, chunk plans."""

import dataclasses

import pytest

from lowbit_comm_b200 import CompressionConfig, ReducedShard
from lowbit_comm_b200.core.chunking import ChunkPlan, GroupShardPlan
from lowbit_comm_b200.ops.sizing import WireLayout, estimate_quantized_size


def test_config_defaults_and_immutability():
    cfg = CompressionConfig()
    assert (cfg.bit, cfg.group_size, cfg.topk, cfg.quant_type, cfg.stochastic) == (8, 64, 0, "linear", False)
    assert cfg.error_feedback and cfg.target == "tensor" and cfg.fallback == "bf16_compress"
    assert cfg.error_feedback_policy == "always" and cfg.error_feedback_period == 1 and not cfg.compact
    assert len(dataclasses.fields(cfg)) == 15
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.bit = 4
    assert hash(cfg) == hash(CompressionConfig())
    assert CompressionConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("kwargs", [dict(bit=2), dict(bit=4), dict(group_size=48), dict(topk=3), dict(quant_type="log"),
                                    dict(target="kv_cache"), dict(error_feedback_policy="sometimes"),
                                    dict(error_feedback_min_numel=-1), dict(error_feedback_warmup_steps=-1),
                                    dict(error_feedback_period=0)])
def test_config_validation(kwargs):
    with pytest.raises(ValueError):
        CompressionConfig(**kwargs)


def test_config_experimental_and_effective_policy():
    assert CompressionConfig(bit=4, allow_experimental=True).bit == 4
    assert CompressionConfig(error_feedback=False, error_feedback_policy="periodic").effective_error_feedback_policy() == "none"
    assert CompressionConfig(error_feedback_policy="periodic").effective_error_feedback_policy() == "periodic"
    assert CompressionConfig().is_production_profile and not CompressionConfig(topk=1).is_production_profile


@pytest.mark.parametrize("dtype,bit,group,topk,per_group", [
    ("bf16", 8, 64, 0, 66), ("fp16", 8, 64, 1, 70), ("bf16", 8, 64, 2, 72), ("fp32", 8, 64, 0, 68),
    ("fp32", 8, 64, 1, 76), ("fp32", 8, 64, 2, 80), ("bf16", 4, 64, 0, 34), ("fp16", 8, 16, 0, 18), ("fp32", 4, 32, 2, 32)])
def test_wire_size_contract(dtype, bit, group, topk, per_group):
    cfg = CompressionConfig(bit=bit, group_size=group, topk=topk, allow_experimental=True)
    est = estimate_quantized_size(10 * group + 1, dtype=dtype, config=cfg)
    assert est.num_groups == 11 and est.padded_numel == 11 * group and est.padding_numel == group - 1
    assert est.quantized_bytes == 11 * per_group
    assert est.original_bytes == (10 * group + 1) * (4 if dtype == "fp32" else 2)


def test_size_estimate_edges():
    cfg = CompressionConfig()
    zero = estimate_quantized_size(0, dtype="bf16", config=cfg)
    assert zero.num_groups == 0 and zero.quantized_bytes == 0 and zero.compression_ratio == 0.0
    assert abs(estimate_quantized_size(64 * 1000, dtype="bf16", config=cfg).compression_ratio - 128 / 66) < 1e-12
    with pytest.raises(ValueError):
        estimate_quantized_size(-1, dtype="bf16", config=cfg)
    with pytest.raises(ValueError):
        estimate_quantized_size(1, dtype="int8", config=cfg)


def test_wire_layout_offsets():
    planar = WireLayout.of(640, "bf16", CompressionConfig())
    assert planar.total_bytes == 660 and planar.value_offset(3) == 192 and planar.meta_offset(3) == 640 + 6
    compact = WireLayout.of(640, "bf16", CompressionConfig(compact=True))
    assert compact.value_offset(3) == 198 and compact.meta_offset(3) == 198 + 64


def test_reduced_shard_invariants_and_derived_values():
    s = ReducedShard(shard=None, shard_index=3, shard_numel=25, original_shape=(9, 11), original_numel=99, world_size=4,
                     reduce="mean")
    assert s.padded_numel == 100 and s.shard_offset == 75 and s.shard_end == 99 and s.valid_numel == 24
    assert s.padding_numel == 1 and s.logical_range == (75, 99) and s.has_padding and not s.is_padding_only
    meta = s.to_metadata()
    assert meta["shard_index"] == 3 and meta["original_shape"] == (9, 11) and meta["metadata"] == {}
    with pytest.raises(TypeError):
        s.metadata["x"] = 1
    empty = ReducedShard(shard=None, shard_index=1, shard_numel=8, original_shape=(5,), original_numel=5, world_size=2,
                         reduce="sum")
    assert empty.is_padding_only and empty.valid_numel == 0


@pytest.mark.parametrize("kwargs", [dict(shard_index=-1), dict(shard_index=4), dict(world_size=0), dict(shard_numel=-1),
                                    dict(original_numel=-1), dict(padded_numel=96), dict(padded_numel=104),
                                    dict(original_shape=(3, -1)), dict(original_shape=(True, 2))])
def test_reduced_shard_rejects_bad_input(kwargs):
    base = dict(shard=None, shard_index=0, shard_numel=25, original_shape=(99,), original_numel=99, world_size=4,
                reduce="mean")
    base.update(kwargs)
    with pytest.raises(ValueError):
        ReducedShard(**base)


def test_chunk_plans():
    p = ChunkPlan.build(10, 4)
    assert (p.shard_numel, p.padded_numel, p.padding_numel) == (3, 12, 2)
    assert p.bounds(3) == (9, 12) and p.valid_bounds(3) == (9, 10) and p.owner(2) == 2
    with pytest.raises(ValueError):
        p.bounds(4)
    assert ChunkPlan.build(0, 3).shard_numel == 0
    g = GroupShardPlan.build(64 * 21 + 5, 4, 64, 8)
    assert g.num_groups == 22 and g.shard_groups == 8 and g.total_groups == 32 and g.shard_numel == 512
    assert [g.shard_valid_numel(r) for r in range(4)] == [512, 512, 64 * 21 + 5 - 1024, 0]
    assert [g.shard_valid_groups(r) for r in range(4)] == [8, 8, 6, 0]
    assert g.padded_numel >= g.numel and g.padded_numel == g.shard_numel * 4
