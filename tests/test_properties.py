"""Property-based checks (hypothesis): invariants that must hold for any size, world size and profile."""

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from lowbit_comm_b200.config import CompressionConfig  # noqa: E402
from lowbit_comm_b200.core.chunking import ChunkPlan, GroupShardPlan, hierarchy_groups  # noqa: E402
from lowbit_comm_b200.core.schedules import compile_pipelined_ring_schedule, tree_edges  # noqa: E402
from lowbit_comm_b200.ops import host_codec, oracle  # noqa: E402
from lowbit_comm_b200.ops.build import build_host_library  # noqa: E402
from lowbit_comm_b200.ops.sizing import estimate_quantized_size  # noqa: E402

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
profiles = st.builds(
    lambda bit_group, topk, compact: CompressionConfig(bit=bit_group[0], group_size=bit_group[1], topk=topk,
                                                       compact=compact, allow_experimental=True),
    st.sampled_from([(8, 64), (8, 32), (8, 16), (4, 64), (4, 32), (4, 16)]), st.integers(0, 2), st.booleans())


@pytest.fixture(scope="module", autouse=True)
def _host_library():
    build_host_library()
    host_codec._tried = False
    assert host_codec.library() is not None


@settings(max_examples=60, deadline=None, derandomize=True)
@given(n=st.integers(0, 5000), world=st.integers(1, 16), group=st.sampled_from([16, 32, 64]))
def test_shard_plans_cover_the_tensor_exactly_once(n, world, group):
    plan = ChunkPlan.build(n, world)
    assert plan.padded_numel >= n and plan.padded_numel - n < max(world, 1) + (0 if n else 1)
    covered = 0
    for c in range(world):
        lo, hi = plan.valid_bounds(c)
        assert lo <= hi and plan.owner(c) == c
        covered += hi - lo
    assert covered == n
    gplan = GroupShardPlan.build(n, world, group)
    assert gplan.shard_numel % (8 * group) == 0 or n == 0
    assert gplan.shard_numel * world >= n
    if n:
        assert (gplan.shard_numel - 8 * group) * world < n + world * 8 * group   # no more than one alignment unit each


@settings(max_examples=40, deadline=None, derandomize=True)
@given(nodes=st.integers(1, 6), local=st.integers(1, 6), offset=st.integers(0, 50))
def test_hierarchy_groups_partition_the_ranks_twice(nodes, local, offset):
    ranks = [offset + i for i in range(nodes * local)]
    loc, inter = hierarchy_groups(ranks, local)
    assert sorted(r for g in loc for r in g) == ranks and sorted(r for g in inter for r in g) == ranks
    assert all(len(g) == local for g in loc) and all(len(g) == nodes for g in inter)
    for g in inter:                                   # members of an inter group share their local index
        assert len({ranks.index(r) % local for r in g}) == 1


@settings(max_examples=30, deadline=None, derandomize=True)
@given(world=st.integers(1, 12), root=st.integers(0, 11), n=st.integers(0, 1000))
def test_schedules_are_consistent_for_any_world(world, root, n):
    root %= world
    plan = ChunkPlan.build(n, world)
    scheds = [compile_pipelined_ring_schedule(chunk_plan=plan, rank=r) for r in range(world)]
    for s in range(world - 1):
        for r in range(world):
            step = scheds[r].steps[s]
            assert scheds[step.send_peer].steps[s].recv_chunk_owner == step.send_chunk_owner
    assert world == 1 or all(scheds[r].steps[-1].recv_chunk_owner == r for r in range(world))
    edges = tree_edges(world, root)
    assert {e.child_rank for e in edges} == set(range(world)) - {root}
    parents = {e.child_rank: e.parent_rank for e in edges}
    for r in range(world):                            # every rank reaches the root
        hops, at = 0, r
        while at != root:
            at, hops = parents[at], hops + 1
            assert hops <= world
        assert hops <= max(1, world.bit_length())


@settings(max_examples=60, deadline=None, derandomize=True)
@given(cfg=profiles, dtype=st.sampled_from(["bf16", "fp16", "fp32"]), n=st.integers(1, 700),
       seed=st.integers(0, 2 ** 16), scale=st.sampled_from([1e-6, 1e-3, 1.0, 1e3]))
def test_host_codec_equals_oracle_and_error_is_bounded(cfg, dtype, n, seed, scale):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n, generator=g) * scale).to(DT[dtype])
    want = oracle.encode(x, cfg)
    est = estimate_quantized_size(n, dtype=dtype, config=cfg)
    assert want.numel() == est.quantized_bytes and est.padded_numel % cfg.group_size == 0
    out = torch.empty_like(want)
    host_codec.quantize(x, cfg, dtype, out)
    assert torch.equal(out, want)
    dec = torch.empty(n, dtype=DT[dtype])
    host_codec.dequantize(want, n, cfg, dtype, dec)
    ref = oracle.decode(want, n, cfg, dtype)
    assert torch.equal(dec.view(torch.uint8), ref.view(torch.uint8))
    # reconstruction error: at most half a quantization step of the group's scale (plus the source dtype's rounding)
    levels = 127.0 if cfg.bit == 8 else 7.0
    groups = oracle._grouped(x, cfg.group_size).float()
    # A group whose largest magnitude is below 1e-6 is encoded against the clamped scale 1e-6 but decoded with its
    # stored (smaller) scale: such groups shrink towards zero, so their error is only bounded by the magnitude
    # itself.  fp16 results below 6e-5 are subnormal: absolute slack 1e-7.
    amax = groups.abs().amax(dim=1, keepdim=True)
    step_bound = amax / levels * 0.51 + amax * 2 ** -7
    bound = torch.where(amax < 1e-4, amax, step_bound) + 1e-7   # margin: top-k removal lowers the scale further
    err = (oracle._grouped(dec, cfg.group_size).float() - groups).abs()
    assert bool((err <= bound).all())
