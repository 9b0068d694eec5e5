"""Ring, tree and direct-exchange schedules, executed on integers: every chunk must end up fully reduced on
its owner after the reduce-scatter and on every rank after the gather / broadcast."""

import pytest

from lowbit_comm_b200.core.chunking import ChunkPlan, compile_chunk_plan
from lowbit_comm_b200.core.schedules import (compile_direct_exchange_schedule, compile_pipelined_ring_schedule,
                                             compile_tree_schedule, tree_edges)


@pytest.mark.parametrize("world", (1, 2, 3, 4, 8))
def test_ring_schedule_reduces_and_restores(world):
    plan = compile_chunk_plan(original_numel=10 * world + 3, world_size=world)
    sched = [compile_pipelined_ring_schedule(chunk_plan=plan, rank=r) for r in range(world)]
    # data[r][c] = set of ranks whose contribution to chunk c is currently held by rank r
    held = [[{r} for _ in range(world)] for r in range(world)]
    for s in range(world - 1):
        sends = []
        for r in range(world):
            st = sched[r].steps[s]
            assert st.step_index == s and st.send_peer == (r + 1) % world and st.recv_peer == (r - 1) % world
            assert sched[st.send_peer].steps[s].recv_chunk_owner == st.send_chunk_owner      # both ends agree
            assert st.send_chunk == plan.chunk_for_rank(st.send_chunk_owner)
            sends.append((st.send_peer, st.send_chunk_owner, set(held[r][st.send_chunk_owner])))
        for r in range(world):
            st = sched[r].steps[s]
            src = [x for x in sends if x[0] == r]
            assert len(src) == 1 and src[0][1] == st.recv_chunk_owner
            assert src[0][2] == set(st.received_contributors) and len(st.received_contributors) == s + 1
            held[r][st.recv_chunk_owner] |= src[0][2]
    for r in range(world):
        assert held[r][r] == set(range(world)), (world, r)            # rank r owns the full sum of chunk r
        assert sched[r].local_chunk == plan.chunk_for_rank(r)
    done = [{r} for r in range(world)]                                # chunks whose final value each rank holds
    for s in range(world - 1):
        moved = []
        for r in range(world):
            g = sched[r].gather_steps[s]
            assert g.send_chunk_owner in done[r]
            moved.append((g.send_peer, g.send_chunk_owner))
        for peer, chunk in moved:
            done[peer].add(chunk)
    assert all(d == set(range(world)) for d in done)


@pytest.mark.parametrize("world,root", [(1, 0), (2, 1), (5, 0), (8, 3), (7, 6)])
def test_tree_schedule_reduces_to_the_root_and_broadcasts_back(world, root):
    plan = ChunkPlan.build(64, world)
    edges = tree_edges(world, root)
    assert len(edges) == world - 1 and len({e.child_rank for e in edges}) == world - 1
    have = [{r} for r in range(world)]
    for e in edges:                                   # replay order: a child is complete before it is sent
        sched = compile_tree_schedule(chunk_plan=plan, rank=e.child_rank, root=root)
        assert sched.parent == e.parent_rank
        for child in sched.children:
            assert have[child] <= have[e.child_rank]
        have[e.parent_rank] |= have[e.child_rank]
    assert have[root] == set(range(world))
    informed = {root}
    rs = compile_tree_schedule(chunk_plan=plan, rank=root, root=root)
    assert rs.parent is None and rs.broadcast_edges == tuple(reversed(rs.reduce_edges))
    for e in rs.broadcast_edges:
        assert e.parent_rank in informed
        informed.add(e.child_rank)
    assert informed == set(range(world))
    depth = max([0] + [len(bin(p + 1)) - 3 for p in range(world)])
    assert depth <= max(0, (world - 1).bit_length())


def test_direct_exchange_orders_are_rotations_and_never_collide():
    world = 8
    plan = ChunkPlan.build(1 << 20, world)
    scheds = [compile_direct_exchange_schedule(chunk_plan=plan, rank=r) for r in range(world)]
    for k in range(world):                            # at position k of the sweep all ranks target different peers
        assert len({s.scatter_order[k] for s in scheds}) == world
        assert len({s.gather_order[k] for s in scheds}) == world
    assert scheds[3].scatter_order[0] == 3 and scheds[3].local_chunk == plan.chunk_for_rank(3)
    assert scheds[0].link_crossings == 2


def test_argument_checks():
    plan = ChunkPlan.build(10, 2)
    with pytest.raises(ValueError):
        compile_pipelined_ring_schedule(chunk_plan=plan, rank=2)
    with pytest.raises(TypeError):
        compile_pipelined_ring_schedule(chunk_plan="plan", rank=0)
    with pytest.raises(TypeError):
        compile_tree_schedule(chunk_plan=plan, rank=True)
    with pytest.raises(ValueError):
        compile_tree_schedule(chunk_plan=plan, rank=0, root=5)


@pytest.mark.parametrize("world,groups_total,group,grid,depth", [
    (8, 8 * 1024, 64, 592, 4), (8, 8 * 1000 + 8, 64, 7, 2), (4, 4 * 40, 16, 3, 4), (2, 2 * 8, 32, 1, 2),
    (8, 8 * 8, 64, 1000, 4), (3, 3 * 24, 64, 5, 1),
])
def test_gather_tiles_cover_every_chunk_once_and_stay_inside_the_shard(world, groups_total, group, grid, depth):
    """Mirror of the decode kernel's addressing: element ranges are covered exactly once and every byte
    offset a thread computes lies inside the owner's shard payload (codes, then scales)."""

    from lowbit_comm_b200.core.schedules import gather_tiles

    lanes, value_bytes, scale_bytes, chunk_bytes = group // 16, group, 2, 16      # int8 codes, 16-bit scales
    shard_groups = groups_total // world
    shard_chunks = shard_groups * lanes
    payload_bytes = shard_groups * (value_bytes + scale_bytes)
    for first_owner in {0, world - 1}:
        seen = []
        for block in range(grid):
            for batch in gather_tiles(block=block, grid=grid, shard_chunks=shard_chunks, world_size=world,
                                      first_owner=first_owner, tiles_in_flight=depth):
                assert len(batch) <= depth
                for tile in batch:
                    assert 0 <= tile.owner < world and tile.count > 0
                    for within in range(tile.start, tile.start + tile.count):
                        group_in_shard, lane = divmod(within, lanes)
                        code_offset = group_in_shard * value_bytes + lane * chunk_bytes
                        scale_offset = shard_groups * value_bytes + group_in_shard * scale_bytes
                        assert code_offset + chunk_bytes <= shard_groups * value_bytes
                        assert shard_groups * value_bytes <= scale_offset and scale_offset + scale_bytes <= payload_bytes
                        seen.append(tile.owner * shard_chunks + within)
        assert sorted(seen) == list(range(world * shard_chunks))


def test_gather_tiles_start_at_the_rank_and_spread_over_owners():
    from lowbit_comm_b200.core.schedules import gather_tiles

    first = [gather_tiles(block=0, grid=16, shard_chunks=4096, world_size=8, first_owner=r, tiles_in_flight=4)[0]
             for r in range(8)]
    assert [batch[0].owner for batch in first] == list(range(8))          # every rank begins with its own shard
    in_flight = gather_tiles(block=3, grid=17, shard_chunks=4096, world_size=8, first_owner=2, tiles_in_flight=4)[0]
    assert len({t.owner for t in in_flight}) == 4                          # grid not a multiple of W: 4 owners at once
    with pytest.raises(ValueError):
        gather_tiles(block=0, grid=0, shard_chunks=1, world_size=1, first_owner=0)
    with pytest.raises(ValueError):
        gather_tiles(block=4, grid=4, shard_chunks=1, world_size=1, first_owner=0)


@pytest.mark.parametrize("world", (1, 2, 3, 5, 8))
def test_pairwise_schedule_delivers_every_contribution_to_its_owner(world):
    from lowbit_comm_b200.core.chunking import ChunkPlan
    from lowbit_comm_b200.core.schedules import compile_pairwise_schedule

    plan = ChunkPlan.build(world * 4, world)
    scheds = [compile_pairwise_schedule(chunk_plan=plan, rank=r) for r in range(world)]
    received = {r: {r} for r in range(world)}                  # contributors summed into chunk r at its owner
    for k in range(world - 1):
        sends = {(r, s.steps[k].send_peer) for r, s in enumerate(scheds)}
        recvs = {(s.steps[k].recv_peer, r) for r, s in enumerate(scheds)}
        assert sends == recvs and len({dst for _, dst in sends}) == world       # every round is a permutation
        for r, s in enumerate(scheds):
            step = s.steps[k]
            assert step.send_chunk == plan.chunk_for_rank(step.send_peer) and step.recv_chunk == s.local_chunk
            received[r].add(step.recv_peer)
    assert all(received[r] == set(range(world)) for r in range(world))


def test_butterfly_schedule_pairs_are_mutual_and_need_a_power_of_two():
    from lowbit_comm_b200.core.schedules import compile_butterfly_schedule

    scheds = [compile_butterfly_schedule(world_size=8, rank=r) for r in range(8)]
    reach = [{r} for r in range(8)]
    for k in range(3):
        assert all(scheds[scheds[r].peers[k]].peers[k] == r for r in range(8))
        reach = [reach[r] | reach[scheds[r].peers[k]] for r in range(8)]
    assert all(known == set(range(8)) for known in reach)
    assert compile_butterfly_schedule(world_size=1, rank=0).peers == ()
    with pytest.raises(ValueError, match="power-of-two"):
        compile_butterfly_schedule(world_size=6, rank=0)
