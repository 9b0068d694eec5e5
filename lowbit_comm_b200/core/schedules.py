"""Rank-local communication schedules as plain data (torch-free).

The reference drives its ring, tree and hierarchical all-reduce from immutable schedules compiled once per
(world size, rank): `PipelinedRingSchedule`, `TreeSchedule`, hierarchical stages
(ccdl_comm/cuda/transports/pipelined_ring.py:14-120, 285-332; tree.py:15-75, 277-307).  On an NVSwitch
node this library executes none of them hop by hop: every strategy name lands on the direct one-hop
exchange of the fused kernels (`DirectExchangeSchedule` below states who writes to and reads from whom,
`gather_tiles` in which order a decode kernel reads).  The ring and tree schedules, with the reference's
field names, drive `parallel/schedule_executors.py` for groups without peer access (other nodes, CPU ranks);
`tests/test_schedules.py` executes them on integers and checks that they reduce and restore every chunk.
"""

from __future__ import annotations

from dataclasses import dataclass

from .chunking import ChunkPlan, ChunkRange


def _index(value: object, bound: int, name: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer")
    if not 0 <= value < bound:
        raise ValueError(f"{name} must be in [0, {bound})")
    return value


def _plan(chunk_plan: object) -> ChunkPlan:
    if not isinstance(chunk_plan, ChunkPlan):
        raise TypeError("chunk_plan must be a ChunkPlan")
    return chunk_plan


# ---- ring ----------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RingReduceScatterStep:
    """Step s of the reduce-scatter: send one partially reduced chunk to the next rank, receive another from
    the previous rank and add it.  `received_contributors` are the ranks already summed into what arrives."""

    step_index: int
    send_peer: int
    recv_peer: int
    send_chunk_owner: int
    recv_chunk_owner: int
    received_contributors: tuple[int, ...]
    send_chunk: ChunkRange
    recv_chunk: ChunkRange


@dataclass(frozen=True)
class RingAllGatherStep:
    """Step s of the all-gather that follows: pass a finished chunk on, receive the one before it."""

    step_index: int
    send_peer: int
    recv_peer: int
    send_chunk_owner: int
    recv_chunk_owner: int
    send_chunk: ChunkRange
    recv_chunk: ChunkRange


@dataclass(frozen=True)
class PipelinedRingSchedule:
    chunk_plan: ChunkPlan
    rank: int
    steps: tuple[RingReduceScatterStep, ...]
    gather_steps: tuple[RingAllGatherStep, ...]

    @property
    def local_chunk(self) -> ChunkRange:
        """The shard this rank owns once the reduce-scatter is done."""

        return self.chunk_plan.chunk_for_rank(self.rank)


def compile_pipelined_ring_schedule(*, chunk_plan: ChunkPlan, rank: int) -> PipelinedRingSchedule:
    """Ring over ranks 0..W-1, data flowing r -> r + 1.  In reduce-scatter step s rank r forwards the chunk
    that will end at rank r - s - 1 and receives the one bound for r - s - 2, so after W - 1 steps it holds
    the complete sum of chunk r; the all-gather then walks the finished chunks around the same way."""

    plan = _plan(chunk_plan)
    W = plan.world_size
    r = _index(rank, W, "rank")
    nxt, prv = (r + 1) % W, (r - 1) % W
    steps, gathers = [], []
    for s in range(W - 1):
        out_owner, in_owner = (r - s - 1) % W, (r - s - 2) % W
        steps.append(RingReduceScatterStep(
            step_index=s, send_peer=nxt, recv_peer=prv, send_chunk_owner=out_owner, recv_chunk_owner=in_owner,
            received_contributors=tuple((r - s - 1 + k) % W for k in range(s + 1)),
            send_chunk=plan.chunk_for_rank(out_owner), recv_chunk=plan.chunk_for_rank(in_owner)))
        g_out, g_in = (r - s) % W, (r - s - 1) % W
        gathers.append(RingAllGatherStep(
            step_index=s, send_peer=nxt, recv_peer=prv, send_chunk_owner=g_out, recv_chunk_owner=g_in,
            send_chunk=plan.chunk_for_rank(g_out), recv_chunk=plan.chunk_for_rank(g_in)))
    return PipelinedRingSchedule(plan, r, tuple(steps), tuple(gathers))


# ---- tree ----------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TreeEdge:
    """Child-to-parent edge of the reduction tree; the broadcast uses it in the other direction."""

    child_rank: int
    parent_rank: int

    def __post_init__(self) -> None:
        if self.child_rank == self.parent_rank:
            raise ValueError("child_rank and parent_rank must differ")


@dataclass(frozen=True)
class TreeSchedule:
    chunk_plan: ChunkPlan
    rank: int
    root: int
    parent: int | None
    children: tuple[int, ...]
    reduce_edges: tuple[TreeEdge, ...]
    broadcast_edges: tuple[TreeEdge, ...]

    @property
    def local_chunk(self) -> ChunkRange:
        return self.chunk_plan.chunk_for_rank(self.rank)


def tree_edges(world_size: int, root: int = 0) -> tuple[TreeEdge, ...]:
    """Heap-ordered binary tree over the ranks renumbered from `root`: position p hangs under (p - 1) // 2.
    Edges come deepest position first, so replaying them in order reduces every subtree before its parent."""

    if isinstance(world_size, bool) or not isinstance(world_size, int) or world_size <= 0:
        raise ValueError("world_size must be a positive integer")
    root = _index(root, world_size, "root")
    at = [(root + p) % world_size for p in range(world_size)]
    return tuple(TreeEdge(child_rank=at[p], parent_rank=at[(p - 1) // 2]) for p in range(world_size - 1, 0, -1))


def compile_tree_schedule(*, chunk_plan: ChunkPlan, rank: int, root: int = 0) -> TreeSchedule:
    plan = _plan(chunk_plan)
    r = _index(rank, plan.world_size, "rank")
    edges = tree_edges(plan.world_size, root)
    parent = next((e.parent_rank for e in edges if e.child_rank == r), None)
    children = tuple(e.child_rank for e in edges if e.parent_rank == r)
    return TreeSchedule(plan, r, _index(root, plan.world_size, "root"), parent, children, edges,
                        tuple(reversed(edges)))


# ---- what the fused kernels do -------------------------------------------------------------------------
@dataclass(frozen=True)
class DirectExchangeSchedule:
    """One-hop exchange of the two-stage fused all-reduce, from rank `rank`'s point of view.

    scatter: this rank's quantize kernel stores shard d of its tensor into rank d's receive slot `rank`
    (all d, its own included), in the order `scatter_order` (rotated by the rank, so no two senders start
    at the same receiver); reduce: it sums the W slots of its own shard; gather: its decode kernel loads
    the reduced shard s from rank s, in the order `gather_order`.
    """

    chunk_plan: ChunkPlan
    rank: int
    scatter_order: tuple[int, ...]
    gather_order: tuple[int, ...]

    @property
    def local_chunk(self) -> ChunkRange:
        return self.chunk_plan.chunk_for_rank(self.rank)

    @property
    def link_crossings(self) -> int:
        """Times a byte of payload crosses NVLink per rank and direction: (W - 1) / W of it, twice."""

        return 2


def compile_direct_exchange_schedule(*, chunk_plan: ChunkPlan, rank: int) -> DirectExchangeSchedule:
    plan = _plan(chunk_plan)
    r = _index(rank, plan.world_size, "rank")
    order = tuple((r + k) % plan.world_size for k in range(plan.world_size))
    return DirectExchangeSchedule(plan, r, order, order)


@dataclass(frozen=True)
class GatherTile:
    """One 256-thread tile of the decode stage: `count` 16-element chunks of owner `owner`'s reduced shard,
    starting at chunk `start` of that shard."""

    owner: int
    start: int
    count: int


def gather_tiles(*, block: int, grid: int, shard_chunks: int, world_size: int, first_owner: int,
                 tiles_in_flight: int = 1, tile_chunks: int = 256) -> tuple[tuple[GatherTile, ...], ...]:
    """The order in which block `block` of a `grid`-block decode kernel reads the reduced shards.

    Tiles are numbered so that consecutive tiles belong to consecutive owners, starting at `first_owner`
    (the rank itself): tile t is chunks [(t // W) * tile_chunks, ...) of owner (t + first_owner) % W.  A
    block takes tiles block, block + grid, block + 2 grid ... and issues the loads of `tiles_in_flight`
    of them before it decodes the first; each inner tuple is one such batch.  At any instant the blocks of
    a GPU therefore read from all owners at once, and the GPUs, which start at their own index, never
    gang up on one owner.  This is the tiling of `gather_decode_kernel` (and, with one tile in flight, of
    the general reduce kernel's gather order 1), stated on the host so that it can be checked there.
    """

    if min(grid, shard_chunks, world_size, tiles_in_flight, tile_chunks) <= 0:
        raise ValueError("grid, shard_chunks, world_size, tiles_in_flight and tile_chunks must be positive")
    _index(block, grid, "block")
    _index(first_owner, world_size, "first_owner")
    tiles_per_shard = -(-shard_chunks // tile_chunks)
    num_tiles = tiles_per_shard * world_size
    batches = []
    for t0 in range(block, num_tiles, grid * tiles_in_flight):
        batch = []
        for j in range(tiles_in_flight):
            tile = t0 + j * grid
            if tile >= num_tiles:
                continue
            start = (tile // world_size) * tile_chunks
            batch.append(GatherTile((tile + first_owner) % world_size, start, min(tile_chunks, shard_chunks - start)))
        batches.append(tuple(batch))
    return tuple(batches)


# ---- pairwise exchange and butterfly: the other two hop-by-hop shapes ------------------------------------
@dataclass(frozen=True)
class PairwiseStep:
    """Round k of the shifted pairwise exchange: this rank sends its contribution to the chunk owned by
    `send_peer` straight to that owner and receives `recv_peer`'s contribution to its own chunk.  In the
    gather phase the same pairs exchange finished chunks: own chunk out, `recv_peer`'s chunk in."""

    step_index: int
    send_peer: int
    recv_peer: int
    send_chunk: ChunkRange
    recv_chunk: ChunkRange


@dataclass(frozen=True)
class PairwiseSchedule:
    chunk_plan: ChunkPlan
    rank: int
    steps: tuple[PairwiseStep, ...]

    @property
    def local_chunk(self) -> ChunkRange:
        return self.chunk_plan.chunk_for_rank(self.rank)


def compile_pairwise_schedule(*, chunk_plan: ChunkPlan, rank: int) -> PairwiseSchedule:
    """W - 1 rounds; in round k rank r sends to r + k and receives from r - k (mod W), so every round is a
    permutation and works for any world size (the reference pairs ranks by XOR, which needs a power of two:
    ccdl_comm/communication/topology_transport.py:751-863).  Every contribution crosses the network once and
    is quantized once, unlike the ring, where a chunk is re-quantized at each of its W - 1 hops."""

    plan = _plan(chunk_plan)
    W = plan.world_size
    r = _index(rank, W, "rank")
    steps = tuple(PairwiseStep(k - 1, (r + k) % W, (r - k) % W, plan.chunk_for_rank((r + k) % W),
                               plan.chunk_for_rank(r)) for k in range(1, W))
    return PairwiseSchedule(plan, r, steps)


@dataclass(frozen=True)
class ButterflySchedule:
    """Recursive doubling: in round k the rank exchanges its whole partial sum with `peers[k]` = rank XOR 2^k.
    log2(W) rounds of full-size messages: the latency-optimal shape for small tensors."""

    world_size: int
    rank: int
    peers: tuple[int, ...]


def compile_butterfly_schedule(*, world_size: int, rank: int) -> ButterflySchedule:
    if isinstance(world_size, bool) or not isinstance(world_size, int) or world_size <= 0:
        raise ValueError("world_size must be a positive integer")
    if world_size & (world_size - 1):
        raise ValueError("recursive doubling needs a power-of-two world size")
    r = _index(rank, world_size, "rank")
    return ButterflySchedule(world_size, r, tuple(r ^ (1 << k) for k in range(world_size.bit_length() - 1)))
