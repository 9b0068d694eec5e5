"""Hop-by-hop ring and tree all-reduce (quantize -> send/recv -> decode-and-add) on real gloo ranks, compared
bit for bit with a single-process replay of the same schedule through the same codec."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
from conftest import spawn_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * 0.02 * (r + 1)).to(DT[dtype]) for r in range(world)]


def _enc(x, cfg):
    from lowbit_comm_b200.ops import codec

    return codec.quantize_tensor(x.contiguous(), cfg)


def _dec(payload, n, cfg, dtype, into=None, add=False):
    from lowbit_comm_b200.ops import codec

    return codec.dequantize_tensor(payload, (n,), cfg, dtype=dtype, output=into, reduce_op="sum" if add else "none")


_SHARDS = {}        # (method, owner) -> the owner's exact reduced chunk of the most recent replay


def _scaled(x, world, op):
    return x if op == "sum" or world == 1 else (x.float() * (1.0 / world)).to(x.dtype)


def _replay_ring(xs, cfg, dtype, op):
    """What every rank must end with after the ring, computed for all ranks at once."""

    world, n = len(xs), xs[0].numel()
    unit = cfg.group_size * world
    padded = -(-n // unit) * unit
    shard = padded // world
    work = [torch.zeros(padded, dtype=DT[dtype]) for _ in range(world)]
    for w, x in zip(work, xs):
        w[:n] = x
    for s in range(world - 1):
        sent = [_enc(work[r][((r - s - 1) % world) * shard:((r - s - 1) % world + 1) * shard], cfg) for r in range(world)]
        for r in range(world):
            owner = (r - s - 2) % world
            _dec(sent[(r - 1) % world], shard, cfg, dtype, into=work[r][owner * shard:(owner + 1) * shard], add=True)
    final = torch.empty(padded, dtype=DT[dtype])
    for owner in range(world):
        mine = _scaled(work[owner][owner * shard:(owner + 1) * shard], world, op)
        _SHARDS[("ring", owner)] = mine.clone()
        final[owner * shard:(owner + 1) * shard] = _dec(_enc(mine, cfg), shard, cfg, dtype)
    return final[:n]


def _replay_tree(xs, cfg, dtype, op, root=0):
    from lowbit_comm_b200.core.schedules import tree_edges

    world, n = len(xs), xs[0].numel()
    padded = -(-n // cfg.group_size) * cfg.group_size
    work = [torch.zeros(padded, dtype=DT[dtype]) for _ in range(world)]
    for w, x in zip(work, xs):
        w[:n] = x
    for edge in tree_edges(world, root):         # deepest first: a child's buffer already holds its subtree
        _dec(_enc(work[edge.child_rank], cfg), padded, cfg, dtype, into=work[edge.parent_rank], add=True)
    return _dec(_enc(_scaled(work[root], world, op), cfg), padded, cfg, dtype)[:n]


def _replay_pairwise(xs, cfg, dtype, op):
    world, n = len(xs), xs[0].numel()
    unit = cfg.group_size * world
    padded = -(-n // unit) * unit
    shard = padded // world
    work = [torch.zeros(padded, dtype=DT[dtype]) for _ in range(world)]
    for w, x in zip(work, xs):
        w[:n] = x
    final = torch.empty(padded, dtype=DT[dtype])
    for owner in range(world):
        mine = work[owner][owner * shard:(owner + 1) * shard].clone()
        for k in range(1, world):                                    # contributions arrive from owner - k
            sender = (owner - k) % world
            _dec(_enc(work[sender][owner * shard:(owner + 1) * shard], cfg), shard, cfg, dtype, into=mine, add=True)
        _SHARDS[("p2p", owner)] = _scaled(mine, world, op).clone()
        final[owner * shard:(owner + 1) * shard] = _dec(_enc(_scaled(mine, world, op), cfg), shard, cfg, dtype)
    return final[:n]


def _replay_butterfly(xs, cfg, dtype, op):
    world, n = len(xs), xs[0].numel()
    padded = -(-n // cfg.group_size) * cfg.group_size
    work = [torch.zeros(padded, dtype=DT[dtype]) for _ in range(world)]
    for w, x in zip(work, xs):
        w[:n] = x
    for k in range(world.bit_length() - 1):
        sent = [_enc(w, cfg) for w in work]
        for r in range(world):
            _dec(sent[r], padded, cfg, dtype, into=work[r])
            _dec(sent[r ^ (1 << k)], padded, cfg, dtype, into=work[r], add=True)
    assert all(torch.equal(w.view(torch.uint8), work[0].view(torch.uint8)) for w in work)
    return _scaled(work[0], world, op)[:n]


def _worker(rank: int, world: int, port: int) -> None:
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import lowbit_comm_b200 as lbc
        from lowbit_comm_b200.exceptions import UnsupportedCollective
        from lowbit_comm_b200.parallel.schedule_executors import (ButterflyExecutor, PairwiseExecutor,
                                                                  PipelinedRingExecutor, TreeExecutor,
                                                                  make_schedule_all_reduce)

        cases = [("bf16", lbc.CompressionConfig(), 64 * 13 + 5, "mean"),
                 ("fp32", lbc.CompressionConfig(group_size=16, compact=True), 1000, "sum"),
                 ("fp16", lbc.CompressionConfig(bit=4, group_size=32, allow_experimental=True), 7, "mean")]
        for dtype, cfg, n, op in cases:
            xs = _inputs(world, n, dtype, seed=n)
            exact = torch.stack([x.float() for x in xs]).sum(0) / (world if op == "mean" else 1)
            shapes = [(PipelinedRingExecutor, _replay_ring), (TreeExecutor, _replay_tree), (PairwiseExecutor, _replay_pairwise)]
            if world & (world - 1) == 0:
                shapes.append((ButterflyExecutor, _replay_butterfly))
            else:
                with pytest.raises(UnsupportedCollective):
                    ButterflyExecutor(numel=n, dtype=dtype, config=cfg, op=op)
            for cls, replay in shapes:
                executor = cls(numel=n, dtype=dtype, config=cfg, op=op)
                want = replay(xs, cfg, dtype, op)
                for _ in range(2):                                   # buffers are reused across runs
                    got = executor.run(xs[rank].clone())
                    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), (cls.__name__, dtype, n, rank)
                assert executor.runs == 2 and executor.quarantined == 0
                if cfg.bit == 8:
                    bound = 0.03 * world * exact.abs().max().item() + 1e-6
                    assert (got.float() - exact).abs().max().item() <= bound
                if hasattr(executor, "run_reduce_scatter"):
                    shard = executor.run_reduce_scatter(xs[rank].clone())
                    want_shard = _SHARDS[(executor.method, rank)]
                    assert shard.shard_index == rank and shard.world_size == world and shard.original_numel == n
                    assert shard.transport == f"schedule_{executor.method}" and shard.reduce == op
                    assert torch.equal(shard.shard.view(torch.uint8), want_shard.view(torch.uint8))
                    mine_out = torch.empty(shard.shard_numel, dtype=DT[dtype])
                    assert executor.run_reduce_scatter(xs[rank].clone(), out=mine_out).shard is mine_out
                    assert torch.equal(mine_out.view(torch.uint8), want_shard.view(torch.uint8))
                out = torch.empty(n, dtype=DT[dtype])
                kept = xs[rank].clone()
                assert executor.run(kept, out=out) is out and torch.equal(kept, xs[rank])
                assert torch.equal(out.view(torch.uint8), want.view(torch.uint8))
            with pytest.raises(ValueError):
                executor.run(torch.zeros(n + 1, dtype=DT[dtype]))
            with pytest.raises(TypeError):
                executor.run(torch.zeros(n, dtype=torch.float64))

        # the factory form plugs into the public collective like any other topology transport
        cfg = lbc.CompressionConfig()
        xs = _inputs(world, 64 * 9, "bf16", seed=3)
        ring_t = make_schedule_all_reduce(method="ring")
        got = lbc.compressed_all_reduce(xs[rank].clone(), config=cfg, strategy="topology", topology_all_reduce=ring_t)
        assert torch.equal(got.view(torch.uint8), _replay_ring(xs, cfg, "bf16", "mean").view(torch.uint8))
        work = make_schedule_all_reduce(method="tree", root=world - 1)(
            xs[rank].clone(), config=cfg, op="sum", async_op=True, dtype="bf16")
        assert torch.equal(work.wait().view(torch.uint8),
                           _replay_tree(xs, cfg, "bf16", "sum", root=world - 1).view(torch.uint8))
        assert len(ring_t.executors) == 1
        shard_t = lbc.make_native_topology_reduce_scatter_shard(method="ring", hop_by_hop=True)
        _replay_ring(xs, cfg, "bf16", "mean")
        shard = lbc.compressed_reduce_scatter_shard(xs[rank].clone(), config=cfg, reduce_scatter_shard=shard_t)
        assert torch.equal(shard.shard.view(torch.uint8), _SHARDS[("ring", rank)].view(torch.uint8))
        direct = lbc.make_native_topology_all_reduce(method="p2p", hop_by_hop=True)(
            xs[rank].clone(), config=cfg, op="mean", async_op=False, dtype="bf16")
        assert torch.equal(direct.view(torch.uint8), _replay_pairwise(xs, cfg, "bf16", "mean").view(torch.uint8))

        # shared-scale int8 all-reduce: the library adds the codes; floor(127 / W) levels keep the sum inside int8
        from lowbit_comm_b200.parallel.shared_scale import shared_scale_levels

        scale_t = lbc.make_native_topology_all_reduce(method="overlap-scale", hop_by_hop=True)
        worst = [torch.full((130,), 3.0 * (1 if r % 2 == 0 else 1), dtype=torch.bfloat16) for r in range(world)]
        got = scale_t(worst[rank].clone(), config=cfg, op="sum", async_op=False, dtype="bf16")
        assert torch.equal(got, torch.full((130,), 3.0 * world, dtype=torch.bfloat16))      # same sign everywhere: no overflow
        exact = torch.stack([x.float() for x in xs]).mean(0)
        got = scale_t(xs[rank].clone(), config=cfg, op="mean", async_op=True, dtype="bf16").wait()
        amax = torch.stack([x.float().abs() for x in xs]).amax()
        assert (got.float() - exact).abs().max() <= amax / shared_scale_levels(world) / 2 + 1e-3
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        assert all(torch.equal(g, got) for g in gathered)

        if world >= 4:                                                # a sub-group: peers are addressed globally
            members = [1, 3]
            sub = dist.new_group(members, backend="gloo")
            if rank in members:
                pair = [xs[m] for m in members]
                executor = PipelinedRingExecutor(numel=64 * 9, dtype="bf16", config=cfg, group=sub, op="mean")
                got = executor.run(xs[rank].clone())
                assert torch.equal(got.view(torch.uint8), _replay_ring(pair, cfg, "bf16", "mean").view(torch.uint8))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 3, 4, 8))
def test_ring_and_tree_executors_match_their_replay(world):
    spawn_ranks(_worker, lambda port: (world, port), world)


def test_unknown_method_and_reduction_are_refused():
    from lowbit_comm_b200.exceptions import UnsupportedCollective
    from lowbit_comm_b200.parallel.schedule_executors import compile_schedule_all_reduce, make_schedule_all_reduce

    with pytest.raises(UnsupportedCollective):
        make_schedule_all_reduce(method="hypercube")
    with pytest.raises(UnsupportedCollective):
        compile_schedule_all_reduce("mesh", numel=1, dtype="bf16", config=None)
    from lowbit_comm_b200.parallel.shared_scale import shared_scale_levels

    assert [shared_scale_levels(w) for w in (1, 2, 8, 127)] == [127, 63, 15, 1]
    with pytest.raises(UnsupportedCollective):
        shared_scale_levels(128)


class _Request:
    def __init__(self, done):
        self.done = done

    def wait(self):
        if not self.done:
            raise RuntimeError("peer went away")

    def is_completed(self):
        return self.done


class _FakeDist:
    """A two-rank world in which the peer echoes whatever this rank sends; the k-th batch can be made to fail."""

    def __init__(self, fail_at=None):
        self.fail_at, self.batches, self.stuck = fail_at, 0, []

    class P2POp:
        def __init__(self, op, tensor, peer, group=None):
            self.op, self.tensor, self.peer = op, tensor, peer

    isend, irecv = "isend", "irecv"

    def get_rank(self, group=None):
        return 0

    def get_world_size(self, group=None):
        return 2

    def batch_isend_irecv(self, ops):
        self.batches += 1
        failing = self.batches == self.fail_at
        sent = next((o.tensor for o in ops if o.op == "isend"), None)
        for o in ops:
            if o.op == "irecv" and sent is not None and not failing:
                o.tensor.copy_(sent)
        requests = [_Request(not failing) for _ in ops]
        if failing:
            self.stuck = requests
        return requests


def test_failed_step_quarantines_buffers_until_their_requests_complete():
    from lowbit_comm_b200.config import CompressionConfig
    from lowbit_comm_b200.parallel.schedule_executors import PipelinedRingExecutor

    fake = _FakeDist(fail_at=2)
    executor = PipelinedRingExecutor(numel=256, dtype="fp32", config=CompressionConfig(), op="sum", dist=fake)
    x = torch.linspace(-1, 1, 256)
    with pytest.raises(RuntimeError, match="peer went away"):
        executor.run(x.clone())
    assert executor.quarantined == 1 and executor.runs == 0
    first_buffers = executor._quarantine[0][0]
    got = executor.run(x.clone())                      # fresh buffers; the peer echoes: chunk 0 += chunk 1, then comes back
    assert executor._buffers is not first_buffers and executor.runs == 1 and executor.quarantined == 1
    folded = x[:128] + x[128:]
    assert (got[:128] - folded).abs().max() < 0.02 and torch.equal(got[128:], got[:128])
    for request in fake.stuck:
        request.done = True
    assert executor.pending_submission_count == 1 and executor.reap_pending() == 0 and executor.reap() == 0


def test_executor_is_not_reentrant():
    from lowbit_comm_b200.config import CompressionConfig
    from lowbit_comm_b200.parallel.schedule_executors import TreeExecutor

    executor = TreeExecutor(numel=64, dtype="fp32", config=CompressionConfig(), op="sum", dist=_FakeDist())
    assert executor._busy.acquire(blocking=False)
    try:
        with pytest.raises(RuntimeError, match="not re-entrant"):
            executor.run(torch.zeros(64))
    finally:
        executor._busy.release()
