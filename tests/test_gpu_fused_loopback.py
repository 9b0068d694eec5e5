"""Fused push/reduce collectives on ONE GPU with emulated ranks.

Every emulated rank has its own arena on the same device; the phases of a
collective are enqueued for all ranks in turn on one stream, so a kernel that
waits for a flag always starts after the kernels that set it.  Results are
compared with the torch oracle composed the same way.
"""

import os

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.exceptions import AsyncCommunicationError
from lowbit_comm_b200.ops import oracle
from lowbit_comm_b200.parallel.fused import FusedWorkspace, geometry, run_loopback
from lowbit_comm_b200.parallel.peer_memory import PHASE_P2P_DATA, PeerGroup

pytestmark = pytest.mark.gpu

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * 1e-2 * (r + 1)).to(DT[dtype]) for r in range(world)]


def _expected_two_stage(xs, residuals, cfg, dtype, op="mean"):
    n = xs[0].numel()
    prepared = [oracle.prepare(x, r) for x, r in zip(xs, residuals)]
    payloads = [oracle.encode(p, cfg) for p in prepared]
    y, _ = oracle.reduce_mean(payloads, n, cfg, dtype, None if op == "mean" else 1.0)
    again = oracle.encode(y, cfg)
    z32 = oracle.decode_fp32(again, n, cfg, dtype)
    return z32.to(DT[dtype]), [oracle.residual_update(p, z32) for p in prepared], prepared


def _expected_one_stage(xs, residuals, cfg, dtype, op="mean"):
    n = xs[0].numel()
    prepared = [oracle.prepare(x, r) for x, r in zip(xs, residuals)]
    payloads = [oracle.encode(p, cfg) for p in prepared]
    y, y32 = oracle.reduce_mean(payloads, n, cfg, dtype, None if op == "mean" else 1.0)
    return y, [oracle.residual_update(p, y32) for p in prepared], prepared


def _make(world, dtype, cfg, max_numel, **kw):
    need = FusedWorkspace.required_bytes(world, dtype, cfg, max_numel, True) + (1 << 20)
    groups = PeerGroup.loopback(world, need, timeout_ns=2_000_000_000)
    return groups, [FusedWorkspace(g, dtype=dtype, config=cfg, max_numel=max_numel, with_gather_region=True, **kw)
                    for g in groups]


@pytest.mark.parametrize("engine", ("pipe", "legacy"))
@pytest.mark.parametrize("world", (1, 2, 4, 8))
@pytest.mark.parametrize("dtype,bit,group", [("bf16", 8, 64), ("fp16", 8, 32), ("fp32", 8, 64), ("bf16", 4, 16)])
@pytest.mark.parametrize("stages", (1, 2))
def test_all_reduce_matches_oracle(ext, engine, world, dtype, bit, group, stages):
    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    max_numel = 40_000
    groups, wss = _make(world, dtype, cfg, max_numel, engine=engine)
    try:
        for step, n in enumerate((world * group * 8, 3001, 1, max_numel, 64 * 511 + 7)):
            xs = _inputs(world, n, dtype, seed=step)
            rs = _inputs(world, n, dtype, seed=100 + step)
            dev_x = [x.cuda() for x in xs]
            dev_r = [r.cuda() for r in rs]
            outs = [torch.empty_like(x) for x in dev_x]
            run_loopback(wss, "all_reduce", [(dev_x[r], outs[r]) for r in range(world)],
                         residual=None, stages=stages)
            expect = (_expected_one_stage if stages == 1 else _expected_two_stage)(xs, [None] * world, cfg, dtype)
            for r in range(world):
                assert torch.equal(outs[r].cpu().view(torch.uint8), expect[0].view(torch.uint8)), (n, r)
            # with error feedback, in place (the DDP hook's form)
            dev_x = [x.cuda() for x in xs]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)], stages=stages)
            expect = (_expected_one_stage if stages == 1 else _expected_two_stage)(xs, rs, cfg, dtype)
            for r in range(world):
                assert torch.equal(dev_x[r].cpu().view(torch.uint8), expect[0].view(torch.uint8)), (n, r, "ef")
                assert torch.equal(dev_r[r].cpu().view(torch.uint8), expect[1][r].view(torch.uint8)), (n, r, "res")
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("push_variant,reduce_bulk,push_blocks",
                         [(0, False, -1), (0, True, 0), (1, False, 0), (1, True, -1), (2, False, 3), (2, True, 0)])
@pytest.mark.parametrize("dtype,bit,group", [("bf16", 8, 64), ("fp32", 4, 32)])
def test_every_push_variant_writes_the_same_bytes(ext, push_variant, reduce_bulk, push_blocks, dtype, bit, group):
    """Classic, shard-interleaved and bulk-store pushes (and both broadcast forms of the reduce
    stage, with and without a grid cap) must be indistinguishable to the consumer."""

    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    world, max_numel = 4, 300_000
    groups, wss = _make(world, dtype, cfg, max_numel, engine="legacy")
    ext.set_push_variant(push_variant, reduce_bulk, push_blocks)
    try:
        for step, n in enumerate((world * group * 8, 70_001, max_numel)):
            xs = _inputs(world, n, dtype, seed=step)
            rs = _inputs(world, n, dtype, seed=50 + step)
            for stages, expected, gather in ((1, _expected_one_stage, "pull"), (2, _expected_two_stage, "pull"),
                                             (2, _expected_two_stage, "push")):
                for ws in wss:
                    ws.set_gather_mode(gather)
                dev_x = [x.cuda() for x in xs]
                dev_r = [r.cuda() for r in rs]
                run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                             [{"residual": dev_r[r]} for r in range(world)], stages=stages)
                want = expected(xs, rs, cfg, dtype)
                for r in range(world):
                    assert torch.equal(dev_x[r].cpu().view(torch.uint8), want[0].view(torch.uint8)), (n, stages, gather, r)
                    assert torch.equal(dev_r[r].cpu().view(torch.uint8), want[1][r].view(torch.uint8)), (n, stages, gather, r)
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        ext.set_push_variant(1, True, 0)
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("order", (0, 1))
@pytest.mark.parametrize("world", (3, 8))
@pytest.mark.parametrize("dtype,bit,group", [("bf16", 8, 64), ("fp16", 4, 16), ("fp32", 8, 32)])
def test_gather_sweep_orders(ext, order, world, dtype, bit, group):
    """The decode stage may walk the owners' shards linearly or tile by tile round-robin; same result."""

    cfg = CompressionConfig(bit=bit, group_size=group, allow_experimental=True)
    max_numel = 200_000
    groups, wss = _make(world, dtype, cfg, max_numel, engine="legacy")
    ext.set_gather_order(order)
    try:
        for step, n in enumerate((world * group * 8, 12_345, 1, max_numel, group * 8 * world * 31 + 5)):
            xs = _inputs(world, n, dtype, seed=400 + step)
            rs = _inputs(world, n, dtype, seed=500 + step)
            dev_x = [x.cuda() for x in xs]
            dev_r = [r.cuda() for r in rs]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)], stages=2)
            want = _expected_two_stage(xs, rs, cfg, dtype)
            for r in range(world):
                assert torch.equal(dev_x[r].cpu().view(torch.uint8), want[0].view(torch.uint8)), (n, r)
                assert torch.equal(dev_r[r].cpu().view(torch.uint8), want[1][r].view(torch.uint8)), (n, r)
    finally:
        ext.set_gather_order(1)
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("depth", (2, 4))
@pytest.mark.parametrize("world", (3, 8))
@pytest.mark.parametrize("dtype,group", [("bf16", 64), ("fp16", 16), ("fp32", 32)])
def test_gather_decode_with_tiles_in_flight(ext, depth, world, dtype, group):
    """The specialised decode kernel (several tiles of loads in flight) gives the general kernel's bits."""

    cfg = CompressionConfig(bit=8, group_size=group)
    max_numel = 200_000
    groups, wss = _make(world, dtype, cfg, max_numel, engine="legacy")
    ext.set_gather_prefetch(depth)
    try:
        assert ext.get_gather_prefetch() == depth
        for step, n in enumerate((world * group * 8, 12_345, 1, max_numel, group * 8 * world * 31 + 5)):
            xs = _inputs(world, n, dtype, seed=600 + step)
            rs = _inputs(world, n, dtype, seed=700 + step)
            dev_x = [x.cuda() for x in xs]
            dev_r = [r.cuda() for r in rs]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)], stages=2)
            want = _expected_two_stage(xs, rs, cfg, dtype)
            for r in range(world):
                assert torch.equal(dev_x[r].cpu().view(torch.uint8), want[0].view(torch.uint8)), (n, r)
                assert torch.equal(dev_r[r].cpu().view(torch.uint8), want[1][r].view(torch.uint8)), (n, r)
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        ext.set_gather_prefetch(0)
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("engine", ("pipe", "legacy"))
@pytest.mark.parametrize("world,stages", [(2, 1), (4, 2), (8, 2)])
@pytest.mark.parametrize("dtype", ("bf16", "fp32"))
def test_local_error_feedback_mode(ext, engine, world, stages, dtype):
    """ef_mode="local": the residual becomes this rank's own quantization error, over several steps."""

    cfg = CompressionConfig()
    n = 64 * 777 + 5
    groups, wss = _make(world, dtype, cfg, n, engine=engine)
    try:
        residual_ref = [torch.zeros(n, dtype=DT[dtype]) for _ in range(world)]
        dev_r = [r.cuda() for r in residual_ref]
        for step in range(3):
            xs = _inputs(world, n, dtype, seed=300 + step)
            dev_x = [x.cuda() for x in xs]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r], "ef_mode": "local"} for r in range(world)], stages=stages)
            prepared = [oracle.prepare(x, r) for x, r in zip(xs, residual_ref)]
            payloads = [oracle.encode(p, cfg) for p in prepared]
            y, _ = oracle.reduce_mean(payloads, n, cfg, dtype)
            want = y if stages == 1 else oracle.decode(oracle.encode(y, cfg), n, cfg, dtype)
            residual_ref = [oracle.local_error(p, q, cfg) for p, q in zip(prepared, payloads)]
            for r in range(world):
                assert torch.equal(dev_x[r].cpu().view(torch.uint8), want.view(torch.uint8)), (step, r)
                assert torch.equal(dev_r[r].cpu().view(torch.uint8), residual_ref[r].view(torch.uint8)), (step, r)
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world", (2, 4, 8))
def test_reduce_scatter_and_all_gather(ext, world):
    cfg = CompressionConfig()
    dtype, n = "bf16", 64 * 300 + 17
    groups, wss = _make(world, dtype, cfg, n)
    try:
        xs = _inputs(world, n, dtype, seed=5)
        dev = [x.cuda() for x in xs]
        geo = geometry(n, world, dtype, cfg)
        shards = [torch.full((geo.shard_numel,), 7.0, dtype=DT[dtype], device="cuda") for _ in range(world)]
        run_loopback(wss, "reduce_scatter", [(dev[r], shards[r]) for r in range(world)])
        payloads = [oracle.encode(x, cfg) for x in xs]
        y, _ = oracle.reduce_mean(payloads, n, cfg, dtype)
        padded = torch.zeros(geo.shard_numel * world, dtype=DT[dtype])
        padded[:n] = y
        for r in range(world):
            want = padded[r * geo.shard_numel:(r + 1) * geo.shard_numel]
            assert torch.equal(shards[r].cpu().view(torch.uint8), want.view(torch.uint8)), r
        outs = [[torch.empty(n, dtype=DT[dtype], device="cuda") for _ in range(world)] for _ in range(world)]
        run_loopback(wss, "all_gather", [(dev[r], outs[r]) for r in range(world)])
        for r in range(world):
            for s in range(world):
                want = oracle.decode(payloads[s], n, cfg, dtype)
                assert torch.equal(outs[r][s].cpu().view(torch.uint8), want.view(torch.uint8)), (r, s)
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world,stages", [(2, 1), (3, 2), (8, 2)])
@pytest.mark.parametrize("dtype,group", [("bf16", 64), ("fp32", 16)])
@pytest.mark.parametrize("ring", [2, 3, 4])
def test_pipelined_engine_many_rows_and_ring_depths(ext, world, stages, dtype, group, ring):
    """Tensors of many rows through shared-memory rings of every depth: the static row schedule and the
    stage re-use must not change a bit of the result.  Unaligned views exercise the rows that bypass the
    copy engine."""

    cfg = CompressionConfig(bit=8, group_size=group)
    max_numel = 700_000
    groups, wss = _make(world, dtype, cfg, max_numel, engine="pipe")
    for ws in wss:
        ws._pipe.set_ring_depth(ring)
    expected = _expected_one_stage if stages == 1 else _expected_two_stage
    try:
        for step, (n, skew) in enumerate(((max_numel, 0), (4096 * world * 5, 0), (333_333, 0), (250_001, 3))):
            xs = _inputs(world, n, dtype, seed=800 + step)
            rs = _inputs(world, n, dtype, seed=900 + step)
            # `skew` elements of offset make x, the output and the residual 16-byte unaligned
            dev_x = [torch.cat([torch.zeros(skew, dtype=x.dtype), x]).cuda()[skew:] for x in xs]
            dev_r = [torch.cat([torch.zeros(skew, dtype=r.dtype), r]).cuda()[skew:] for r in rs]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)], stages=stages)
            want = expected(xs, rs, cfg, dtype)
            for r in range(world):
                assert torch.equal(dev_x[r].cpu().view(torch.uint8), want[0].view(torch.uint8)), (n, r)
                assert torch.equal(dev_r[r].cpu().view(torch.uint8), want[1][r].view(torch.uint8)), (n, r)
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


def test_pipelined_engine_single_rank_runs_all_phases_in_one_launch(ext):
    """World size 1 (a one-GPU DDP job): the three phases run inside one launch and meet through the flags."""

    cfg = CompressionConfig()
    n = 3_000_000
    groups, wss = _make(1, "bf16", cfg, n, engine="pipe")
    try:
        for stages in (1, 2):
            xs, rs = _inputs(1, n, "bf16", seed=11), _inputs(1, n, "bf16", seed=12)
            dev_x, dev_r = xs[0].cuda(), rs[0].cuda()
            before = wss[0].launches
            wss[0].all_reduce(dev_x, residual=dev_r, stages=stages)
            assert wss[0].launches == before + 1
            want = (_expected_one_stage if stages == 1 else _expected_two_stage)(xs, rs, cfg, "bf16")
            assert torch.equal(dev_x.cpu().view(torch.uint8), want[0].view(torch.uint8)), stages
            assert torch.equal(dev_r.cpu().view(torch.uint8), want[1][0].view(torch.uint8)), stages
        groups[0].check_status()
    finally:
        PeerGroup.close_loopback(groups)


def test_pipelined_engine_wait_runs_out_on_a_flag_nobody_sets(ext):
    """REDUCE rows of a rank whose peer never quantized: the bounded wait gives up, the status word says
    which peer was missing, and after a reset the workspace serves the next collective."""

    cfg = CompressionConfig()
    n = 100_000
    need = FusedWorkspace.required_bytes(2, "bf16", cfg, n, True) + (1 << 20)
    groups = PeerGroup.loopback(2, need, timeout_ns=50_000_000)   # 50 ms
    try:
        wss = [FusedWorkspace(g, dtype="bf16", config=cfg, max_numel=n, engine="pipe") for g in groups]
        x = torch.randn(n).to(torch.bfloat16).cuda()
        ws, g = wss[0], groups[0]
        epoch = g.next_epoch(ws.channel)
        stream = torch.cuda.current_stream().cuda_stream
        # rank 0 quantizes and then wants to reduce; rank 1 never runs, so its flag never comes
        ext.pipe_all_reduce(ws._pipe, x.data_ptr(), x.data_ptr(), 0, n, 1, 0.5, False, False, epoch, stream,
                            int(ext.PIPE_QUANT), False)
        ext.pipe_all_reduce(ws._pipe, x.data_ptr(), x.data_ptr(), 0, n, 1, 0.5, False, False, epoch, stream,
                            int(ext.PIPE_REDUCE), False)
        torch.cuda.synchronize()      # returns: the wait is bounded
        with pytest.raises(AsyncCommunicationError) as info:
            g.check_status()
        assert info.value.status["expected"] == epoch and info.value.status["peer"] == 1
        g.reset_after_error()
        ws.reset_pipe_control()
        groups[1].next_epoch(wss[1].channel)
        g.check_status()
        xs = _inputs(2, n, "bf16", seed=3)
        dev = [t.cuda() for t in xs]
        run_loopback(wss, "all_reduce", [(dev[r],) for r in range(2)], stages=1)
        want = _expected_one_stage(xs, [None, None], cfg, "bf16")
        for r in range(2):
            assert torch.equal(dev[r].cpu().view(torch.uint8), want[0].view(torch.uint8)), r
        g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world", (2, 4))
@pytest.mark.parametrize("dtype,group", [("bf16", 64), ("fp32", 32)])
def test_gather_shards_writes_the_whole_tensor_in_one_decode(ext, world, dtype, group):
    """The closing stage of the hierarchical all-reduce: every rank's dense shard, quantized once, decoded by
    every rank straight into the full tensor; twice in a row (the two halves of the region alternate)."""

    cfg = CompressionConfig(bit=8, group_size=group)
    n = group * 8 * world * 13 + 37
    groups, wss = _make(world, dtype, cfg, n)
    try:
        geo = geometry(n, world, dtype, cfg)
        for step in range(3):
            full = _inputs(1, geo.shard_numel * world, dtype, seed=40 + step)[0]
            shards = [full[r * geo.shard_numel:(r + 1) * geo.shard_numel].clone() for r in range(world)]
            outs = [torch.full((n,), 5.0, dtype=DT[dtype], device="cuda") for _ in range(world)]
            run_loopback(wss, "gather_shards", [(shards[r].cuda(), outs[r]) for r in range(world)])
            want = torch.cat([oracle.decode(oracle.encode(sh, cfg), geo.shard_numel, cfg, dtype) for sh in shards])[:n]
            for r in range(world):
                assert torch.equal(outs[r].cpu().view(torch.uint8), want.view(torch.uint8)), (step, r)
        torch.cuda.synchronize()
        for g in groups:
            g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world", (2, 4, 8))
@pytest.mark.parametrize("dtype", ("bf16", "fp32"))
@pytest.mark.parametrize("kw", [dict(bit=8, group_size=64, topk=1), dict(bit=8, group_size=64, topk=2),
                                dict(bit=4, group_size=32, topk=1, quant_type="e2m1"),
                                dict(bit=4, group_size=16, quant_type="normal")])
@pytest.mark.parametrize("fused", (True, False))
def test_topk_and_codebook_profiles_through_peer_memory(ext, world, dtype, kw, fused):
    """Profiles outside the production kernels (top-k outliers, 4-bit code-books) all-reduced over peer memory,
    by the two fused kernels (quantize-and-push, wait-decode-sum-scale-residual) and by the composition of
    separate launches: bit for bit what the codec gives for the gathered payloads, and the reference's
    error-feedback rule."""

    from lowbit_comm_b200.ops import codec
    from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

    cfg = CompressionConfig(allow_experimental=True, **kw)
    max_numel = 70_000
    need = GeneralPeerWorkspace.required_bytes(world, dtype, cfg, max_numel) + (1 << 20)
    groups = PeerGroup.loopback(world, need, timeout_ns=2_000_000_000)
    try:
        wss = [GeneralPeerWorkspace(g, dtype=dtype, config=cfg, max_numel=max_numel, fused=fused) for g in groups]
        for step, n in enumerate((cfg.group_size * 8 * world, 12_347, 1, max_numel)):
            xs = _inputs(world, n, dtype, seed=30 + step)
            rs = _inputs(world, n, dtype, seed=60 + step)
            dev_x = [x.cuda() for x in xs]
            dev_r = [r.cuda() for r in rs]
            payloads, prepared = [], []
            for x, r in zip(xs, rs):
                keep = r.cuda()
                payloads.append(codec.quantize_tensor(x.cuda(), cfg, residual=keep, prepared_out=keep))
                prepared.append(keep)
            want = codec.dequantize_reduce_tensors(payloads, (n,), cfg, dtype=dtype, reduce="mean")
            want_res = [codec.update_error_feedback_residual(p, want, p.clone()) for p in prepared]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)])
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(dev_x[r].view(torch.uint8), want.view(torch.uint8)), (n, r)
                assert torch.equal(dev_r[r].view(torch.uint8), want_res[r].view(torch.uint8)), (n, r, "residual")
            exact = torch.stack([(x.float() + r.float()) for x, r in zip(xs, rs)]).mean(0)
            rel = ((want.float().cpu() - exact).norm() / exact.norm()).item()
            assert rel < (0.05 if cfg.bit == 8 else 0.25), rel
        if fused:
            assert wss[0].launches == 2 * 4          # two kernels per collective
            # no residual, a separate output, a sum: the other branches of the fused reduce
            xs = _inputs(world, 4_001, dtype, seed=99)
            outs = [torch.empty(4_001, dtype=xs[0].dtype, device="cuda") for _ in range(world)]
            payloads = [codec.quantize_tensor(x.cuda(), cfg) for x in xs]
            want = codec.dequantize_reduce_tensors(payloads, (4_001,), cfg, dtype=dtype, reduce="sum")
            run_loopback(wss, "all_reduce", [(xs[r].cuda(), outs[r]) for r in range(world)], op="sum")
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(outs[r].view(torch.uint8), want.view(torch.uint8)), r
        for g in groups:
            g.check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world", (2, 4, 8))
@pytest.mark.parametrize("dtype", ("bf16", "fp32"))
@pytest.mark.parametrize("kw", [dict(bit=8, group_size=64, topk=1), dict(bit=8, group_size=64, topk=2, compact=True),
                                dict(bit=4, group_size=16, quant_type="normal")])
def test_topk_two_stage_all_reduce_matches_the_two_quantizations(ext, world, dtype, kw):
    """stages=2 of the general-profile all-reduce (scatter, reduce, quantize again, gather): the result is
    decode(quant(y)) for y = the one-stage mean of the ranks' payloads, and the residual T(prepared - result), bit
    for bit, on sizes that leave shards partly or wholly empty."""

    from lowbit_comm_b200.ops import codec
    from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

    cfg = CompressionConfig(allow_experimental=True, **kw)
    max_numel = 70_000
    need = GeneralPeerWorkspace.required_bytes(world, dtype, cfg, max_numel) + (1 << 20)
    groups = PeerGroup.loopback(world, need, timeout_ns=2_000_000_000)
    try:
        wss = [GeneralPeerWorkspace(g, dtype=dtype, config=cfg, max_numel=max_numel) for g in groups]
        for step, n in enumerate((cfg.group_size * 8 * world, 12_347, 1, cfg.group_size * 8 + 3, max_numel)):
            xs = _inputs(world, n, dtype, seed=130 + step)
            rs = _inputs(world, n, dtype, seed=160 + step)
            dev_x = [x.cuda() for x in xs]
            dev_r = [r.cuda() for r in rs]
            payloads, prepared = [], []
            for x, r in zip(xs, rs):
                keep = r.cuda()
                payloads.append(codec.quantize_tensor(x.cuda(), cfg, residual=keep, prepared_out=keep))
                prepared.append(keep)
            y = codec.dequantize_reduce_tensors(payloads, (n,), cfg, dtype=dtype, reduce="mean")
            want = codec.dequantize_tensor(codec.quantize_tensor(y, cfg), (n,), cfg, dtype=dtype)
            want_res = [codec.update_error_feedback_residual(p, want, p.clone()) for p in prepared]
            run_loopback(wss, "all_reduce", [(dev_x[r],) for r in range(world)],
                         [{"residual": dev_r[r]} for r in range(world)], stages=2)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(dev_x[r].view(torch.uint8), want.view(torch.uint8)), (n, r)
                assert torch.equal(dev_r[r].view(torch.uint8), want_res[r].view(torch.uint8)), (n, r, "residual")
        assert wss[0].launches == 4 * 5
        # one- and two-stage calls share the receive regions: alternate them, no residual, a sum
        xs = _inputs(world, 9_999, dtype, seed=199)
        payloads = [codec.quantize_tensor(x.cuda(), cfg) for x in xs]
        y = codec.dequantize_reduce_tensors(payloads, (9_999,), cfg, dtype=dtype, reduce="sum")
        two = codec.dequantize_tensor(codec.quantize_tensor(y, cfg), (9_999,), cfg, dtype=dtype)
        for stages, want in ((1, y), (2, two), (2, two), (1, y)):
            outs = [torch.empty(9_999, dtype=xs[0].dtype, device="cuda") for _ in range(world)]
            run_loopback(wss, "all_reduce", [(xs[r].cuda(), outs[r]) for r in range(world)], op="sum", stages=stages)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(outs[r].view(torch.uint8), want.view(torch.uint8)), (stages, r)
        for g in groups:
            g.check_status()
            g.check_canaries()
    finally:
        PeerGroup.close_loopback(groups)


def test_fused_general_reduce_wait_runs_out_on_a_signal_nobody_sends(ext):
    """One emulated rank of two never pushes: the reduce kernel of the other gives up after its bound, reports
    the missing peer in the status word and leaves the output untouched; the context stays usable."""

    from lowbit_comm_b200.exceptions import AsyncCommunicationError
    from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

    cfg = CompressionConfig(allow_experimental=True, bit=8, group_size=64, topk=1)
    n = 5_000
    need = GeneralPeerWorkspace.required_bytes(2, "bf16", cfg, n) + (1 << 20)
    groups = PeerGroup.loopback(2, need, timeout_ns=50_000_000)
    try:
        ws = GeneralPeerWorkspace(groups[0], dtype="bf16", config=cfg, max_numel=n)
        x = _inputs(1, n, "bf16", seed=5)[0].cuda()
        before = x.clone()
        ws.all_reduce(x)                       # rank 1 stays silent
        torch.cuda.synchronize()
        with pytest.raises(AsyncCommunicationError):
            groups[0].check_status()
        assert torch.equal(x, before)
        groups[0].reset_after_error()
        groups[0].check_status()
    finally:
        PeerGroup.close_loopback(groups)


@pytest.mark.parametrize("world", (2, 8))
def test_all_gather_into_one_buffer_is_a_single_decode_launch(ext, world):
    """Outputs that are the rows of one buffer, payloads of whole 8-group units: one decode launch for all W."""

    cfg = CompressionConfig()
    dtype, n = "bf16", 64 * 8 * 25
    groups, wss = _make(world, dtype, cfg, n)
    try:
        xs = _inputs(world, n, dtype, seed=9)
        dev = [x.cuda() for x in xs]
        bufs = [torch.empty(world, n, dtype=DT[dtype], device="cuda") for _ in range(world)]
        before = wss[0].launches
        run_loopback(wss, "all_gather", [(dev[r], list(bufs[r].unbind(0))) for r in range(world)])
        assert wss[0].launches - before == 3          # quantize + broadcast, gate, one decode
        for r in range(world):
            for src in range(world):
                want = oracle.decode(oracle.encode(xs[src], cfg), n, cfg, dtype)
                assert torch.equal(bufs[r][src].cpu().view(torch.uint8), want.view(torch.uint8)), (r, src)
    finally:
        PeerGroup.close_loopback(groups)


def test_bounded_wait_reports_status_instead_of_hanging(ext):
    """A flag that nothing sets: the kernel gives up after its time limit and says why."""

    groups = PeerGroup.loopback(2, 1 << 20, timeout_ns=50_000_000)  # 50 ms
    try:
        g = groups[0]
        ch = g.new_channel()
        ext.wait_signal(g.wait_all(ch, PHASE_P2P_DATA, epoch=1), None)
        torch.cuda.synchronize()  # returns: the wait is bounded
        with pytest.raises(AsyncCommunicationError) as info:
            g.check_status()
        assert info.value.status["expected"] == 1 and info.value.status["seen"] == 0
        g.reset_after_error()
        g.check_status()
        # the context is still usable
        assert torch.ones(4, device="cuda").sum().item() == 4
    finally:
        PeerGroup.close_loopback(groups)


def test_canaries_catch_a_write_past_a_region(ext):
    """Every arena region is followed by a canary; an overrun (here: a deliberate host-side memset through
    the arena's own tensor view, no kernel misbehaves) is reported by `check_canaries`."""

    from lowbit_comm_b200.exceptions import CCDLError

    groups = PeerGroup.loopback(2, 1 << 20)
    try:
        off = groups[0].alloc(1000)
        groups[1].alloc(1000)
        groups[0].check_canaries()
        groups[0].local_view(off, 1024 + 8)[-1] = 0     # region rounded up to 1024 bytes, then the canary
        with pytest.raises(CCDLError):
            groups[0].check_canaries()
        groups[1].check_canaries()
    finally:
        PeerGroup.close_loopback(groups, check=False)
