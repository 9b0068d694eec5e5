"""Child-process body of the multi-GPU tests: one process per GPU, NCCL rendezvous on
127.0.0.1, results checked against the torch oracle computed from every rank's seed."""

import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _inputs(world, n, dtype, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * 1e-2 * (r + 1)).to(dtype) for r in range(world)]


def collectives_case(rank: int, world: int) -> None:
    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.ops import oracle
    from lowbit_comm_b200.parallel.collectives import (compressed_all_gather, compressed_all_reduce,
                                                        compressed_hierarchical_all_reduce,
                                                        compressed_reduce_scatter_shard)
    from lowbit_comm_b200.parallel.communicator import get_communicator
    from lowbit_comm_b200.parallel.fused import geometry

    cfg = CompressionConfig()
    dt, name = torch.bfloat16, "bf16"
    comm = get_communicator(None)
    for step, n in enumerate((64 * 8 * world, 100_003, 1, 3_000_017)):
        xs = _inputs(world, n, dt, seed=step)
        payloads = [oracle.encode(x, cfg) for x in xs]
        y, _ = oracle.reduce_mean(payloads, n, cfg, name)
        two = oracle.decode(oracle.encode(y, cfg), n, cfg, name)
        for strategy, want in (("all_gather", y), ("reduce_scatter", two)):
            mine = xs[rank].cuda()
            ws = comm.workspace(mine, cfg, name)
            assert ws.engine == "auto"      # the default: one persistent kernel per all-reduce up to a size limit
            got = compressed_all_reduce(mine, config=cfg, op="mean", strategy=strategy)
            torch.cuda.synchronize()
            assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), (strategy, n, rank)
            # with error feedback (residual starts at zero, so prepared == input), through both engines; the
            # kernel sequence of the legacy engine runs its gather stage both as peer loads by the decode
            # kernel and as peer stores by the reduce kernel
            reduced32 = (oracle.reduce_mean(payloads, n, cfg, name)[1] if strategy == "all_gather"
                         else oracle.decode_fp32(oracle.encode(y, cfg), n, cfg, name))
            want_res = oracle.residual_update(xs[rank], reduced32)
            for engine, gather, gate in (("pipe", "pull", False), ("pipe", "pull", True), ("legacy", "push", False),
                                         ("legacy", "pull", False)):
                ws.set_engine(engine)
                ws.set_gather_mode(gather)
                ws.gate = gate
                if engine == "legacy" and n > 50_000:   # the multi-stream launcher with up to 8 chunks
                    ws.set_chunking(1 << 17, 8)
                residual = torch.zeros_like(mine)
                got = ws.all_reduce(xs[rank].cuda(), residual=residual, op="mean",
                                    stages=1 if strategy == "all_gather" else 2)
                torch.cuda.synchronize()
                assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), (strategy, n, engine, gather)
                assert torch.equal(residual.cpu().view(torch.uint8), want_res.view(torch.uint8)), \
                    (strategy, n, engine, gather, "residual")
            ws.set_engine("auto")
            ws.gate = False
        work = compressed_all_reduce(xs[rank].cuda(), config=cfg, strategy="reduce_scatter", async_op=True)
        got = work.wait()
        torch.cuda.current_stream().synchronize()
        assert torch.equal(got.cpu().view(torch.uint8), two.view(torch.uint8)), ("async", n, rank)
        geo = geometry(n, world, name, cfg)
        shard = compressed_reduce_scatter_shard(xs[rank].cuda(), config=cfg, op="mean")
        torch.cuda.synchronize()
        padded = torch.zeros(geo.shard_numel * world, dtype=dt)
        padded[:n] = y
        want = padded[rank * geo.shard_numel:(rank + 1) * geo.shard_numel]
        assert shard.shard_index == rank and shard.transport == "fused_peer_scatter"
        assert torch.equal(shard.shard.cpu().view(torch.uint8), want.view(torch.uint8)), ("shard", n, rank)
        outs = compressed_all_gather(xs[rank].cuda(), config=cfg)
        torch.cuda.synchronize()
        for s in range(world):
            assert torch.equal(outs[s].cpu().view(torch.uint8),
                               oracle.decode(payloads[s], n, cfg, name).view(torch.uint8)), ("gather", n, rank, s)
    if world >= 4 and world % 2 == 0:
        n = 200_000
        xs = _inputs(world, n, dt, seed=77)
        L = world // 2
        for _ in range(2):      # twice: the second run reuses every region and flag of the first
            got = compressed_hierarchical_all_reduce(xs[rank].cuda(), config=cfg, op="mean", local_group_size=L)
            torch.cuda.synchronize()
        # the same three stages on the host: mean inside each group of L ranks (one quantization), mean of
        # the groups' results shard by shard (a second one), and the gather of the shards (a third one)
        geo = geometry(n, L, name, cfg)
        stage1 = [oracle.reduce_mean([oracle.encode(xs[g0 + r], cfg) for r in range(L)], n, cfg, name)[0]
                  for g0 in range(0, world, L)]
        pad = geo.shard_numel * L - n
        padded = [torch.cat([t, torch.zeros(pad, dtype=dt)]) for t in stage1]
        shards = []
        for lane in range(L):
            pieces = [p[lane * geo.shard_numel:(lane + 1) * geo.shard_numel] for p in padded]
            shards.append(oracle.reduce_mean([oracle.encode(p, cfg) for p in pieces], geo.shard_numel, cfg, name)[0])
        want = torch.cat([oracle.decode(oracle.encode(sh, cfg), geo.shard_numel, cfg, name) for sh in shards])[:n]
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), ("hierarchical", rank)
    # the hop-by-hop ring and tree executors over NCCL send / receive (the path for groups without peer access):
    # bit for bit what a single-process replay of the same schedule through the same codec gives
    import test_cpu_gloo_schedule_executors as replay
    from lowbit_comm_b200.parallel.transports import make_native_topology_all_reduce

    n = 64 * world * 37 + 11
    xs = _inputs(world, n, dt, seed=300)
    for method, expected in (("ring", replay._replay_ring), ("tree", replay._replay_tree)):
        transport = make_native_topology_all_reduce(method=method, hop_by_hop=True)
        got = transport(xs[rank].cuda(), config=cfg, op="mean", async_op=False, dtype=name)
        torch.cuda.synchronize()
        want = expected(xs, cfg, name, "mean")
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), ("hop by hop", method, rank)
    # top-k profiles through the two fused general kernels (quantize-and-push over NVLink, then wait + decode +
    # sum + scale + residual in one pass): bit for bit the codec's result for the same payloads, twice in a row
    # (both receive regions), with the reference's error-feedback rule
    from lowbit_comm_b200.ops import codec

    for k in (1, 2):
        kcfg = CompressionConfig(topk=k, allow_experimental=True)
        n = 77_777
        residual = torch.zeros(n, dtype=dt, device="cuda")
        expect_res = [torch.zeros(n, dtype=dt, device="cuda") for _ in range(world)]
        for it in range(2):
            xs = _inputs(world, n, dt, seed=400 + 10 * k + it)
            payloads = [codec.quantize_tensor(xs[r].cuda(), kcfg, residual=expect_res[r], prepared_out=expect_res[r])
                        for r in range(world)]
            want = codec.dequantize_reduce_tensors(payloads, (n,), kcfg, dtype=name, reduce="mean")
            for r in range(world):      # every rank's residual moves on: prepared -> T(prepared - result)
                codec.update_error_feedback_residual(expect_res[r], want, expect_res[r])
            got = comm.all_reduce(xs[rank].cuda(), config=kcfg, op="mean", residual=residual)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), ("top-k", k, it, rank)
            assert torch.equal(residual.view(torch.uint8), expect_res[rank].view(torch.uint8)), ("top-k residual", k, it)
        assert comm.general_workspace(residual, kcfg, name).fused
    # quantized point-to-point through the peer mailboxes: a ring, three rounds (the second and third
    # sends first wait for the receiver's acknowledgement of the previous message)
    import lowbit_comm_b200 as lbc

    comm.enable_peer_mailbox(1 << 20)
    n, nxt, prv = 50_001, (rank + 1) % world, (rank - 1) % world
    for it in range(3):
        xs = _inputs(world, n, dt, seed=200 + it)
        recv = torch.empty(n, dtype=dt, device="cuda")
        sent = lbc.iqsend(xs[rank].cuda(), nxt, config=cfg, transport="peer")
        work = lbc.iqrecv(recv, prv, config=cfg, transport="peer")
        sent.wait()
        got = work.wait()
        torch.cuda.synchronize()
        want = oracle.decode(oracle.encode(xs[prv], cfg), n, cfg, name)
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), ("mailbox", it, rank)
        assert work.execution_info.fast_path == "cuda_peer_mailbox_recv"
    comm.check_status()
    comm.peer_group.check_canaries()   # nobody, local or remote, wrote past the end of a region of this arena
    assert comm.stats["peer_ops"] > 0 and comm.stats["torch_ops"] == 0, comm.stats


def ddp_case(rank: int, world: int) -> None:
    import torch
    from torch.nn.parallel import DistributedDataParallel as DDP

    from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook
    from lowbit_comm_b200.models import GPT2, GPT2Config

    def run(with_hook: bool):
        torch.manual_seed(7)
        cfg = GPT2Config.tiny()
        model = GPT2(cfg).to(device="cuda", dtype=torch.bfloat16)
        ddp = DDP(model, device_ids=[torch.cuda.current_device()], gradient_as_bucket_view=True)
        hook = None
        if with_hook:
            hook = create_ddp_comm_hook(CompressionConfig(target="ddp_gradient_bucket"), strategy="auto")
            ddp.register_comm_hook(state=None, hook=hook)
        opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
        gen = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(8):
            tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=gen).cuda()
            loss = ddp(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            losses.append(loss.item())
        params = torch.cat([p.detach().float().reshape(-1) for p in ddp.parameters()])
        return losses, params, hook

    base_losses, base_params, _ = run(False)
    losses, params, hook = run(True)
    assert hook.gpu_launches() > 0
    hook.peer_engine.group.check_status()
    gathered = [torch.empty_like(params) for _ in range(world)]
    import torch.distributed as dist

    dist.all_gather(gathered, params)
    for other in gathered:
        assert torch.equal(other, params), "ranks diverged"
    drift = ((params - base_params).norm() / base_params.norm()).item()
    assert drift < 2e-2, drift
    assert abs(losses[-1] - base_losses[-1]) < 0.05 * abs(base_losses[-1]) + 0.05, (losses[-1], base_losses[-1])
    state = hook.state_dict()
    assert state["feedback"]["residuals"], "error-feedback residuals must be checkpointable"


def _exit_barrier(world: int, limit_s: float = 120.0) -> None:
    """No rank leaves (and unmaps its arena) before every rank has drained its GPU work: with a
    multicast arena a store that reaches an unmapped replica would fault the other GPUs."""

    import time

    import torch
    import torch.distributed as dist

    try:
        torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        pass
    try:
        store = dist.distributed_c10d._get_default_store()
        store.add("lbc_exit_barrier", 1)
        t0 = time.time()
        while int(store.add("lbc_exit_barrier", 0)) < world and time.time() - t0 < limit_s:
            time.sleep(0.05)
    except Exception:  # noqa: BLE001
        time.sleep(5.0)


def main() -> None:
    import torch
    import torch.distributed as dist

    case = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    try:
        {"collectives": collectives_case, "ddp": ddp_case}[case](rank, world)
        _exit_barrier(world)
        if rank == 0:
            from lowbit_comm_b200.parallel.communicator import get_communicator

            group = get_communicator(None).peer_group
            mc = bool(group is not None and group.multicast_ptr)
            print(f"MULTIRANK-OK {case} world={world} multicast={int(mc)}")
    except BaseException:
        traceback.print_exc()
        sys.stdout.flush()
        _exit_barrier(world)
        os._exit(1)
    finally:
        try:
            from lowbit_comm_b200.parallel.communicator import shutdown_communicators

            shutdown_communicators()
        except Exception:  # noqa: BLE001
            pass
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
