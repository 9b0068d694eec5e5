"""Host-side logic of the peer-memory engine, exercised with fakes (no GPU, no process group):
arena sizing and growth in the DDP hook, the order of teardown, epoch arithmetic across the 32-bit wrap,
and the status check in front of every bucket."""

import pytest
import torch

from lowbit_comm_b200.config import CompressionConfig
from lowbit_comm_b200.exceptions import AsyncCommunicationError, CCDLUnavailableError
from lowbit_comm_b200.parallel import ddp_hook, peer_memory
from lowbit_comm_b200.parallel.fused import FusedWorkspace
from lowbit_comm_b200.parallel.peer_memory import PeerGroup


class FakeExt:
    """Records the calls `PeerGroup` makes into the native extension."""

    def __init__(self, log):
        self.log = log
        self.status = (0, 0, 0, 0, 0)

    def status_alloc(self):
        return 1, 2

    def status_read(self, host):
        return self.status

    def status_clear(self, host):
        self.status = (0, 0, 0, 0, 0)

    def status_free(self, host):
        self.log.append("status_free")

    def ipc_close_handle(self, ptr):
        self.log.append(f"ipc_close {ptr}")

    def arena_free(self, ptr):
        self.log.append(f"arena_free {ptr}")

    def memset_async(self, ptr, value, nbytes):
        pass


def _group(log, world=2, nbytes=1 << 30, **kw):
    return PeerGroup(rank=0, world_size=world, device=torch.device("cpu"), nbytes=nbytes,
                     peer_ptrs=[1000 * (r + 1) for r in range(world)], ext=FakeExt(log), owner=True,
                     process_group=object(), opened=[2000], **kw)


def test_close_synchronises_then_meets_the_peers_then_frees(monkeypatch):
    log = []
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: log.append("synchronize"))
    monkeypatch.setattr(torch.cuda, "device", lambda device: __import__("contextlib").nullcontext())
    group = _group(log, barrier=lambda: log.append("barrier"))
    group.close()
    assert log == ["synchronize", "barrier", "ipc_close 2000", "status_free", "arena_free 1000"]
    group.close()                                   # idempotent
    assert len(log) == 5


def test_close_of_a_single_rank_group_needs_no_barrier(monkeypatch):
    log = []
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: log.append("synchronize"))
    group = PeerGroup(rank=0, world_size=1, device=torch.device("cpu"), nbytes=1 << 20, peer_ptrs=[1000],
                      ext=FakeExt(log), owner=True, process_group=object(),
                      barrier=lambda: log.append("barrier"))
    group.close()
    assert "barrier" not in log and log[0] == "synchronize" and log[-1] == "arena_free 1000"


def test_store_barrier_counts_every_rank_and_is_bounded(monkeypatch):
    import torch.distributed as dist

    class Store:
        def __init__(self):
            self.values = {}

        def add(self, key, amount):
            self.values[key] = self.values.get(key, 0) + amount
            return self.values[key]

    store = Store()
    monkeypatch.setattr(dist.distributed_c10d, "_get_default_store", lambda: store)
    monkeypatch.setenv("LBC_CLOSE_TIMEOUT_S", "0.2")
    group = _group([], uid="abc")
    store.add("lbc_close_abc", 1)                   # the other rank already arrived
    group._store_barrier()
    assert store.values["lbc_close_abc"] == 2
    lonely = _group([], uid="xyz")                  # nobody else arrives: returns after the limit
    lonely._store_barrier()
    assert store.values["lbc_close_xyz"] == 1


def _reached(seen: int, epoch: int) -> bool:
    """The kernels' test `int(seen - epoch) >= 0` on 32-bit words."""

    return ((seen - epoch) & 0xFFFFFFFF) < 0x80000000


def test_epochs_wrap_through_the_whole_32_bit_range():
    group = _group([])
    ch = group.new_channel()
    group._epochs[ch] = 0xFFFFFFF0
    flag = 0xFFFFFFF0                               # the value the last collective left in the flag
    for _ in range(40):
        epoch = group.next_epoch(ch)
        assert 0 <= epoch <= 0xFFFFFFFF
        assert not _reached(flag, epoch), (flag, epoch)     # the stale flag never passes for the new epoch
        flag = epoch                                        # ... and the new signal does
        assert _reached(flag, epoch)
    assert group._epochs[ch] == 0x18                # walked across zero


def test_mailbox_epochs_wrap_and_every_peer_has_its_own_counter(monkeypatch):
    import contextlib

    from lowbit_comm_b200.parallel.p2p import PeerMailbox

    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())

    calls = []

    class Ext(FakeExt):
        PUSH_BROADCAST = 0

        def wait_signal(self, wait, signal):
            calls.append(("wait", wait[2]))

        def quant_push(self, *args):
            calls.append(("push", args[11]))

    group = _group([], world=4)
    group._ext = Ext([])
    box = PeerMailbox(group, capacity_bytes=4096)
    box._sent[1], box._any_sent[1] = 0xFFFFFFFF, True
    x = torch.zeros(64, dtype=torch.bfloat16)
    box.send(x, 1, CompressionConfig(), "bf16")
    box.send(x, 2, CompressionConfig(), "bf16")
    assert calls[0] == ("wait", 0xFFFFFFFF) and calls[1][1][2] == 0      # waits for the old ack, sends epoch 0
    assert calls[2][0] == "push" and calls[2][1][2] == 1                  # first message to rank 2: no wait
    counters = {calls[1][1][3], calls[2][1][3]}
    assert len(counters) == 2                                            # two destinations, two block counters


# ---------------------------------------------------------------------------------------------------
# arena sizing of the hook's engine
# ---------------------------------------------------------------------------------------------------
class FakeGroup:
    def __init__(self, total, world):
        self.nbytes, self.world_size, self.used, self.closed = total, world, 0, False

    @property
    def bytes_free(self):
        return self.nbytes - self.used

    def check_status(self):
        pass

    def close(self):
        self.closed = True


class FakeWorkspace:
    launches = 0

    def __init__(self, group, need, cap):
        if group.bytes_free < need:
            raise CCDLUnavailableError("peer arena exhausted")
        group.used += need
        self.group, self.max_numel = group, cap


def _engine(world, **kw):
    eng = ddp_hook._PeerEngine(config=CompressionConfig(), process_group=None, peer_group=kw.pop("peer_group", None),
                               arena_bytes=kw.pop("arena_bytes", None), max_bucket_numel=kw.pop("max_bucket_numel", None),
                               max_blocks=0, ef_mode="reference")
    made = []
    eng._world = lambda: world
    eng._make_group = lambda total, device: made.append(FakeGroup(total, world)) or made[-1]
    eng._make_workspace = lambda dtype, cap: FakeWorkspace(eng.group, eng._need(world, dtype, cap) - (1 << 20), cap)
    eng.stream = object()
    return eng, made


class Bucket:
    def __init__(self, numel):
        self._numel = numel
        self.device = torch.device("cpu")

    def numel(self):
        return self._numel


@pytest.mark.parametrize("world", (2, 4, 8))
def test_growing_bucket_sizes_never_exhaust_the_arena(world):
    """The first-iteration bucket sizes DDP produces for GPT-2 small with `find_unused_parameters=True`
    (tiny first, then growing), followed by the rebuilt 25 MB buckets."""

    eng, made = _engine(world)
    for numel in (2304, 14_200_000, 15_000_000, 38_600_000, 13_000_000, 2304, 38_600_000):
        ws = eng.ensure(Bucket(numel), "bf16")
        assert ws.max_numel >= numel
    assert eng.rebuilds >= 1 and all(g.closed for g in made[:-1]) and not made[-1].closed
    # no arena is a multiple of what the largest bucket needs
    need = FusedWorkspace.required_bytes(world, "bf16", CompressionConfig(), 1 << 26, False, engine="pipe")
    assert made[-1].nbytes <= 2 * need + (8 << 20)


def test_a_stated_maximum_sizes_the_arena_once():
    eng, made = _engine(4, max_bucket_numel=40_000_000)
    for numel in (2304, 14_200_000, 38_600_000):
        eng.ensure(Bucket(numel), "bf16")
    assert len(made) == 1 and eng.rebuilds == 0


def test_a_callers_arena_is_never_rebuilt():
    group = FakeGroup(64 << 20, 2)
    eng, made = _engine(2, peer_group=group)
    eng.ensure(Bucket(1 << 20), "bf16")
    with pytest.raises(CCDLUnavailableError):
        eng.ensure(Bucket(1 << 27), "bf16")
    assert not made and not group.closed


def test_the_hook_checks_the_status_word_before_every_bucket():
    """A wait that ran out in an earlier bucket must surface in the next hook call, and `reset_after_error`
    must restore service."""

    log = []
    group = _group(log)
    group._ext.status = (1, 9, 1, 0, 7)
    eng, _ = _engine(2, peer_group=group)
    with pytest.raises(AsyncCommunicationError) as info:
        eng.check_status()
    assert info.value.status["peer"] == 1 and "quantized rows" in str(info.value)
    holder = ddp_hook.DDPCommHook(lambda bucket: None, lambda: None)
    holder.peer_engine = eng
    with pytest.raises(AsyncCommunicationError):
        holder.check_status()
    group._ext.status_clear(0)
    holder.check_status()


def test_default_wait_limit_is_on_the_scale_of_a_watchdog():
    assert peer_memory.DEFAULT_TIMEOUT_NS >= 300 * 10**9


class _FakeGeneralExt:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def record(*a, **k):
            self.calls.append((name, a))

        return record


class _FakeGeneralGroup:
    """Symmetric bump allocation and address arithmetic of a peer group, nothing else."""

    world_size, rank, local_ptr = 4, 2, 0x20000

    def __init__(self):
        self._ext, self._top, self._epoch = _FakeGeneralExt(), 0, 0

    def alloc(self, nbytes):
        off, self._top = self._top, self._top + nbytes
        return off

    def new_channel(self):
        return 0

    def next_epoch(self, channel):
        self._epoch += 1
        return self._epoch

    def addr(self, rank, off):
        return 0x10000 * (rank + 1) + off       # rank 2's own arena is local_ptr

    def signal_all(self, channel, phase, epoch):
        return ("signal", epoch)

    def wait_all(self, channel, phase, epoch):
        return ("wait", epoch)

    def local_view(self, off, nbytes):
        return ("view", off, nbytes)


@pytest.mark.parametrize("fused", (True, False))
def test_general_profile_all_reduce_launch_plan(fused):
    """Top-k all-reduce over peer memory: the fused form is two launches whose destinations are slot [me] of every
    rank's receive region and whose sources are this rank's W slots; regions alternate with the epoch."""

    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.parallel.fused_general import GeneralPeerWorkspace

    cfg = CompressionConfig(topk=2, allow_experimental=True)
    group = _FakeGeneralGroup()
    ws = GeneralPeerWorkspace(group, dtype="bf16", config=cfg, max_numel=4096, fused=fused)
    x, res = torch.zeros(1000, dtype=torch.bfloat16), torch.zeros(1000, dtype=torch.bfloat16)
    ws.all_reduce(x, residual=res)
    names = [c[0] for c in group._ext.calls]
    if not fused:
        assert names == (["quant_general", "push_bytes", "wait_signal"] + ["dequant_general"] * 4
                         + ["scale_inplace", "error_feedback_update"]) and ws.launches == 9
        return
    assert names == ["quant_general_push", "reduce_general"] and ws.launches == 2
    push, reduce = group._ext.calls[0][1], group._ext.calls[1][1]
    region = ws.recv_off[1]                                     # first epoch is 1: the odd region
    assert push[3] == [0x10000 * (r + 1) + region + 2 * ws.slot_bytes for r in range(4)]
    assert reduce[0] == [group.local_ptr + region + r * ws.slot_bytes for r in range(4)]
    same = lambda t: t is not None and t.data_ptr() == res.data_ptr()      # noqa: E731
    assert reduce[7] == 0.25 and same(reduce[8]) and same(reduce[9]) and same(push[2]) and same(push[1])
    assert push[-2] == ("signal", 1) and reduce[-2] == ("wait", 1)
    group._ext.calls.clear()
    ws.all_reduce(x, op="sum", update_residual=False, residual=res)
    push, reduce = group._ext.calls[0][1], group._ext.calls[1][1]
    assert push[3][0] == 0x10000 + ws.recv_off[0] + 2 * ws.slot_bytes and push[2] is None and same(push[1])
    assert reduce[7] == 1.0 and reduce[8] is None and reduce[9] is None
    # two stages: scatter to the owners, reduce my shard, push it to everybody, gather-decode: four launches
    group._ext.calls.clear()
    before = ws.launches
    big = torch.zeros(4096, dtype=torch.bfloat16)
    ws.all_reduce(big, residual=torch.zeros(4096, dtype=torch.bfloat16), stages=2)
    names = [c[0] for c in group._ext.calls]
    assert names == ["quant_general_push", "reduce_general", "quant_general_push", "reduce_general"]
    assert ws.launches == before + 4
    scatter, shard_reduce, push, gather = (c[1] for c in group._ext.calls)
    shard_groups = GeneralPeerWorkspace.shard_numel(4, cfg, 4096) // 64
    assert shard_groups == 16 and scatter[-1] == shard_groups and push[-1] == 0
    assert shard_reduce[-2:] == (shard_groups, 0) and gather[-2:] == (0, shard_groups)
    assert shard_reduce[1].numel() == 16 * 64 and push[0].numel() == 16 * 64          # rank 2's shard is full
    assert push[3] == [0x10000 * (r + 1) + ws.gather_off[1] + 2 * (ws.gather_off[1] - ws.gather_off[0]) // 4
                       for r in range(4)]
    tiny = torch.zeros(100, dtype=torch.bfloat16)              # two groups: ranks 1..3 own nothing
    group._ext.calls.clear()
    ws.all_reduce(tiny, stages=2)
    assert [c[0] for c in group._ext.calls] == ["quant_general_push", "wait_signal", "quant_general_push", "reduce_general"]
    with pytest.raises(ValueError):
        GeneralPeerWorkspace(_FakeGeneralGroup(), dtype="bf16", config=cfg, max_numel=64, fused=False).all_reduce(tiny, stages=2)


def test_route_picks_engine_and_stage_count_from_size_and_world():
    """`FusedWorkspace.route`: "auto" is the single kernel except on two ranks and above its size limit; without a
    requested stage count the single kernel reduces in one stage up to 16 MiB / W, the kernel sequence up to its own
    crossover; a requested count is kept."""

    from types import SimpleNamespace

    from lowbit_comm_b200.parallel.fused import FusedWorkspace, default_stages

    def ws(world, engine="auto", pipe_mib=192):
        return SimpleNamespace(engine=engine, pipe_numel=pipe_mib << 19,
                               group=SimpleNamespace(world_size=world, multicast_ptr=0))

    route = FusedWorkspace.route
    mib = 1 << 19                                            # bf16 elements per MiB
    assert route(ws(8), 2 * mib, 2) == (True, 1) and route(ws(8), 4 * mib, 2) == (True, 2)
    assert route(ws(4), 4 * mib, 2) == (True, 1) and route(ws(4), 8 * mib, 2) == (True, 2)
    assert route(ws(8), 256 * mib, 2) == (False, default_stages(8, 256 << 20))       # above the single kernel's limit
    assert route(ws(2), 8 * mib, 2) == (False, default_stages(2, 8 << 20))            # two ranks: the kernel sequence
    assert route(ws(2, "pipe"), 8 * mib, 2) == (True, default_stages(2, 8 << 20))     # forced engine, its stage rule at W <= 2
    assert route(ws(8, "legacy"), 2 * mib, 2) == (False, default_stages(8, 2 << 20))
    assert route(ws(8), 2 * mib, 2, stages=2) == (True, 2) and route(ws(8, "legacy"), 64 * mib, 2, stages=1) == (False, 1)
    assert route(ws(1), 64 * mib, 2)[0] is True                                       # a one-GPU job takes the single kernel


def test_communicator_arena_grows_collectively_and_refuses_when_it_cannot(monkeypatch):
    """A workspace that does not fit: the communicator closes its arena (the safe close) and creates a larger one,
    drops the workspaces that lived in the old one, and counts the rebuild; a caller-fixed size or an enabled
    mailbox make it say why it cannot."""

    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.exceptions import CCDLUnavailableError
    from lowbit_comm_b200.parallel import communicator as mod
    from lowbit_comm_b200.parallel import fused, peer_memory

    made = []

    class Group:
        def __init__(self, nbytes):
            self.nbytes, self.bytes_free, self.closed, self.world_size, self.rank = nbytes, nbytes, False, 2, 0

        def check_status(self):
            assert not self.closed

        def close(self):
            self.closed = True

    class Workspace:
        @staticmethod
        def required_bytes(world_size, dtype, config, max_numel, with_gather_region, engine="both"):
            return 8 * max_numel                      # any fixed rule will do: the test is about growing, not sizing

        def __init__(self, group, *, dtype, config, max_numel, **kw):
            need = self.required_bytes(group.world_size, dtype, config, max_numel, True)
            assert group.bytes_free >= need
            group.bytes_free -= need
            self.group, self.max_numel = group, max_numel

    def create(pg, total, device):
        made.append(Group(total))
        return made[-1]

    fake_dist = type("D", (), {"group": type("G", (), {"WORLD": object()})(), "is_available": staticmethod(lambda: True),
                               "is_initialized": staticmethod(lambda: True), "get_rank": staticmethod(lambda *a: 0),
                               "get_world_size": staticmethod(lambda *a: 2)})
    monkeypatch.setattr(mod, "_dist", lambda: fake_dist)
    monkeypatch.setattr(peer_memory.PeerGroup, "create", staticmethod(create))
    monkeypatch.setattr(fused, "FusedWorkspace", Workspace)
    monkeypatch.setenv("LBC_ARENA_MIB", "8")
    cfg = CompressionConfig()

    class T:
        device = torch.device("cpu")

        def __init__(self, n):
            self._n = n

        def numel(self):
            return self._n

    comm = mod.Communicator(None)
    small = comm.workspace(T(100_000), cfg, "bf16")
    assert len(made) == 1 and small.group is made[0]
    big = comm.workspace(T(16_000_000), cfg, "bf16")          # does not fit beside the first one
    assert len(made) == 2 and made[0].closed and not made[1].closed and big.group is made[1]
    assert made[1].nbytes >= 2 * made[0].nbytes and comm.stats["arena_rebuilds"] == 1
    again = comm.workspace(T(100_000), cfg, "bf16")          # same key, now served by the larger workspace
    assert again is big and len(made) == 2
    fixed = mod.Communicator(None, arena_bytes=8 << 20)
    fixed.workspace(T(100_000), cfg, "bf16")
    with pytest.raises(CCDLUnavailableError, match="fixed by arena_bytes"):
        fixed.workspace(T(16_000_000), cfg, "bf16")
    boxed = mod.Communicator(None)
    boxed.workspace(T(100_000), cfg, "bf16")
    boxed.mailbox = object()
    with pytest.raises(CCDLUnavailableError, match="mailbox"):
        boxed.workspace(T(16_000_000), cfg, "bf16")
