"""Symmetric peer-visible arenas, flag pads and status words.

Every rank of a single-node group allocates one device arena, exports it with
a CUDA IPC handle and maps the arenas of all other ranks.  Offsets inside the
arena mean the same thing on every rank (symmetric allocation), so a kernel can
address "my slot in rank d's receive region" as `peer_base[d] + offset`.

Arena layout:
  [0, 64 KiB)      flags[channel][phase][source rank]  (uint32 epochs, written by peers)
  [64, 68 KiB)     block counters[channel][phase]      (local scratch of the signalling kernels)
  [128 KiB, ...)   data regions handed out by `alloc`

Two ways to obtain the arenas.  The default is `cudaMalloc` + CUDA IPC.  With
`multicast=True` (or LBC_MULTICAST=1) the arena comes from torch's symmetric
memory allocator, which additionally binds the arenas of all ranks to one
NVLink multicast object: a `multimem.st` through `multicast_ptr + offset`
writes the same bytes at `offset` of every rank's arena (the NVSwitch
replicates them), so a broadcast leaves the sending GPU once instead of W - 1
times.  torch only does the allocation and the handle exchange; every kernel
that touches the memory is this library's.

The reference has no counterpart (its payloads travel through torch.distributed
calls, ccdl_comm/communication/torch_transport.py:61-188).
"""

from __future__ import annotations

import os
import threading
from typing import Any

import torch

from ..exceptions import AsyncCommunicationError, CCDLError, CCDLUnavailableError, DeviceWaitStatus
from ..ops.loader import require_extension

MAX_CHANNELS = 256
NUM_PHASES = 4
MAX_RANKS = 16
FLAG_BYTES = MAX_CHANNELS * NUM_PHASES * MAX_RANKS * 4
COUNTER_OFFSET = FLAG_BYTES
DATA_OFFSET = 128 * 1024
CANARY_BYTES, CANARY_VALUE = 256, 0xA5
# How long a kernel waits for a peer's flag before it gives up and reports through the status word: the
# scale of a collective library's watchdog (minutes), because a rank may legitimately be late by a whole
# evaluation pass or a checkpoint write.  Tests pass short limits explicitly.
DEFAULT_TIMEOUT_NS = 600_000_000_000
CLOSE_BARRIER_LIMIT_S = 60.0

PHASE_REDUCE_SCATTER, PHASE_ALL_GATHER, PHASE_P2P_DATA, PHASE_P2P_ACK = range(NUM_PHASES)


def _round_up(value: int, align: int) -> int:
    return -(-value // align) * align


class PeerGroup:
    """One rank's handle on the group's arenas."""

    def __init__(self, *, rank: int, world_size: int, device: torch.device, nbytes: int, peer_ptrs: list[int],
                 ext: Any, owner: bool, process_group: Any = None, opened: list[int] | None = None,
                 timeout_ns: int = DEFAULT_TIMEOUT_NS, multicast_ptr: int = 0, keepalive: Any = None,
                 uid: str = "", barrier: Any = None) -> None:
        if world_size > MAX_RANKS:
            raise CCDLUnavailableError(f"peer groups support at most {MAX_RANKS} ranks")
        self.rank = rank
        self.world_size = world_size
        self.device = device
        self.nbytes = nbytes
        self.peer_ptrs = list(peer_ptrs)
        self.local_ptr = self.peer_ptrs[rank]
        self.multicast_ptr = int(multicast_ptr)   # 0: no multicast mapping, broadcasts use W unicast stores
        self._keepalive = keepalive               # symmetric-memory tensor + handle backing the arena
        self.process_group = process_group
        self.timeout_ns = timeout_ns
        self._ext = ext
        self._owner = owner
        self._opened = list(opened or [])
        self._cursor = DATA_OFFSET
        self._canaries: list[int] = []
        self._epochs = [0] * MAX_CHANNELS
        self._channels_used = 0
        self._lock = threading.Lock()
        self._closed = False
        self._uid = uid                           # the same string on every rank of the group: names its store keys
        self._barrier = barrier                   # host-side barrier of the group used by close(); None = store counter
        host, dev = ext.status_alloc()
        self.status_host, self.status_device = host, dev

    # -- construction -------------------------------------------------------
    @classmethod
    def create(cls, process_group: Any, nbytes: int, device: torch.device | None = None, *,
               timeout_ns: int = DEFAULT_TIMEOUT_NS, multicast: bool | None = None) -> "PeerGroup":
        """Collective: every rank of `process_group` (one node) calls this.

        `multicast=None` reads LBC_MULTICAST (default off); when the multicast
        arena cannot be set up on every rank, all ranks fall back to CUDA IPC.
        """

        import torch.distributed as dist

        ext = require_extension()
        device = device or torch.device("cuda", torch.cuda.current_device())
        rank = dist.get_rank(process_group)
        world = dist.get_world_size(process_group)
        nbytes = _round_up(max(nbytes, DATA_OFFSET + 4096), 2 << 20)
        if timeout_ns == DEFAULT_TIMEOUT_NS and os.environ.get("LBC_WAIT_TIMEOUT_MS"):
            timeout_ns = max(1, int(os.environ["LBC_WAIT_TIMEOUT_MS"])) * 1_000_000
        if multicast is None:
            multicast = os.environ.get("LBC_MULTICAST", "0").lower() in ("1", "true", "on", "yes")
        if multicast and world > 1:
            made = cls._create_symmetric(process_group, nbytes, device, ext, rank, world, timeout_ns)
            if made is not None:
                return made
        with torch.cuda.device(device):
            local = ext.arena_alloc(nbytes)
            handle = ext.ipc_get_handle(local) if world > 1 else b""
            infos: list[Any] = [None] * world
            dist.all_gather_object(infos, (device.index, handle, os.urandom(8).hex()), group=process_group)
            ptrs, opened = [], []
            for peer, (peer_dev, peer_handle, _) in enumerate(infos):
                if peer == rank:
                    ptrs.append(local)
                    continue
                if not ext.can_access_peer(device.index, peer_dev):
                    ext.arena_free(local)
                    raise CCDLUnavailableError(f"GPU {device.index} cannot access GPU {peer_dev} as a peer")
                mapped = ext.ipc_open_handle(peer_handle)
                ptrs.append(mapped)
                opened.append(mapped)
            torch.cuda.synchronize(device)
        dist.barrier(group=process_group)
        return cls(rank=rank, world_size=world, device=device, nbytes=nbytes, peer_ptrs=ptrs, ext=ext, owner=True,
                   process_group=process_group, opened=opened, timeout_ns=timeout_ns, uid=infos[0][2])

    @classmethod
    def _create_symmetric(cls, process_group: Any, nbytes: int, device: torch.device, ext: Any, rank: int,
                          world: int, timeout_ns: int) -> "PeerGroup | None":
        """Arena from torch's symmetric-memory allocator, with the NVLink multicast mapping.

        Returns None (on every rank alike) when any rank could not get a
        multicast pointer; the caller then uses the IPC arena.
        """

        import torch.distributed as dist

        tensor = handle = None
        error = ""
        try:
            import torch.distributed._symmetric_memory as symm_mem

            pg = process_group if process_group is not None else dist.group.WORLD
            with torch.cuda.device(device):
                tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
                handle = symm_mem.rendezvous(tensor, pg)
                tensor.zero_()
                torch.cuda.synchronize(device)
            ok = int(handle.multicast_ptr) != 0 and len(handle.buffer_ptrs) == world
            if not ok:
                error = "no multicast pointer"
        except Exception as exc:  # noqa: BLE001 - any failure means "use the IPC arena"
            ok = False
            error = f"{type(exc).__name__}: {exc}"
        votes: list[Any] = [None] * world
        dist.all_gather_object(votes, (bool(ok), os.urandom(8).hex()), group=process_group)
        uid = votes[0][1]
        if not all(v[0] for v in votes):
            if rank == 0 and os.environ.get("LBC_DEBUG"):
                print(f"[lowbit_comm_b200] multicast arena unavailable ({error or 'a peer failed'}); using CUDA IPC")
            del tensor, handle
            return None
        dist.barrier(group=process_group)
        return cls(rank=rank, world_size=world, device=device, nbytes=nbytes,
                   peer_ptrs=[int(p) for p in handle.buffer_ptrs], ext=ext, owner=False,
                   process_group=process_group, opened=[], timeout_ns=timeout_ns,
                   multicast_ptr=int(handle.multicast_ptr), keepalive=(tensor, handle), uid=uid)

    @classmethod
    def loopback(cls, world_size: int, nbytes: int, device: torch.device | None = None, *,
                 timeout_ns: int = DEFAULT_TIMEOUT_NS) -> list["PeerGroup"]:
        """`world_size` emulated ranks whose arenas all live on one GPU.

        For single-GPU tests and benchmarks: the phases of a collective are run
        one after the other for all emulated ranks on one stream, so every flag
        is already set when a waiting kernel starts.
        """

        ext = require_extension()
        device = device or torch.device("cuda", torch.cuda.current_device())
        nbytes = _round_up(max(nbytes, DATA_OFFSET + 4096), 2 << 20)
        with torch.cuda.device(device):
            ptrs = [ext.arena_alloc(nbytes) for _ in range(world_size)]
        return [cls(rank=r, world_size=world_size, device=device, nbytes=nbytes, peer_ptrs=ptrs, ext=ext,
                    owner=True, timeout_ns=timeout_ns, opened=[]) for r in range(world_size)]

    # -- symmetric allocation ----------------------------------------------
    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserve `nbytes`; returns the offset (identical on every rank).

        Every region is followed by a 256-byte canary (0xA5) in this rank's own arena; `check_canaries`
        finds any kernel, local or remote, that wrote past the end of a region.
        """

        with self._lock:
            start = _round_up(self._cursor, align)
            end = _round_up(start + nbytes, 256)
            if end + CANARY_BYTES > self.nbytes:
                raise CCDLUnavailableError(
                    f"peer arena exhausted: need {nbytes} bytes at {start}, arena has {self.nbytes}")
            self._cursor = end + CANARY_BYTES
            self._canaries.append(end)
            with torch.cuda.device(self.device):
                self._ext.memset_async(self.local_ptr + end, CANARY_VALUE, CANARY_BYTES)
            return start

    def check_canaries(self) -> None:
        """Raises when a canary behind one of this rank's regions was overwritten (synchronises the device)."""

        torch.cuda.synchronize(self.device)
        for offset in self._canaries:
            view = self.local_view(offset, CANARY_BYTES)
            if not bool((view == CANARY_VALUE).all().item()):
                raise CCDLError(f"rank {self.rank}: the canary at arena offset {offset} was overwritten")

    def new_channel(self) -> int:
        with self._lock:
            if self._channels_used >= MAX_CHANNELS:
                raise CCDLUnavailableError("no free signal channel")
            self._channels_used += 1
            return self._channels_used - 1

    @property
    def bytes_free(self) -> int:
        return self.nbytes - self._cursor

    # -- addresses ----------------------------------------------------------
    def addr(self, rank: int, offset: int) -> int:
        return self.peer_ptrs[rank] + offset

    def multicast_addr(self, offset: int) -> int:
        """Multicast alias of `offset` in every rank's arena (0 when there is no multicast mapping)."""

        return self.multicast_ptr + offset if self.multicast_ptr else 0

    def flags_addr(self, rank: int, channel: int, phase: int) -> int:
        return self.peer_ptrs[rank] + ((channel * NUM_PHASES + phase) * MAX_RANKS) * 4

    def counter_addr(self, channel: int, phase: int) -> int:
        return self.local_ptr + COUNTER_OFFSET + (channel * NUM_PHASES + phase) * 4

    def local_view(self, offset: int, nbytes: int) -> torch.Tensor:
        """uint8 tensor aliasing a region of this rank's own arena."""

        return self._ext.tensor_from_address(self.local_ptr + offset, nbytes, self.device.index)

    # -- signalling helpers ---------------------------------------------------
    def next_epoch(self, channel: int) -> int:
        """Epochs count modulo 2^32, 0 included: the kernels compare `int(seen - epoch) >= 0`, which stays
        right across the wrap as long as a flag is never more than 2^31 collectives behind."""

        if getattr(self, "_closed", False):
            # every collective of every workspace starts here: one that outlived its arena (a communicator closed
            # or grew it) must not launch kernels on freed memory
            raise CCDLUnavailableError("this workspace's peer arena was closed; ask the communicator for a workspace again")
        self._epochs[channel] = (self._epochs[channel] + 1) & 0xFFFFFFFF
        return self._epochs[channel]

    def signal_all(self, channel: int, phase: int, epoch: int, ranks=None):
        """Signal tuple: write `epoch` into slot `rank` of the flag pad of every listed rank."""

        ranks = range(self.world_size) if ranks is None else ranks
        return ([self.flags_addr(r, channel, phase) for r in ranks], self.rank, epoch,
                self.counter_addr(channel, phase))

    def wait_all(self, channel: int, phase: int, epoch: int, count: int | None = None, first: int = 0):
        """Wait tuple: local flags [first, first+count) of (channel, phase) must reach `epoch`."""

        count = self.world_size if count is None else count
        return (self.flags_addr(self.rank, channel, phase) + 4 * first, count, epoch, self.timeout_ns,
                self.status_device, phase)

    # -- status ---------------------------------------------------------------
    def read_status(self) -> dict:
        return DeviceWaitStatus(*self._ext.status_read(self.status_host))._asdict()

    def check_status(self) -> None:
        """Raises when a kernel of this group gave up waiting.  Reads pinned host memory: no device
        synchronisation, cheap enough to call before every collective."""

        if getattr(self, "_closed", False):
            return                                   # the status word went with the arena
        status = DeviceWaitStatus(*self._ext.status_read(self.status_host))
        if status.timed_out:
            raise AsyncCommunicationError.from_wait(self.rank, status)

    def clear_status(self) -> None:
        self._ext.status_clear(self.status_host)

    def reset_after_error(self) -> None:
        """Zero this rank's counters after a failed collective (flags keep their epochs)."""

        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            self._ext.memset_async(self.local_ptr + COUNTER_OFFSET, 0, DATA_OFFSET - COUNTER_OFFSET)
            torch.cuda.synchronize(self.device)
        self.clear_status()

    # -- teardown ---------------------------------------------------------------
    def _store_barrier(self) -> None:
        """Every rank of the group adds one to a counter in the job's key-value store and waits (bounded)
        until the counter shows all of them.  Host only: no kernel, no collective on a GPU."""

        import time

        import torch.distributed as dist

        limit = float(os.environ.get("LBC_CLOSE_TIMEOUT_S", CLOSE_BARRIER_LIMIT_S))
        try:
            store = dist.distributed_c10d._get_default_store()
            key = f"lbc_close_{self._uid or id(self.process_group)}"
            store.add(key, 1)
            deadline = time.monotonic() + limit
            while int(store.add(key, 0)) < self.world_size and time.monotonic() < deadline:
                time.sleep(0.01)
        except Exception:  # noqa: BLE001 - no store (torn-down job): give the peers a moment instead
            time.sleep(min(limit, 2.0))

    def close(self, *, free_arena: bool = True) -> None:
        """Collective over the group.  A peer's kernel may still be loading from this rank's arena (the
        gather stage reads the owners' memory) or storing into it after this rank's own stream has drained,
        so the arena is unmapped and freed only after every rank has drained its device AND said so on the
        host: synchronize, barrier, then free."""

        if self._closed:
            return
        self._closed = True
        try:
            torch.cuda.synchronize(self.device)
        except Exception:  # noqa: BLE001
            pass
        if self.process_group is not None and self.world_size > 1:
            try:
                (self._barrier or self._store_barrier)()
            except Exception:  # noqa: BLE001
                pass
        for ptr in self._opened:
            try:
                self._ext.ipc_close_handle(ptr)
            except Exception:  # noqa: BLE001
                pass
        self._ext.status_free(self.status_host)
        if self._owner and free_arena and self.process_group is not None:
            self._ext.arena_free(self.local_ptr)
        self._keepalive = None                    # dropping the symmetric-memory tensor unmaps it

    @staticmethod
    def close_loopback(groups: list["PeerGroup"], *, check: bool = True) -> None:
        """Frees the emulated ranks' arenas; with `check` it first verifies every canary."""

        if not groups:
            return
        torch.cuda.synchronize(groups[0].device)
        problem = None
        if check:
            for g in groups:
                try:
                    g.check_canaries()
                except CCDLError as exc:
                    problem = problem or exc
        for g in groups:
            g._closed = True
            g._ext.status_free(g.status_host)
        for ptr in groups[0].peer_ptrs:
            groups[0]._ext.arena_free(ptr)
        if problem is not None:
            raise problem
