"""Stream-safe workspace pool, leases and the caller-visible output lease.

Parity: ccdl_comm/cuda/workspace.py:18-648 (keyed LRU pool; a released buffer
becomes reusable only once its completion event reports ready, or is handed to
a new stream by making that stream wait on the event; `record_stream` on every
hand-out; hit/miss/eviction/byte statistics; byte and entry budgets; output
lease state machine ACQUIRED -> SUBMITTING -> BOUND -> RELEASED with an owner
token) and ccdl_comm/communication/workspace.py:35-196 (the two small legacy
caches).  The pool is backend neutral: allocator, stream and completion objects
are injected, so its logic is tested on CPU with fakes.

Peer-visible regions are *not* pooled here: they are carved once out of the
symmetric arena (`parallel/peer_memory.py`) and reused under the epoch rules
documented in `parallel/fused.py`.
"""

from __future__ import annotations

import threading
from collections import OrderedDict
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, NamedTuple

_DTYPE_BYTES = {"fp16": 2, "bf16": 2, "fp32": 4, "uint8": 1, "int8": 1}
WORKSPACE_KINDS = ("send", "recv", "reduced", "reduced_output")


@dataclass(frozen=True)
class WorkspaceKey:
    backend: str
    collective: str
    strategy: str
    shape_class: tuple[int, ...]
    dtype: str
    world_size: int
    bit: int
    group_size: int
    chunk_config: tuple[int, ...]
    workspace_kind: str
    device: str = "cuda"

    def __post_init__(self) -> None:
        for name in ("backend", "collective", "strategy", "workspace_kind"):
            if not getattr(self, name):
                raise ValueError(f"{name} must not be empty")
        if any(d < 0 for d in self.shape_class):
            raise ValueError("shape_class dimensions must be >= 0")
        for name in ("world_size", "bit", "group_size"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")

    @property
    def estimated_bytes(self) -> int:
        total = _DTYPE_BYTES.get(self.dtype, 4)
        for d in self.shape_class:
            total *= d
        return total


class WorkspaceStats(NamedTuple):
    hits: int
    misses: int
    evictions: int
    cached_bytes: int
    in_flight_bytes: int


class _Entry:
    __slots__ = ("ident", "key", "buffer", "nbytes", "completion")

    def __init__(self, ident: int, key: WorkspaceKey, buffer: Any, nbytes: int) -> None:
        self.ident, self.key, self.buffer, self.nbytes = ident, key, buffer, nbytes
        self.completion: Any = None


def _nbytes(buffer: Any, fallback: int) -> int:
    try:
        return int(buffer.numel()) * int(buffer.element_size())
    except Exception:  # noqa: BLE001
        return fallback


def _ready(completion: Any) -> bool:
    return completion is None or bool(completion.query())


class WorkspaceLease:
    """Exclusive use of one pooled buffer until `release(completion=...)`."""

    def __init__(self, pool: "CudaWorkspacePool", entry: _Entry) -> None:
        self._pool, self._entry = pool, entry
        self._released = False
        self._guard = threading.Lock()

    @property
    def buffer(self) -> Any:
        return self._entry.buffer

    @property
    def key(self) -> WorkspaceKey:
        return self._entry.key

    @property
    def size_bytes(self) -> int:
        return self._entry.nbytes

    @property
    def released(self) -> bool:
        with self._guard:
            return self._released

    def release(self, *, completion: Any) -> None:
        with self._guard:
            if self._released:
                raise RuntimeError("workspace lease is already released")
            self._released = True
            try:
                self._pool._give_back(self._entry, completion)
            except BaseException:
                self._released = False
                raise


class CudaWorkspacePool:
    def __init__(self, *, allocator: Callable[[WorkspaceKey, Any], Any], max_cached_bytes: int | None = None,
                 max_entries: int | None = None) -> None:
        if not callable(allocator):
            raise TypeError(f"the pool needs a function that allocates a workspace, got {type(allocator).__name__}")
        if max_cached_bytes is not None and max_cached_bytes < 0:
            raise ValueError(f"a byte budget cannot be negative (max_cached_bytes={max_cached_bytes}); None means unlimited")
        if max_entries is not None and max_entries < 1:
            raise ValueError(f"an entry budget below one caches nothing (max_entries={max_entries}); None means unlimited")
        self._alloc = allocator
        self._byte_budget, self._entry_budget = max_cached_bytes, max_entries
        self._idle: "OrderedDict[int, _Entry]" = OrderedDict()      # ready for anyone, LRU order
        self._pending: "OrderedDict[int, _Entry]" = OrderedDict()   # released, completion not ready yet
        self._busy: dict[int, _Entry] = {}
        self._next = 0
        self._hits = self._misses = self._evictions = 0
        self._lock = threading.Lock()

    # -- public -------------------------------------------------------------
    def acquire(self, key: WorkspaceKey, stream: Any) -> WorkspaceLease:
        if not isinstance(key, WorkspaceKey):
            raise TypeError("key must be a WorkspaceKey")
        with self._lock:
            self._promote_ready()
            entry = self._pop_matching(self._idle, key)
            if entry is None:
                entry = self._pop_matching(self._pending, key)
                if entry is not None:
                    # not finished yet: order the new user's stream after the previous use
                    waiter = getattr(entry.completion, "wait_stream", None)
                    if callable(waiter):
                        waiter(stream)
                    entry.completion = None
            if entry is None:
                buffer = self._alloc(key, stream)
                entry = _Entry(self._next, key, buffer, _nbytes(buffer, key.estimated_bytes))
                self._next += 1
                self._misses += 1
            else:
                self._hits += 1
            recorder = getattr(entry.buffer, "record_stream", None)
            if callable(recorder) and stream is not None:
                try:
                    recorder(stream)
                except (RuntimeError, TypeError):
                    pass
            self._busy[entry.ident] = entry
            return WorkspaceLease(self, entry)

    @property
    def stats(self) -> WorkspaceStats:
        with self._lock:
            self._promote_ready()
            cached = sum(e.nbytes for e in self._idle.values()) + sum(e.nbytes for e in self._pending.values())
            return WorkspaceStats(self._hits, self._misses, self._evictions, cached,
                                  sum(e.nbytes for e in self._busy.values()))

    def clear(self) -> None:
        with self._lock:
            self._promote_ready()
            self._idle.clear()

    # -- internals ------------------------------------------------------------
    def _give_back(self, entry: _Entry, completion: Any) -> None:
        if completion is not None and not callable(getattr(completion, "query", None)):
            raise TypeError("completion must provide query()")
        with self._lock:
            if self._busy.pop(entry.ident, None) is None:
                raise RuntimeError("workspace does not belong to this pool or is not in flight")
            entry.completion = completion
            (self._idle if _ready(completion) else self._pending)[entry.ident] = entry
            if _ready(completion):
                entry.completion = None
            self._enforce_budgets()

    def _promote_ready(self) -> None:
        for ident in [i for i, e in self._pending.items() if _ready(e.completion)]:
            entry = self._pending.pop(ident)
            entry.completion = None
            self._idle[ident] = entry
        self._enforce_budgets()

    @staticmethod
    def _pop_matching(table: "OrderedDict[int, _Entry]", key: WorkspaceKey) -> _Entry | None:
        for ident in reversed(table):  # most recently released first: warm in cache
            if table[ident].key == key:
                return table.pop(ident)
        return None

    def _enforce_budgets(self) -> None:
        def over() -> bool:
            count = len(self._idle) + len(self._pending)
            size = sum(e.nbytes for e in self._idle.values()) + sum(e.nbytes for e in self._pending.values())
            return (self._entry_budget is not None and count > self._entry_budget) or \
                   (self._byte_budget is not None and size > self._byte_budget)

        while self._idle and over():   # only finished buffers may be dropped
            self._idle.popitem(last=False)
            self._evictions += 1


class LeaseState(Enum):
    ACQUIRED = "ACQUIRED"
    SUBMITTING = "SUBMITTING"
    BOUND = "BOUND"
    RELEASED = "RELEASED"


def _completion_for(manager: Any, value: Any, stream: Any = None) -> Any:
    if callable(getattr(value, "query", None)) and not hasattr(value, "shape"):
        return value
    record = getattr(manager, "record_for", None)
    if not callable(record):
        raise TypeError("completion_manager must provide record_for()")
    completion = record(value) if stream is None else record(value, stream=stream)
    if not callable(getattr(completion, "query", None)):
        raise TypeError("completion_manager.record_for() must return completion with query()")
    return completion


def _work_done(work: Any) -> bool:
    for name in ("query", "is_completed"):
        probe = getattr(work, name, None)
        if callable(probe):
            return bool(probe())
    return False


class CudaOutputLease:
    """Caller-visible ownership of one pooled reduced-shard output buffer."""

    def __init__(self, lease: WorkspaceLease, *, owner_token: object, completion_manager: Any,
                 acquisition_stream: Any) -> None:
        if not isinstance(lease, WorkspaceLease):
            raise TypeError("lease must be a WorkspaceLease")
        if owner_token is None:
            raise TypeError("owner_token must not be None")
        if completion_manager is None:
            raise TypeError("completion_manager must not be None")
        self._lease, self._owner, self._manager = lease, owner_token, completion_manager
        self._stream = acquisition_stream
        self._state = LeaseState.ACQUIRED
        self._work: Any = None
        self._lock = threading.Lock()

    @property
    def buffer(self) -> Any:
        return self._lease.buffer

    tensor = buffer

    @property
    def state(self) -> str:
        return self._state.value

    def _check(self, owner_token: object, *, allowed: LeaseState, message: str) -> None:
        if self._state is LeaseState.RELEASED:
            raise RuntimeError("CUDA output lease is already released")
        if owner_token is not self._owner:
            raise RuntimeError("CUDA output lease belongs to a different executor")
        if self._state is not allowed:
            raise RuntimeError(message)

    def mark_used(self, owner_token: object) -> Any:
        with self._lock:
            self._check(owner_token, allowed=LeaseState.ACQUIRED, message="CUDA output lease is already in use")
            self._state = LeaseState.SUBMITTING
            return self._lease.buffer

    mark_submitting = mark_used

    def bind_work(self, owner_token: object, work: Any) -> None:
        with self._lock:
            self._check(owner_token, allowed=LeaseState.SUBMITTING,
                        message="CUDA output lease must be submitting before binding work")
            self._work, self._state = work, LeaseState.BOUND

    def abort_use(self, owner_token: object) -> None:
        with self._lock:
            self._check(owner_token, allowed=LeaseState.SUBMITTING,
                        message="CUDA output lease can abort only while submitting")
            self._state = LeaseState.ACQUIRED

    def release_after(self, value_or_completion: Any) -> None:
        with self._lock:
            if self._state is LeaseState.RELEASED:
                raise RuntimeError("CUDA output lease is already released")
            if self._state is LeaseState.ACQUIRED:
                raise RuntimeError("CUDA output lease must be marked used before release_after")
            if self._state is LeaseState.SUBMITTING or self._work is None:
                raise RuntimeError("CUDA output lease must be bound to work before release_after")
            if not _work_done(self._work):
                raise RuntimeError("CUDA output lease cannot release until associated work completes")
            self._finish(_completion_for(self._manager, value_or_completion))

    def release_unused(self) -> None:
        with self._lock:
            if self._state is LeaseState.RELEASED:
                raise RuntimeError("CUDA output lease is already released")
            if self._state is not LeaseState.ACQUIRED:
                raise RuntimeError("CUDA output lease cannot release_unused after mark_used")
            self._finish(_completion_for(self._manager, self._lease.buffer, self._stream))

    def _finish(self, completion: Any) -> None:
        before = self._state
        self._state = LeaseState.RELEASED
        try:
            self._lease.release(completion=completion)
            self._work = None
        except BaseException:
            self._state = before
            raise


class DequantizedWorkspaceCache:
    """Per-hook cache of restored (dequantized) buffers, default one entry (legacy parity)."""

    def __init__(self, *, allocator: Callable[[Any, tuple[int, ...], Any], Any], max_entries: int | None = 1,
                 max_cached_bytes: int | None = None) -> None:
        self._alloc, self._max_entries, self._max_bytes = allocator, max_entries, max_cached_bytes
        self._items: "OrderedDict[Any, Any]" = OrderedDict()
        self.hits = self.misses = 0

    def get(self, key: Any, like: Any, shape: tuple[int, ...], config: Any) -> Any:
        held = self._items.get(key)
        if held is not None and tuple(held.shape) == tuple(shape) and held.dtype == like.dtype \
                and held.device == like.device:
            self._items.move_to_end(key)
            self.hits += 1
            return held
        self.misses += 1
        buf = self._alloc(like, tuple(shape), config)
        size = _nbytes(buf, 0)
        if self._max_entries == 0 or (self._max_bytes is not None and size > self._max_bytes):
            return buf
        self._items[key] = buf
        self._items.move_to_end(key)
        while (self._max_entries is not None and len(self._items) > self._max_entries) or \
                (self._max_bytes is not None and sum(_nbytes(b, 0) for b in self._items.values()) > self._max_bytes):
            self._items.popitem(last=False)
        return buf

    def clear(self) -> None:
        self._items.clear()


def _held_bytes(buffer: Any) -> int:
    """Bytes a cached buffer keeps alive (0 for objects that do not say)."""

    nbytes = getattr(buffer, "nbytes", None)
    if nbytes is not None:
        return int(nbytes)
    numel, width = getattr(buffer, "numel", None), getattr(buffer, "element_size", None)
    return int(numel()) * int(width()) if callable(numel) and callable(width) else 0


class ShardCommunicationWorkspaceCache:
    """send / recv / reduced buffers of the torch.distributed reduce-scatter path, by bucket key.

    An LRU with two optional limits, entries and bytes (ccdl_comm/communication/workspace.py:83-200): whatever
    was used least recently is dropped until both hold again, so a buffer larger than the byte budget is
    handed out but not kept.  The two allocators can be replaced (a pool, a recording fake)."""

    def __init__(self, *, quantized_allocator: Callable[[Any, Any, str], Any] | None = None,
                 reduced_allocator: Callable[[Any, tuple[int, ...], Any], Any] | None = None,
                 max_entries: int | None = None, max_cached_bytes: int | None = None) -> None:
        if max_entries is not None and max_entries < 1:
            raise ValueError("max_entries must be >= 1 or None")
        if max_cached_bytes is not None and max_cached_bytes < 0:
            raise ValueError("max_cached_bytes must be >= 0 or None")
        self._allocate_quantized = quantized_allocator
        self._allocate_reduced = reduced_allocator
        self._max_entries, self._max_bytes = max_entries, max_cached_bytes
        self._items: "OrderedDict[tuple, Any]" = OrderedDict()
        self._bytes = 0

    @property
    def cached_bytes(self) -> int:
        return self._bytes

    def __len__(self) -> int:
        return len(self._items)

    def _over_budget(self) -> bool:
        return (self._max_entries is not None and len(self._items) > self._max_entries) or \
            (self._max_bytes is not None and self._bytes > self._max_bytes)

    def get(self, key: Any, kind: str, index: int, factory: Callable[[], Any]) -> Any:
        if kind not in ("send", "recv", "reduced"):
            raise ValueError(f"unknown workspace kind {kind!r}")
        full = (key, kind, index)
        held = self._items.get(full)
        if held is not None:
            self._items.move_to_end(full)
            return held
        held = factory()
        self._items[full] = held
        self._bytes += _held_bytes(held)
        while self._items and self._over_budget():
            _, dropped = self._items.popitem(last=False)
            self._bytes -= _held_bytes(dropped)
        return held

    def clear(self, key: Any | None = None) -> None:
        doomed = [f for f in self._items if key is None or f[0][0] == key or f[0] == key]
        for full in doomed:
            self._bytes -= _held_bytes(self._items.pop(full))

    # The reference's three accessors (ccdl_comm/communication/workspace.py:105-170): one cached buffer per
    # (bucket, role, index, world size, tensor signature); a changed signature allocates a new one.
    @staticmethod
    def _signature(tensor: Any) -> tuple:
        return (str(getattr(tensor, "device", "")), str(getattr(tensor, "dtype", "")),
                tuple(getattr(tensor, "shape", ())))

    def get_quantized_chunk(self, bucket_key: Any, chunk_index: int, tensor: Any, config: Any, *, dtype: str,
                            world_size: int) -> Any:
        """uint8 payload buffer for chunk `chunk_index` of `tensor` (the send side of the all-to-all)."""

        def allocate() -> Any:
            if self._allocate_quantized is not None:
                return self._allocate_quantized(tensor, config, dtype)
            from ..ops.codec import allocate_quantized_buffer

            return allocate_quantized_buffer(tensor, config, dtype=dtype)

        key = (bucket_key, world_size, self._signature(tensor), dtype, config)
        return self.get(key, "send", chunk_index, allocate)

    def get_received_payload(self, bucket_key: Any, payload_template: Any, index: int, *, world_size: int,
                             config: Any) -> Any:
        """A buffer shaped like `payload_template` for the payload arriving from rank `index`."""

        key = (bucket_key, world_size, self._signature(payload_template), config)
        return self.get(key, "recv", index, lambda: payload_template.new_empty(payload_template.shape))

    def get_reduced_shard(self, bucket_key: Any, tensor: Any, shape: tuple[int, ...], config: Any, *, dtype: str,
                          world_size: int, rank: int) -> Any:
        """The reduced shard of this rank, in the source dtype."""

        key = (bucket_key, world_size, self._signature(tensor), tuple(shape), dtype, config)
        if self._allocate_reduced is not None:
            return self.get(key, "reduced", rank, lambda: self._allocate_reduced(tensor, tuple(shape), config))
        return self.get(key, "reduced", rank, lambda: tensor.new_empty(tuple(shape)))


class CudaShardWorkspaceProvider:
    """Binds the send / recv / reduced buffers of one reduced-shard executor to a `CudaWorkspacePool`.

    `begin(stream=...)` opens a session for one collective call; every buffer the session hands out is an
    exclusive lease of the pool, and `session.release(completion=...)` gives all of them back at once behind
    the call's completion event.  Parity: ccdl_comm/cuda/workspace.py:418-581.  The fused peer path does not
    need it (its buffers live in the peer arena); the torch.distributed path and external callers do.
    """

    def __init__(self, pool: CudaWorkspacePool, *, backend: str, collective: str, strategy: str, device: str,
                 pool_reduced_output: bool = True) -> None:
        if not isinstance(pool, CudaWorkspacePool):
            raise TypeError("pool must be a CudaWorkspacePool")
        self.pool = pool
        self.backend, self.collective, self.strategy, self.device = backend, collective, strategy, device
        self.pool_reduced_output = bool(pool_reduced_output)

    def begin(self, *, stream: Any) -> "CudaShardWorkspaceSession":
        return CudaShardWorkspaceSession(self, stream=stream)


class CudaShardWorkspaceSession:
    """Exclusive leases of one shard collective call; same accessor names as `ShardCommunicationWorkspaceCache`."""

    def __init__(self, provider: CudaShardWorkspaceProvider, *, stream: Any) -> None:
        self._provider, self._stream = provider, stream
        self._leases: list[WorkspaceLease] = []

    @property
    def leases(self) -> tuple[WorkspaceLease, ...]:
        return tuple(self._leases)

    def _take(self, *, shape: tuple[int, ...], dtype: str, world_size: int, config: Any, chunk_config: tuple[int, ...],
              kind: str) -> Any:
        p = self._provider
        key = WorkspaceKey(backend=p.backend, collective=p.collective, strategy=p.strategy, shape_class=tuple(shape),
                           dtype=dtype, world_size=world_size, bit=config.bit, group_size=config.group_size,
                           chunk_config=tuple(chunk_config), workspace_kind=kind, device=p.device)
        lease = p.pool.acquire(key, self._stream)
        self._leases.append(lease)
        return lease.buffer

    @staticmethod
    def _payload_bytes(tensor: Any, dtype: str, config: Any) -> int:
        from ..ops.sizing import estimate_quantized_size

        return estimate_quantized_size(int(tensor.numel()), dtype=dtype, config=config).quantized_bytes

    def get_quantized_chunk(self, bucket_key: Any, chunk_index: int, tensor: Any, config: Any, *, dtype: str,
                            world_size: int) -> Any:
        return self._take(shape=(self._payload_bytes(tensor, dtype, config),), dtype="uint8", world_size=world_size,
                          config=config, chunk_config=(chunk_index, int(tensor.numel())), kind="send")

    def get_received_payload(self, bucket_key: Any, payload_template: Any, index: int, *, world_size: int,
                             config: Any) -> Any:
        name = {"torch.uint8": "uint8"}.get(str(payload_template.dtype), str(payload_template.dtype))
        return self._take(shape=tuple(payload_template.shape), dtype=name, world_size=world_size, config=config,
                          chunk_config=(index,), kind="recv")

    def get_received_tensor_payload(self, bucket_key: Any, index: int, tensor: Any, config: Any, *, dtype: str,
                                    world_size: int) -> Any:
        """Receive storage sized from the source chunk's metadata (no payload template needed)."""

        return self._take(shape=(self._payload_bytes(tensor, dtype, config),), dtype="uint8", world_size=world_size,
                          config=config, chunk_config=(index, int(tensor.numel())), kind="recv")

    def get_reduced_shard(self, bucket_key: Any, tensor: Any, shape: tuple[int, ...], config: Any, *, dtype: str,
                          world_size: int, rank: int) -> Any:
        """The reduced shard, padded to whole groups; None when the provider leaves the output to the caller."""

        if not self._provider.pool_reduced_output:
            return None
        numel = 1
        for d in shape:
            numel *= int(d)
        padded = -(-numel // config.group_size) * config.group_size
        return self._take(shape=(padded,), dtype=dtype, world_size=world_size, config=config, chunk_config=(rank,),
                          kind="reduced")

    def release(self, *, completion: Any) -> None:
        while self._leases:
            self._leases.pop(0).release(completion=completion)


def _allocate_torch_buffer(key: WorkspaceKey, stream: Any) -> Any:
    import torch

    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32, "uint8": torch.uint8,
             "int64": torch.int64}.get(key.dtype, torch.uint8)
    return torch.empty(key.shape_class, dtype=dtype, device=key.device)


def create_torch_workspace_pool(*, max_cached_bytes: int | None = None,
                                max_entries: int | None = None) -> CudaWorkspacePool:
    """A pool whose misses allocate torch tensors lazily (ccdl_comm/cuda/workspace.py:444-455)."""

    return CudaWorkspacePool(allocator=_allocate_torch_buffer, max_cached_bytes=max_cached_bytes,
                             max_entries=max_entries)
