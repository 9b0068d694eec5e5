"""Compressed all-gather of tensors whose shapes differ across ranks.

Parity: ccdl_comm/collectives/dynamic_all_gather.py:12-82 (one-shot) and
ccdl_comm/cuda/dynamic_gather_executor.py:30-506 (compiled executor with a fixed
cross-rank shape class capacity, `object_v1` pickle metadata or `tensor_v1`
16 x int64 packets, `auto` = tensor_v1, LRU executor cache, zero-element bypass).
Payloads are padded to the capacity of the shape class, gathered with one
collective, trimmed and decoded.
"""

from __future__ import annotations

from collections import OrderedDict
from collections.abc import Callable
from dataclasses import dataclass
from importlib import import_module
from typing import Any, NamedTuple

from ...config import CompressionConfig
from ...core.executor import ObjectIdentity
from ...core.info import ExecutionCounters, ExecutionInfo
from ...ops import codec
from ...ops.oracle import TORCH_DTYPES
from ...ops.sizing import estimate_quantized_size
from ..metadata_packet import FLAG_EMPTY, PACKET_WORDS, MetadataPacket, decode_all

METADATA_PROTOCOLS = ("object_v1", "tensor_v1", "auto")


def _numel(shape) -> int:
    total = 1
    for d in shape:
        total *= int(d)
    return total


@dataclass(frozen=True)
class DynamicGatherMetadata:
    """What a rank announces before its fixed-size payload (protocol `object_v1` pickles `to_wire()`; `tensor_v1`
    sends the same facts as a 16 x int64 `MetadataPacket`).  Field names are the reference's
    (ccdl_comm/cuda/dynamic_gather_executor.py:36-52); `flags` is an addition (bit 0: empty tensor)."""

    protocol_version: int
    shape: tuple[int, ...]
    dtype: str
    payload_numel: int
    flags: int = 0

    def to_wire(self) -> dict[str, object]:
        return {"protocol_version": self.protocol_version, "shape": self.shape, "dtype": self.dtype,
                "payload_numel": self.payload_numel, "flags": self.flags}

    @classmethod
    def from_wire(cls, wire: dict) -> "DynamicGatherMetadata":
        version = int(wire.get("protocol_version", 1))
        if version != 1:
            raise ValueError(f"unsupported dynamic all-gather metadata version {version}")
        return cls(version, tuple(int(d) for d in wire["shape"]), str(wire["dtype"]), int(wire["payload_numel"]),
                   int(wire.get("flags", 0)))

    def packet(self) -> MetadataPacket:
        return MetadataPacket(self.shape, self.dtype, self.payload_numel, self.flags)


class DynamicGatherCacheKey(NamedTuple):
    """Everything that makes two dynamic all-gathers need different executors.  Objects (process group, injected
    codec functions, the extension status) take part by identity and are kept alive by the key, so an id can
    never be recycled into a stale hit."""

    shape_class: tuple[int, ...]
    dtype: str
    world_size: int | None
    config: CompressionConfig
    metadata_protocol: str
    process_group: ObjectIdentity
    distributed: ObjectIdentity
    extension_status: ObjectIdentity
    quantize: ObjectIdentity
    dequantize: ObjectIdentity


class _GatherSlots:
    """What an executor keeps on one device between runs: the send buffer, one receive buffer cut into a slot per
    rank, and the metadata words on both sides of the bus (pinned on the host for a CUDA device).  The capacity of
    the shape class is fixed, so nothing here is allocated again after the first run."""

    def __init__(self, torch, device, capacity_bytes: int, world: int) -> None:
        cuda = device.type == "cuda"
        self.send = torch.zeros(capacity_bytes, dtype=torch.uint8, device=device)
        self.recv = torch.empty(world * capacity_bytes, dtype=torch.uint8, device=device)
        self.slots = list(self.recv.view(world, capacity_bytes).unbind(0))
        self.words = torch.zeros(PACKET_WORDS, dtype=torch.int64, device=device)
        self.gathered = torch.empty(world * PACKET_WORDS, dtype=torch.int64, device=device)
        self.words_host = torch.zeros(PACKET_WORDS, dtype=torch.int64, pin_memory=cuda) if cuda else self.words
        self.gathered_host = (torch.empty(world * PACKET_WORDS, dtype=torch.int64, pin_memory=True) if cuda
                              else self.gathered)


class CudaDynamicGatherExecutor:
    def __init__(self, *, shape_class: tuple[int, ...], config: CompressionConfig, dtype: str, group: Any | None = None,
                 extension_status: Any | None = None, metadata_protocol: str = "object_v1",
                 import_module_fn: Callable[[str], Any] = import_module, quantize: Callable[..., Any] | None = None,
                 dequantize: Callable[..., Any] | None = None) -> None:
        if metadata_protocol not in METADATA_PROTOCOLS:
            raise ValueError(f"metadata_protocol must be one of {METADATA_PROTOCOLS}")
        if dtype not in TORCH_DTYPES:
            raise ValueError(f"unsupported dtype {dtype!r}")
        self.shape_class = tuple(int(d) for d in shape_class)
        self.config, self.dtype, self.group = config, dtype, group
        self._status = extension_status
        self.protocol = "tensor_v1" if metadata_protocol == "auto" else metadata_protocol
        self._importer = import_module_fn
        self._quantize = quantize or codec.quantize_tensor        # injectable, like the reference's transports
        self._dequantize = dequantize or codec.dequantize_tensor
        self.capacity_numel = _numel(self.shape_class)
        est = estimate_quantized_size(self.capacity_numel, dtype=dtype, config=config)
        self.capacity_bytes = est.quantized_bytes
        self.execution_info = ExecutionInfo(
            requested_strategy="dynamic_all_gather", executed_strategy="dynamic_all_gather", backend="cuda",
            fallback_used=False, fallback_reason=None, stage_names=("metadata", "payload"),
            original_bytes=est.original_bytes, compressed_bytes=max(est.quantized_bytes, 0),
            compression_ratio=est.compression_ratio or 1.0, workspace_cache_hit=False, async_capable=False,
            fast_path="cuda_dynamic_all_gather",
            details={"shape_class": self.shape_class, "metadata_protocol": self.protocol})
        self.execution_counters = ExecutionCounters()
        self.host_sync_count = 0
        self.slot_allocations = 0                       # times a `_GatherSlots` was built (once per device and world)
        self._slots: dict[tuple, _GatherSlots] = {}

    @property
    def metadata_protocol(self) -> str:
        return self.protocol

    @property
    def metadata_protocol_version(self) -> int:
        return 1

    def _kw(self) -> dict:
        return {} if self.group is None else {"group": self.group}

    def _slots_for(self, torch, device, world: int) -> _GatherSlots:
        key = (device.type, device.index, world)
        held = self._slots.get(key)
        if held is None:
            held = self._slots[key] = _GatherSlots(torch, device, max(self.capacity_bytes, 1), world)
            self.slot_allocations += 1
        return held

    def _gather_metadata(self, dist, torch, local: MetadataPacket, device, held: _GatherSlots) -> list[MetadataPacket]:
        world = dist.get_world_size(**self._kw())
        if self.protocol == "object_v1":
            objs: list[Any] = [None] * world
            mine = DynamicGatherMetadata(self.metadata_protocol_version, local.shape, local.dtype,
                                         local.payload_numel, local.flags)
            dist.all_gather_object(objs, mine.to_wire(), **self._kw())
            return [DynamicGatherMetadata.from_wire(o).packet() for o in objs]
        # the packet goes host (pinned) -> device -> all ranks -> host (pinned); the one wait below is the only
        # host synchronisation of a run (the shapes have to be known here to allocate the outputs)
        held.words_host.copy_(torch.tensor(local.encode(), dtype=torch.int64))
        if held.words_host is not held.words:
            held.words.copy_(held.words_host, non_blocking=True)
        dist.all_gather_into_tensor(held.gathered, held.words, **self._kw())
        if held.gathered_host is not held.gathered:
            held.gathered_host.copy_(held.gathered, non_blocking=True)
            torch.cuda.current_stream(device).synchronize()
        self.host_sync_count += 1
        return decode_all(held.gathered_host.tolist(), world)

    def run(self, tensor: Any) -> list[Any]:
        torch = self._importer("torch")
        dist = self._importer("torch.distributed")
        self.execution_counters._record_run()
        try:
            if codec.resolve_dtype("auto", tensor) != self.dtype:
                raise TypeError(f"executor was compiled for {self.dtype}")
            n = tensor.numel()
            if n > self.capacity_numel:
                raise ValueError(f"tensor has {n} elements, the shape class holds {self.capacity_numel}")
            device = tensor.device
            payload_bytes = estimate_quantized_size(n, dtype=self.dtype, config=self.config).quantized_bytes
            local = MetadataPacket(tuple(tensor.shape), self.dtype, payload_bytes, FLAG_EMPTY if n == 0 else 0)
            held = self._slots_for(torch, device, dist.get_world_size(**self._kw()))
            send, slots = held.send, held.slots          # bytes past a payload are never read: no clearing
            if n:  # zero-element tensors never reach a kernel
                self._quantize(tensor.contiguous(), self.config, extension_status=self._status,
                               output=send[:payload_bytes])
            metas = self._gather_metadata(dist, torch, local, device, held)
            dist.all_gather(slots, send, **self._kw())
            outs = []
            for meta, slot in zip(metas, slots):
                if meta.dtype != self.dtype:
                    raise TypeError("ranks disagree on the dtype of a dynamic all-gather")
                if meta.numel == 0:
                    outs.append(torch.empty(meta.shape, dtype=TORCH_DTYPES[self.dtype], device=device))
                    continue
                if meta.payload_numel > self.capacity_bytes:
                    raise ValueError("a rank's payload exceeds the compiled shape class")
                outs.append(self._dequantize(slot[:meta.payload_numel], meta.shape, self.config,
                                             dtype=self.dtype, extension_status=self._status))
            self.execution_counters._record_completed()
            return outs
        except BaseException:
            self.execution_counters._record_failed()
            raise


class DynamicGatherExecutorCache:
    """Bounded LRU of executors; keys are `DynamicGatherCacheKey`s (any hashable is accepted)."""

    def __init__(self, max_entries: int = 32) -> None:
        if isinstance(max_entries, bool) or not isinstance(max_entries, int) or max_entries <= 0:
            raise ValueError("max_entries must be a positive integer")
        self._max = max_entries
        self._items: "OrderedDict[Any, CudaDynamicGatherExecutor]" = OrderedDict()

    @property
    def max_entries(self) -> int:
        return self._max

    def get_or_create(self, key: tuple, factory: Callable[[], CudaDynamicGatherExecutor]):
        hit = self._items.get(key)
        if hit is not None:
            self._items.move_to_end(key)
            return hit
        made = factory()
        self._items[key] = made
        while len(self._items) > self._max:
            self._items.popitem(last=False)
        return made

    def __len__(self) -> int:
        return len(self._items)


_DEFAULT_CACHE = DynamicGatherExecutorCache()


def compile_dynamic_all_gather(*, shape_class, config: CompressionConfig, dtype: str, group: Any | None = None,
                               extension_status: Any | None = None, cache: DynamicGatherExecutorCache | None = None,
                               metadata_protocol: str = "object_v1", **kw) -> CudaDynamicGatherExecutor:
    key = DynamicGatherCacheKey(
        tuple(int(d) for d in shape_class), dtype, None, config, metadata_protocol, ObjectIdentity(group),
        ObjectIdentity(kw.get("import_module_fn")), ObjectIdentity(extension_status), ObjectIdentity(kw.get("quantize")),
        ObjectIdentity(kw.get("dequantize")))

    def build():
        return CudaDynamicGatherExecutor(shape_class=tuple(shape_class), config=config, dtype=dtype, group=group,
                                         extension_status=extension_status, metadata_protocol=metadata_protocol, **kw)

    return build() if cache is None else cache.get_or_create(key, build)


def compressed_all_gather_dynamic(tensor: Any, *, config: CompressionConfig, dtype: str = "auto",
                                  extension_status: Any | None = None, group: Any | None = None,
                                  compiled_executor: CudaDynamicGatherExecutor | None = None,
                                  metadata_protocol: str = "auto",
                                  import_module_fn: Callable[[str], Any] = import_module,
                                  quantize: Callable[..., Any] | None = None,
                                  dequantize: Callable[..., Any] | None = None) -> list[Any]:
    """One-shot form: agrees on the largest element count first, then gathers.

    `import_module_fn`, `quantize` and `dequantize` are injection points (a fake `torch.distributed`, a
    recording codec), as in ccdl_comm/communication/dynamic_all_gather.py; injected codecs bypass the
    executor cache.
    """

    if compiled_executor is not None:
        return compiled_executor.run(tensor)
    dist = import_module_fn("torch.distributed")
    torch = import_module_fn("torch")
    name = codec.resolve_dtype(dtype, tensor)
    kw = {} if group is None else {"group": group}
    biggest = torch.tensor([tensor.numel()], dtype=torch.int64, device=tensor.device)
    dist.all_reduce(biggest, op=dist.ReduceOp.MAX, **kw)
    capacity = max(int(biggest.item()), 1)
    injected = import_module_fn is not import_module or quantize is not None or dequantize is not None
    executor = compile_dynamic_all_gather(shape_class=(capacity,), config=config, dtype=name, group=group,
                                          extension_status=extension_status,
                                          cache=None if injected else _DEFAULT_CACHE,
                                          metadata_protocol=metadata_protocol, import_module_fn=import_module_fn,
                                          quantize=quantize, dequantize=dequantize)
    return executor.run(tensor)


qall_gather_dyn = compressed_all_gather_dynamic
