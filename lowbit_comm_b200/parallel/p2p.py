"""Quantized point-to-point: `qsend` / `qrecv` / `iqsend` / `iqrecv` and compiled endpoints.

Parity: ccdl_comm/communication/point_to_point.py:57-257 (one-shot functions)
and ccdl_comm/cuda/p2p_executor.py:25-299 (`CudaP2PExecutor`, `P2PMetadata`
protocol v1, per-run validation).  This is the primitive a pipeline-parallel
stage boundary uses.

Two transports:
* torch.distributed `isend`/`irecv` of the payload bytes (any device, any tag);
* peer mailboxes over NVLink (`PeerMailbox`): the sender's quantize kernel
  stores the payload straight into the receiver's mailbox and signals; the
  receiver's decode kernel waits (bounded), decodes and acknowledges, and the
  next send to the same peer first waits (bounded) for that acknowledgement.
  Messages between a pair are matched by order, so this path needs tag 0.
  Mailbox operations are kernels on the caller's current stream, in call order:
  a rank that both sends and receives in one step posts its sends first (a
  receive kernel waits on the device for the peer's send, and a send queued
  behind it on the same stream could not start), or uses two streams.  It is
  enabled per group with `Communicator.enable_peer_mailbox`, a collective call.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass
from importlib import import_module
from typing import Any

from ..config import CompressionConfig
from ..core.info import ExecutionCounters, ExecutionInfo
from ..core.work import CompletionWork, bind_execution_work
from ..exceptions import TorchDistributedUnavailableError, UnsupportedCollective
from ..ops import codec
from ..ops.sizing import estimate_quantized_size
from .peer_memory import PHASE_P2P_ACK, PHASE_P2P_DATA, PeerGroup

P2P_METADATA_PROTOCOL_VERSION = 1
PointToPointWork = CompletionWork


@dataclass(frozen=True)
class P2PMetadata:
    protocol_version: int
    shape: tuple[int, ...]
    dtype: str
    payload_numel: int


def _dist(importer: Callable[[str], Any]):
    try:
        dist = importer("torch.distributed")
    except (ImportError, ModuleNotFoundError) as exc:
        raise TorchDistributedUnavailableError("torch.distributed is not available") from exc
    if not dist.is_available() or not dist.is_initialized():
        raise TorchDistributedUnavailableError("torch.distributed is not initialized")
    return dist


def _kw(group, tag) -> dict:
    kw = {"tag": tag}
    if group is not None:
        kw["group"] = group
    return kw


class PeerMailbox:
    """Per-pair payload slots inside a peer arena, with data/ack epochs per pair."""

    def __init__(self, group: PeerGroup, *, capacity_bytes: int) -> None:
        self.group = group
        self.capacity = -(-capacity_bytes // 256) * 256
        self.offset = group.alloc(self.capacity * group.world_size)   # slot [source rank] on every rank
        self.channel = group.new_channel()
        # The kernels of a send (or a receive) count their blocks on a scratch counter before the last one
        # signals.  Sends to different peers may overlap on different streams, so every peer has its own
        # counters: a channel per peer, used for its counter words only (the flags stay on `self.channel`).
        self._counter_channels = [group.new_channel() for _ in range(group.world_size)]
        self._sent = [0] * group.world_size       # epochs count modulo 2^32, like the kernels' comparison
        self._received = [0] * group.world_size
        self._any_sent = [False] * group.world_size
        self.ext = group._ext

    def send(self, tensor, dst: int, config: CompressionConfig, dtype: str) -> None:
        g = self.group
        n = tensor.numel()
        groups = -(-n // config.group_size)
        need = estimate_quantized_size(n, dtype=dtype, config=config).quantized_bytes
        if need > self.capacity:
            raise ValueError(f"payload of {need} bytes exceeds the mailbox capacity {self.capacity}")
        previous = self._sent[dst]
        epoch = self._sent[dst] = (previous + 1) & 0xFFFFFFFF
        if self._any_sent[dst]:  # the receiver must have drained the previous message
            self.ext.wait_signal((g.flags_addr(g.rank, self.channel, PHASE_P2P_ACK) + 4 * dst, 1, previous,
                                  g.timeout_ns, g.status_device, PHASE_P2P_ACK), None)
        self._any_sent[dst] = True
        signal = ([g.flags_addr(dst, self.channel, PHASE_P2P_DATA)], g.rank, epoch,
                  g.counter_addr(self._counter_channels[dst], PHASE_P2P_DATA))
        self.ext.quant_push(tensor.reshape(-1), None, None, None, [g.addr(dst, self.offset + g.rank * self.capacity)],
                            self.ext.PUSH_BROADCAST, 0, groups, 0, config.group_size, config.bit, signal, 0)

    def recv(self, out, src: int, config: CompressionConfig, dtype: str) -> None:
        g = self.group
        n = out.numel()
        groups = -(-n // config.group_size)
        epoch = self._received[src] = (self._received[src] + 1) & 0xFFFFFFFF
        wait = (g.flags_addr(g.rank, self.channel, PHASE_P2P_DATA) + 4 * src, 1, epoch, g.timeout_ns,
                g.status_device, PHASE_P2P_DATA)
        ack = ([g.flags_addr(src, self.channel, PHASE_P2P_ACK)], g.rank, epoch,
               g.counter_addr(self._counter_channels[src], PHASE_P2P_ACK))
        self.ext.reduce([g.local_ptr + self.offset + src * self.capacity], groups, 0, False, n,
                        codec._DTYPE_CODE[dtype], config.group_size, config.bit, 1.0, out.reshape(-1), False, None, None,
                        [], 0, 0, ack, wait, 0)


class CudaP2PExecutor:
    """One compiled endpoint: direction, peer, group, tag, shape, dtype and config are frozen."""

    def __init__(self, *, direction: str, peer: int | None, tensor: Any, config: CompressionConfig,
                 group: Any | None = None, tag: int = 0, dtype: str = "auto", extension_status: Any | None = None,
                 import_module_fn: Callable[[str], Any] = import_module, quantize: Callable[..., Any] | None = None,
                 allocate_quantized: Callable[..., Any] | None = None, dequantize: Callable[..., Any] | None = None,
                 completion_manager: Any | None = None, mailbox: PeerMailbox | None = None) -> None:
        if direction not in ("send", "recv"):
            raise ValueError("direction must be 'send' or 'recv'")
        if direction == "send" and peer is None:
            raise ValueError("compiled send requires a destination peer")
        if peer is not None and (isinstance(peer, bool) or not isinstance(peer, int) or peer < 0):
            raise ValueError("peer must be a non-negative integer or None")
        if isinstance(tag, bool) or not isinstance(tag, int) or tag < 0:
            raise ValueError("tag must be a non-negative integer")
        if not isinstance(config, CompressionConfig):
            raise TypeError("config must be a CompressionConfig")
        if mailbox is not None and (tag != 0 or peer is None or not codec.is_fast_profile(config)):
            raise ValueError("the peer mailbox transport needs tag 0, an explicit peer and a linear/top-k 0 profile")
        self._direction, self._peer, self._group, self._tag, self._config = direction, peer, group, tag, config
        self._dtype = codec.resolve_dtype(dtype, tensor)
        self._shape = tuple(tensor.shape)
        self._device = str(getattr(tensor, "device", "cuda"))
        self._importer = import_module_fn
        self._status = extension_status
        self._quantize = quantize or codec.quantize_tensor
        self._allocate = allocate_quantized or codec.allocate_quantized_buffer
        self._dequantize = dequantize or codec.dequantize_tensor
        self._manager = completion_manager
        self._mailbox = mailbox
        n = 1
        for d in self._shape:
            n *= d
        est = estimate_quantized_size(n, dtype=self._dtype, config=config)
        self._metadata = P2PMetadata(P2P_METADATA_PROTOCOL_VERSION, self._shape, self._dtype, est.quantized_bytes)
        self.execution_info = ExecutionInfo(
            requested_strategy="compressed_p2p", executed_strategy="compressed_p2p", backend="cuda",
            fallback_used=False, fallback_reason=None, stage_names=(), original_bytes=est.original_bytes,
            compressed_bytes=est.quantized_bytes, compression_ratio=est.compression_ratio or 1.0,
            workspace_cache_hit=False, async_capable=True,
            fast_path=f"cuda_{'peer_mailbox' if mailbox is not None else 'compiled'}_{direction}",
            details={"direction": direction, "peer": peer, "tag": tag, "dtype": self._dtype, "shape": self._shape,
                     "metadata_protocol_version": P2P_METADATA_PROTOCOL_VERSION})
        self.execution_counters = ExecutionCounters()

    @property
    def metadata(self) -> P2PMetadata:
        return self._metadata

    # the frozen endpoint description, under the reference's attribute names
    direction = property(lambda self: self._direction)
    peer = property(lambda self: self._peer)
    group = property(lambda self: self._group)
    tag = property(lambda self: self._tag)
    config = property(lambda self: self._config)

    def _validate(self, tensor: Any) -> None:
        if tuple(tensor.shape) != self._shape:
            raise ValueError(f"tensor shape {tuple(tensor.shape)} does not match compiled shape {self._shape}")
        if codec.resolve_dtype("auto", tensor) != self._dtype:
            raise TypeError(f"tensor dtype {tensor.dtype} does not match compiled dtype {self._dtype}")
        if str(tensor.device) != self._device:
            raise ValueError(f"tensor device {tensor.device} does not match compiled device {self._device}")

    def run(self, tensor: Any):
        self.execution_counters._record_run()
        try:
            self._validate(tensor)
            work = self._send(tensor) if self._direction == "send" else self._recv(tensor)
        except BaseException:
            self.execution_counters._record_failed()
            raise
        return bind_execution_work(work, self.execution_info, self.execution_counters)

    def _send(self, tensor: Any) -> CompletionWork:
        if self._mailbox is not None:
            self._mailbox.send(tensor.contiguous(), self._peer, self._config, self._dtype)
            return CompletionWork(None, resources=(tensor,))
        dist = _dist(self._importer)
        payload = self._quantize(tensor, self._config, extension_status=self._status)
        if payload.numel() != self._metadata.payload_numel:
            raise ValueError("quantized payload size does not match the compiled metadata")
        handle = dist.isend(payload, self._peer, **_kw(self._group, self._tag))
        return CompletionWork(None, handle=handle, resources=(payload, tensor))

    def _recv(self, tensor: Any) -> CompletionWork:
        if self._mailbox is not None:
            self._mailbox.recv(tensor, self._peer, self._config, self._dtype)
            return CompletionWork(tensor, resources=(tensor,))
        dist = _dist(self._importer)
        payload = self._allocate(tensor, self._config, dtype=self._dtype)
        if payload.numel() != self._metadata.payload_numel:
            raise ValueError("receive payload size does not match the compiled metadata")
        handle = dist.irecv(payload, self._peer, **_kw(self._group, self._tag)) if self._peer is not None \
            else dist.irecv(payload, **_kw(self._group, self._tag))

        def complete() -> Any:
            self._dequantize(payload, self._shape, self._config, dtype=self._dtype, extension_status=self._status,
                             output=tensor)
            return tensor

        return CompletionWork(tensor, handle=handle, complete=complete, resources=(payload, tensor))


def compile_p2p_executor(*, direction: str, peer: int | None, tensor: Any, config: CompressionConfig,
                         **kwargs: Any) -> CudaP2PExecutor:
    """One immutable quantized point-to-point endpoint (ccdl_comm/cuda/p2p_executor.py:220-236)."""

    return CudaP2PExecutor(direction=direction, peer=peer, tensor=tensor, config=config, **kwargs)


def compile_qsend(tensor: Any, dst: int, *, config: CompressionConfig, **kw) -> CudaP2PExecutor:
    return CudaP2PExecutor(direction="send", peer=dst, tensor=tensor, config=config, **kw)


def compile_qrecv(tensor: Any, src: int | None = None, *, config: CompressionConfig, **kw) -> CudaP2PExecutor:
    return CudaP2PExecutor(direction="recv", peer=src, tensor=tensor, config=config, **kw)


def _mailbox_for(tensor: Any, peer: int | None, config: CompressionConfig, group: Any | None, tag: int,
                 dtype: str, transport: str) -> PeerMailbox | None:
    """The group's peer mailbox when this message can use it, else None ("peer" insists and raises)."""

    if transport not in ("auto", "peer", "torch"):
        raise ValueError("transport must be 'auto', 'peer' or 'torch'")
    if transport == "torch":
        return None
    reason = None
    mailbox = None
    if not bool(getattr(tensor, "is_cuda", False)):
        reason = "the tensor is not on a CUDA device"
    elif peer is None or tag != 0:
        reason = "the mailbox needs an explicit peer and tag 0"
    elif not codec.is_fast_profile(config):
        reason = "the mailbox serves linear / top-k 0 / deterministic profiles"
    else:
        from .communicator import _REGISTRY

        comm = _REGISTRY.get(id(group) if group is not None else 0)
        mailbox = None if comm is None or comm.closed else comm.mailbox
        if mailbox is None:
            reason = "Communicator.enable_peer_mailbox() was not called for this group"
        else:
            need = estimate_quantized_size(tensor.numel(), dtype=codec.resolve_dtype(dtype, tensor),
                                           config=config).quantized_bytes
            if need > mailbox.capacity:
                mailbox, reason = None, f"payload of {need} bytes exceeds the mailbox capacity"
    if mailbox is None and transport == "peer":
        raise UnsupportedCollective("p2p:peer", reason=reason or "peer mailbox unavailable")
    return mailbox


def iqsend(tensor: Any, dst: int, *, config: CompressionConfig, group: Any | None = None, tag: int = 0,
           dtype: str = "auto", extension_status: Any | None = None, compiled_executor: CudaP2PExecutor | None = None,
           transport: str = "auto", **kw):
    """Quantized send.  transport="auto" uses the group's peer mailbox when one was enabled and the message
    qualifies, else a torch.distributed send of the payload (the reference's only form,
    ccdl_comm/communication/point_to_point.py)."""

    if compiled_executor is None and "mailbox" not in kw:
        kw["mailbox"] = _mailbox_for(tensor, dst, config, group, tag, dtype, transport)
    executor = compiled_executor or compile_qsend(tensor, dst, config=config, group=group, tag=tag, dtype=dtype,
                                                  extension_status=extension_status, **kw)
    return executor.run(tensor)


def iqrecv(tensor: Any, src: int | None = None, *, config: CompressionConfig, group: Any | None = None, tag: int = 0,
           dtype: str = "auto", extension_status: Any | None = None, compiled_executor: CudaP2PExecutor | None = None,
           transport: str = "auto", **kw):
    if compiled_executor is None and "mailbox" not in kw:
        kw["mailbox"] = _mailbox_for(tensor, src, config, group, tag, dtype, transport)
    executor = compiled_executor or compile_qrecv(tensor, src, config=config, group=group, tag=tag, dtype=dtype,
                                                  extension_status=extension_status, **kw)
    return executor.run(tensor)


def qsend(tensor: Any, dst: int, *, config: CompressionConfig, **kw) -> None:
    iqsend(tensor, dst, config=config, **kw).wait()


def qrecv(tensor: Any, src: int | None = None, *, config: CompressionConfig, **kw) -> Any:
    return iqrecv(tensor, src, config=config, **kw).wait()
