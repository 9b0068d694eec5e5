"""Hop-by-hop compressed all-reduce over `torch.distributed` point-to-point operations: ring, tree, pairwise
exchange and recursive doubling.

Inside one NVSwitch domain the fused peer-memory kernels make every peer one hop away and these schedules are
not needed.  They are for the groups those kernels cannot serve: ranks on different nodes (NCCL over the
network), or processes without peer access (gloo on CPUs, which is also how they are tested).  Each executor is
compiled once for a tensor size and replays a rank-local schedule from `core.schedules`:

ring   W - 1 reduce-scatter steps -- quantize the outgoing chunk, exchange payloads with the neighbours,
       decode-and-add the incoming one -- then W - 1 gather steps that pass the finished chunks around.
tree   reduce towards the root along the binary tree (children's payloads are decoded and added, the partial
       sum is quantized and sent up), then the root's payload travels back down.
p2p    W - 1 rounds in which every rank sends its contribution to a chunk straight to the chunk's owner; the
       owners reduce; the finished payloads are exchanged in W - 1 more rounds.  One quantization per
       contribution, like the fused two-stage path.
butterfly  recursive doubling, power-of-two groups: log2(W) exchanges of the whole partial sum.

Role parity: the reference's pipelined ring and tree executors (ccdl_comm/cuda/transports/pipelined_ring.py:
166-282, tree.py:141-274, torch_topology.py:67-230).  Two deliberate differences.  A finished chunk is
quantized once, by its owner, and the *bytes* are forwarded in the gather / broadcast phase; every rank,
the owner included, decodes those same bytes, so all ranks end with bit-identical tensors (the reference
re-quantizes at every gather hop).  And sizes need not divide by the world size or the group size: the work
buffer is padded to W shards of whole groups.

Under NCCL `wait()` on a point-to-point request only orders streams, so a whole schedule is enqueued without
the host blocking; under gloo every step blocks, which is what a CPU run wants anyway.  Buffers belong to the
executor.  If a step raises, the buffers and the requests still in flight are moved to a quarantine list and
fresh buffers are allocated on the next run; `reap()` frees quarantined sets whose requests have completed,
without waiting for any.
"""

from __future__ import annotations

import threading
from collections.abc import Callable
from importlib import import_module
from typing import Any

from ..config import CompressionConfig
from ..core.chunking import ChunkPlan
from ..core.schedules import (compile_butterfly_schedule, compile_pairwise_schedule, compile_pipelined_ring_schedule,
                              compile_tree_schedule)
from ..exceptions import UnsupportedCollective

_REDUCTIONS = ("sum", "mean")


def _ceil_to(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class _Buffers:
    """Everything one run writes to: the padded work tensor and the payload buffers."""

    def __init__(self, torch: Any, numel: int, payload_bytes: int, count: int, dtype: Any, device: Any) -> None:
        self.work = torch.zeros(numel, dtype=dtype, device=device)
        self.payloads = [torch.empty(payload_bytes, dtype=torch.uint8, device=device) for _ in range(count)]


class _ScheduleExecutor:
    """What ring and tree share: group facts, codec binding, buffers, the busy flag and the quarantine."""

    method = "schedule"

    def __init__(self, *, numel: int, dtype: str, config: CompressionConfig, group: Any | None = None,
                 device: Any = "cpu", op: str = "mean", dist: Any | None = None, torch: Any | None = None,
                 quantize: Callable[..., Any] | None = None, dequantize: Callable[..., Any] | None = None) -> None:
        if op not in _REDUCTIONS:
            raise UnsupportedCollective(f"{self.method}:{op}", reason="only op='sum' and op='mean' are implemented")
        if numel <= 0:
            raise ValueError("numel must be positive")
        self._torch = torch or import_module("torch")
        self._dist = dist or import_module("torch.distributed")
        from ..ops import codec, oracle, sizing

        self.numel, self.dtype, self.config, self.group, self.op = int(numel), dtype, config, group, op
        self.device = self._torch.device(device)
        self.rank = int(self._dist.get_rank(group))
        self.world_size = int(self._dist.get_world_size(group))
        self._torch_dtype = oracle.TORCH_DTYPES[codec.resolve_dtype(dtype)]
        self._quantize = quantize or codec.quantize_tensor
        self._dequantize = dequantize or codec.dequantize_tensor
        self._payload_bytes = lambda n: sizing.estimate_quantized_size(n, dtype=dtype, config=config).quantized_bytes
        self._buffers: _Buffers | None = None
        self._busy = threading.Lock()
        self._quarantine: list[tuple[_Buffers, list[Any]]] = []
        self.runs = 0

    # -- group plumbing ---------------------------------------------------------------------------------
    def _global(self, group_rank: int) -> int:
        """P2P operations address peers by their rank in the default group."""

        if self.group is None:
            return group_rank
        return int(self._dist.get_global_rank(self.group, group_rank))

    def _exchange(self, send: Any | None, send_to: int | None, recv: Any | None, recv_from: int | None,
                  inflight: list[Any]) -> None:
        """One batch of at most one send and one receive; returns when both are ordered before what follows."""

        dist, ops = self._dist, []
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send, self._global(send_to), self.group))
        if recv is not None:
            ops.append(dist.P2POp(dist.irecv, recv, self._global(recv_from), self.group))
        if not ops:
            return
        requests = dist.batch_isend_irecv(ops)
        inflight.extend(requests)
        for request in requests:
            request.wait()
        del inflight[-len(requests):]

    # -- codec ------------------------------------------------------------------------------------------
    def _encode(self, values: Any, payload: Any) -> None:
        self._quantize(values, self.config, output=payload)

    def _decode(self, payload: Any, into: Any, *, add: bool) -> None:
        self._dequantize(payload, (into.numel(),), self.config, dtype=self.dtype, output=into,
                         reduce_op="sum" if add else "none")

    # -- buffers, failures ------------------------------------------------------------------------------
    def _make_buffers(self) -> _Buffers:
        raise NotImplementedError

    def _steps(self, buffers: _Buffers, inflight: list[Any]) -> None:
        raise NotImplementedError

    @property
    def quarantined(self) -> int:
        return len(self._quarantine)

    # the reference's names for the same two things (cuda/transports/pipelined_ring.py:166-204)
    @property
    def pending_submission_count(self) -> int:
        return len(self._quarantine)

    def reap_pending(self) -> int:
        return self.reap()

    def reap(self) -> int:
        """Frees quarantined buffer sets whose requests have all completed; never waits.  Returns how many
        sets are still held."""

        def done(request: Any) -> bool:
            probe = getattr(request, "is_completed", None)
            return bool(probe()) if callable(probe) else False

        self._quarantine = [(buffers, requests) for buffers, requests in self._quarantine
                            if not all(done(r) for r in requests)]
        return len(self._quarantine)

    def _guarded(self, tensor: Any, steps: Callable[[_Buffers, list[Any]], None],
                 collect: Callable[[_Buffers], Any]) -> Any:
        """Loads `tensor` into the work buffer, runs `steps` with the failure handling described in the module
        docstring, and returns `collect(buffers)`."""

        if tensor.numel() != self.numel:
            raise ValueError(f"this executor was compiled for {self.numel} elements, got {tensor.numel()}")
        if tensor.dtype != self._torch_dtype:
            raise TypeError(f"this executor was compiled for {self._torch_dtype}, got {tensor.dtype}")
        if not self._busy.acquire(blocking=False):
            raise RuntimeError(f"{type(self).__name__} is already running; executors are not re-entrant")
        inflight: list[Any] = []
        try:
            self.reap()
            buffers = self._buffers or self._make_buffers()
            self._buffers = buffers
            buffers.work[: self.numel].copy_(tensor.reshape(-1))
            buffers.work[self.numel:].zero_()
            try:
                steps(buffers, inflight)
            except BaseException:
                # whatever is still in flight may write into these buffers later: never reuse them
                self._quarantine.append((buffers, list(inflight)))
                self._buffers = None
                raise
            result = collect(buffers)
            self.runs += 1
            return result
        finally:
            self._busy.release()

    def run(self, tensor: Any, out: Any | None = None) -> Any:
        """All-reduce `tensor` (flattened); the result goes to `out`, or back into `tensor` when `out` is None."""

        def collect(buffers: _Buffers) -> Any:
            target = tensor if out is None else out
            target.reshape(-1).copy_(buffers.work[: self.numel])
            return target

        return self._guarded(tensor, self._steps, collect)

    def __call__(self, tensor: Any, out: Any | None = None) -> Any:
        return self.run(tensor, out)


class _ChunkedExecutor(_ScheduleExecutor):
    """Shapes whose first phase is a reduce-scatter (ring, pairwise): they can stop there and hand out the
    owner's exact reduced chunk as a `ReducedShard`."""

    chunk_plan: ChunkPlan

    def _reduce_scatter_phase(self, buffers: _Buffers, inflight: list[Any]) -> Any:
        """Runs the reduce-scatter; returns this rank's chunk of the work buffer, reduced and scaled."""

        raise NotImplementedError

    def _gather_phase(self, buffers: _Buffers, inflight: list[Any]) -> None:
        raise NotImplementedError

    def _steps(self, buffers: _Buffers, inflight: list[Any]) -> None:
        self._reduce_scatter_phase(buffers, inflight)
        self._gather_phase(buffers, inflight)

    def _chunk(self, buffers: _Buffers, owner: int) -> Any:
        lo, hi = self.chunk_plan.bounds(owner)
        return buffers.work[lo:hi]

    def _scale_mean(self, mine: Any) -> None:
        if self.op == "mean" and self.world_size > 1:
            mine.copy_((mine.float() * (1.0 / self.world_size)).to(mine.dtype))

    def run_reduce_scatter(self, tensor: Any, out: Any | None = None) -> Any:
        """Reduce-scatter only: a `ReducedShard` holding chunk `rank` of the reduced, padded tensor (not
        re-quantized).  `out`, when given, is a flat tensor of `shard_numel` elements that receives it."""

        from ..core.shard import ReducedShard

        shard_numel = self.chunk_plan.shard_numel
        if out is not None and (out.numel() != shard_numel or out.dtype != self._torch_dtype):
            raise ValueError(f"out must hold {shard_numel} elements of {self._torch_dtype}")

        def collect(buffers: _Buffers) -> Any:
            mine = self._chunk(buffers, self.rank)
            if out is None:
                shard = mine.clone()
            else:
                out.reshape(-1).copy_(mine)
                shard = out
            return ReducedShard(shard=shard, shard_index=self.rank, shard_numel=shard_numel,
                                original_shape=tuple(tensor.shape), original_numel=self.numel,
                                world_size=self.world_size, reduce=self.op, padded_numel=self.chunk_plan.padded_numel,
                                dtype=self.dtype, transport=f"schedule_{self.method}",
                                metadata={"fused": False, "caller_owned_output": out is not None,
                                          "group_aligned": True})

        return self._guarded(tensor, self._reduce_scatter_phase, collect)


class PipelinedRingExecutor(_ChunkedExecutor):
    """Ring reduce-scatter of W group-aligned shards followed by a ring all-gather of the owners' payloads."""

    method = "ring"

    def __init__(self, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        padded = _ceil_to(self.numel, self.config.group_size * self.world_size)
        self.chunk_plan = ChunkPlan.build(padded, self.world_size)
        self.schedule = compile_pipelined_ring_schedule(chunk_plan=self.chunk_plan, rank=self.rank)
        self.chunk_payload_bytes = self._payload_bytes(self.chunk_plan.shard_numel)

    def _make_buffers(self) -> _Buffers:
        # two payloads alternate as send and receive buffers; the gather phase needs one slot per owner so that
        # a payload that arrived can be forwarded while the next one is received
        return _Buffers(self._torch, self.chunk_plan.padded_numel, self.chunk_payload_bytes, 2 + self.world_size,
                        self._torch_dtype, self.device)

    def _reduce_scatter_phase(self, buffers: _Buffers, inflight: list[Any]) -> Any:
        outgoing, incoming = buffers.payloads[0], buffers.payloads[1]
        for step in self.schedule.steps:
            self._encode(self._chunk(buffers, step.send_chunk_owner), outgoing)
            self._exchange(outgoing, step.send_peer, incoming, step.recv_peer, inflight)
            self._decode(incoming, self._chunk(buffers, step.recv_chunk_owner), add=True)
        mine = self._chunk(buffers, self.rank)
        self._scale_mean(mine)
        return mine

    def _gather_phase(self, buffers: _Buffers, inflight: list[Any]) -> None:
        slots = buffers.payloads[2:]                      # slots[owner]: the finished payload of that owner's chunk
        mine = self._chunk(buffers, self.rank)
        self._encode(mine, slots[self.rank])
        self._decode(slots[self.rank], mine, add=False)  # the owner keeps what everybody else will decode
        for step in self.schedule.gather_steps:
            self._exchange(slots[step.send_chunk_owner], step.send_peer, slots[step.recv_chunk_owner], step.recv_peer,
                           inflight)
            self._decode(slots[step.recv_chunk_owner], self._chunk(buffers, step.recv_chunk_owner), add=False)


class TreeExecutor(_ScheduleExecutor):
    """Reduce to `root` along the heap-ordered binary tree, then send the root's payload back down."""

    method = "tree"

    def __init__(self, *, root: int = 0, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        self.padded_numel = _ceil_to(self.numel, self.config.group_size)
        self.schedule = compile_tree_schedule(chunk_plan=ChunkPlan.build(self.padded_numel, self.world_size),
                                              rank=self.rank, root=root)
        self.payload_bytes = self._payload_bytes(self.padded_numel)

    def _make_buffers(self) -> _Buffers:
        return _Buffers(self._torch, self.padded_numel, self.payload_bytes, 2, self._torch_dtype, self.device)

    def _steps(self, buffers: _Buffers, inflight: list[Any]) -> None:
        sched, (up, down) = self.schedule, buffers.payloads
        for child in sched.children:                      # subtrees first: each child's payload is its whole sum
            self._exchange(None, None, up, child, inflight)
            self._decode(up, buffers.work, add=True)
        if sched.parent is not None:
            self._encode(buffers.work, up)
            self._exchange(up, sched.parent, None, None, inflight)
            self._exchange(None, None, down, sched.parent, inflight)
        else:
            if self.op == "mean" and self.world_size > 1:
                buffers.work.copy_((buffers.work.float() * (1.0 / self.world_size)).to(buffers.work.dtype))
            self._encode(buffers.work, down)
        for child in sched.children:
            self._exchange(down, child, None, None, inflight)
        self._decode(down, buffers.work, add=False)      # the root decodes its own payload too


class PairwiseExecutor(_ChunkedExecutor):
    """Shifted pairwise exchange: every contribution goes straight to the owner of its chunk (one hop, one
    quantization), the owners reduce, and the finished payloads are exchanged the same way.  The dataflow of
    the fused two-stage all-reduce, over point-to-point operations."""

    method = "p2p"

    def __init__(self, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        padded = _ceil_to(self.numel, self.config.group_size * self.world_size)
        self.chunk_plan = ChunkPlan.build(padded, self.world_size)
        self.schedule = compile_pairwise_schedule(chunk_plan=self.chunk_plan, rank=self.rank)
        self.chunk_payload_bytes = self._payload_bytes(self.chunk_plan.shard_numel)

    def _make_buffers(self) -> _Buffers:
        return _Buffers(self._torch, self.chunk_plan.padded_numel, self.chunk_payload_bytes, 2 + self.world_size,
                        self._torch_dtype, self.device)

    def _reduce_scatter_phase(self, buffers: _Buffers, inflight: list[Any]) -> Any:
        outgoing, incoming = buffers.payloads[0], buffers.payloads[1]
        mine = self._chunk(buffers, self.rank)
        for step in self.schedule.steps:
            self._encode(self._chunk(buffers, step.send_peer), outgoing)
            self._exchange(outgoing, step.send_peer, incoming, step.recv_peer, inflight)
            self._decode(incoming, mine, add=True)
        self._scale_mean(mine)
        return mine

    def _gather_phase(self, buffers: _Buffers, inflight: list[Any]) -> None:
        slots = buffers.payloads[2:]
        mine = self._chunk(buffers, self.rank)
        self._encode(mine, slots[self.rank])
        self._decode(slots[self.rank], mine, add=False)
        for step in self.schedule.steps:                  # same pairs, the other way round: own chunk out, the sender's in
            self._exchange(slots[self.rank], step.send_peer, slots[step.recv_peer], step.recv_peer, inflight)
            self._decode(slots[step.recv_peer], self._chunk(buffers, step.recv_peer), add=False)


class ButterflyExecutor(_ScheduleExecutor):
    """Recursive doubling on a power-of-two group: log2(W) exchanges of the whole quantized partial sum.  Both
    partners add the same two decoded payloads (their own included), so they stay bit-identical round by round."""

    method = "butterfly"

    def __init__(self, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        self.padded_numel = _ceil_to(self.numel, self.config.group_size)
        try:
            self.schedule = compile_butterfly_schedule(world_size=self.world_size, rank=self.rank)
        except ValueError as exc:
            raise UnsupportedCollective(f"butterfly:W={self.world_size}", reason=str(exc)) from None
        self.payload_bytes = self._payload_bytes(self.padded_numel)

    def _make_buffers(self) -> _Buffers:
        return _Buffers(self._torch, self.padded_numel, self.payload_bytes, 2, self._torch_dtype, self.device)

    def _steps(self, buffers: _Buffers, inflight: list[Any]) -> None:
        outgoing, incoming = buffers.payloads
        for peer in self.schedule.peers:
            self._encode(buffers.work, outgoing)
            self._exchange(outgoing, peer, incoming, peer, inflight)
            self._decode(outgoing, buffers.work, add=False)
            self._decode(incoming, buffers.work, add=True)
        if self.op == "mean" and self.world_size > 1:
            buffers.work.copy_((buffers.work.float() * (1.0 / self.world_size)).to(buffers.work.dtype))


# the reference's topology names for these shapes: its "tree" method is the recursive doubling, its compiled
# tree executor the rooted binary tree; both are offered, under "butterfly" and "tree"
_EXECUTORS = {"ring": PipelinedRingExecutor, "tree": TreeExecutor, "p2p": PairwiseExecutor,
              "butterfly": ButterflyExecutor}


def compile_schedule_all_reduce(method: str, **kwargs: Any) -> _ScheduleExecutor:
    """`method` "ring", "tree", "p2p" or "butterfly"; keyword arguments as for the executor classes."""

    try:
        return _EXECUTORS[method](**kwargs)
    except KeyError:
        raise UnsupportedCollective(f"schedule:{method}", reason=f"hop-by-hop schedules exist for {sorted(_EXECUTORS)}") from None


def make_schedule_all_reduce(*, method: str = "ring", group: Any | None = None, root: int = 0) -> Callable[..., Any]:
    """A transport with the calling convention of the other factories
    (`transport(tensor, *, config, op, async_op, dtype, extension_status=None)`), which compiles one executor
    per (numel, dtype, config, op) it meets and reuses it.  The result replaces `tensor`'s contents and is
    returned; with `async_op` it comes wrapped in a finished work object (the steps are already enqueued)."""

    if method not in _EXECUTORS:
        raise UnsupportedCollective(f"schedule:{method}", reason=f"hop-by-hop schedules exist for {sorted(_EXECUTORS)}")
    compiled: dict[tuple, _ScheduleExecutor] = {}

    def transport(tensor: Any, *, config: CompressionConfig, op: str = "mean", async_op: bool = False,
                  dtype: str = "auto", extension_status: Any | None = None) -> Any:
        from ..core.work import ImmediateWork
        from ..ops import codec

        name = codec.resolve_dtype(dtype, tensor)
        key = (tensor.numel(), name, config, op, str(tensor.device))
        executor = compiled.get(key)
        if executor is None:
            extra = {"root": root} if method == "tree" else {}
            executor = compiled[key] = _EXECUTORS[method](numel=tensor.numel(), dtype=name, config=config, group=group,
                                                         device=tensor.device, op=op, **extra)
        result = executor.run(tensor)
        return ImmediateWork(result) if async_op else result

    transport.executors = compiled
    return transport


def make_schedule_reduce_scatter_shard(*, method: str = "p2p", group: Any | None = None) -> Callable[..., Any]:
    """Like `make_schedule_all_reduce`, but the transport stops after the reduce-scatter and returns a
    `ReducedShard` (`transport(tensor, *, config, op, async_op, dtype, extension_status=None, out=None)`).
    `method` is "ring" or "p2p", the two shapes that reduce-scatter first."""

    cls = _EXECUTORS.get(method)
    if cls is None or not issubclass(cls, _ChunkedExecutor):
        raise UnsupportedCollective(f"schedule:{method}", reason="a reduced shard needs a 'ring' or 'p2p' schedule")
    compiled: dict[tuple, _ChunkedExecutor] = {}

    def transport(tensor: Any, *, config: CompressionConfig, op: str = "mean", async_op: bool = False,
                  dtype: str = "auto", extension_status: Any | None = None, out: Any | None = None) -> Any:
        from ..core.work import ImmediateWork
        from ..ops import codec

        name = codec.resolve_dtype(dtype, tensor)
        key = (tensor.numel(), name, config, op, str(tensor.device))
        executor = compiled.get(key)
        if executor is None:
            executor = compiled[key] = cls(numel=tensor.numel(), dtype=name, config=config, group=group,
                                           device=tensor.device, op=op)
        shard = executor.run_reduce_scatter(tensor, out=out)
        return ImmediateWork(shard) if async_op else shard

    transport.executors = compiled
    return transport
