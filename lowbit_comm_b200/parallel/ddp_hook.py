"""PyTorch DDP communication-hook factory.

Parity: ccdl_comm/communication/ddp_hook.py:48-485 (`create_ddp_comm_hook`, the
same keyword parameters, strategies, small-bucket bypass, error-feedback state
and policies, `_ccdl_strategy_plan` / `_ccdl_effective_strategy`, DDP type
annotations), ccdl_comm/communication/ddp.py:33-97 (`DDPBucketProcessor`) and
async_pipeline.py:10-65 (`AsyncBucketPipeline`).

Two engines sit behind one hook:

* peer engine (CUDA tensors, sm_100a extension, ranks on one NVLink domain):
  the bucket is reduced by the fused kernels of `parallel/fused.py` on a side
  stream that first waits for the producer stream; the hook returns a CUDA
  aware Future immediately, with no host synchronisation anywhere.
* torch engine (CPU/gloo, injected codecs or transports, generic profiles):
  quantize -> torch.distributed collective -> dequantize-reduce, as the
  reference does.

Differences from the reference, on purpose: `strategy="all_reduce"` (its
default) there sums payload *bytes* with NCCL, which is not a valid reduction
for more than one rank; here it means "compressed all-reduce, best transport".
Error feedback is applied on every strategy, not only on `all_gather`.
"""

from __future__ import annotations

import os
from collections.abc import Callable
from importlib import import_module
from typing import Any

from ..config import CompressionConfig
from ..exceptions import CCDLUnavailableError
from ..ops import codec
from ..ops.error_feedback import ErrorFeedbackPolicy, ErrorFeedbackState
from ..ops.loader import CudaExtensionStatus, load_cuda_extension
from ..utils import tracing
from .completion import CudaCompletionManager
from .payload import (CompressedAllGatherReduce, CompressedAllReduce, CompressedPayload, GatheredPayloads,
                      coerce_payload, payload_buffer)
from .payload_packing import (DEFAULT_FUSED_PAYLOAD_MIN_NUMEL, make_fused_payload_all_gather,
                              make_payload_all_gather, should_fuse_payload)
from .strategy import CollectiveCapabilities, plan_ddp_compression_strategy
from .torch_transport import (make_torch_all_gather, make_torch_all_to_all,
                              make_torch_async_all_gather, make_torch_tensor_all_reduce)

_TOPOLOGY_METHODS = {None, "auto", "ring", "tree", "p2p", "overlap-gather", "overlap-p2p", "overlap-tree",
                     "overlap-scale"}


def _torch_future_factory() -> Any:
    return import_module("torch").futures.Future()


def _dist_fact(name: str, default: int) -> int:
    try:
        dist = import_module("torch.distributed")
        if not dist.is_available() or not dist.is_initialized():
            return default
        return int(getattr(dist, name)())
    except (ImportError, ModuleNotFoundError, RuntimeError, ValueError):
        return default


def _env_int(name: str) -> int | None:
    raw = os.environ.get(name, "")
    try:
        return int(raw) if raw else None
    except ValueError:
        return None


def _numel(tensor: Any) -> int:
    fn = getattr(tensor, "numel", None)
    if callable(fn):
        return int(fn())
    total = 1
    for dim in getattr(tensor, "shape", ()):
        total *= int(dim)
    return total


def _resolve_dtype(dtype: str, tensor: Any) -> str:
    if dtype != "auto":
        return dtype
    text = str(getattr(tensor, "dtype", ""))
    for needle, name in (("bfloat16", "bf16"), ("float16", "fp16"), ("half", "fp16"), ("float32", "fp32")):
        if needle in text:
            return name
    if text.endswith("float"):
        return "fp32"
    raise ValueError(f"cannot infer CCDL dtype from bucket tensor dtype: {text!r}")


def _bucket_key(bucket: Any) -> Any:
    index = getattr(bucket, "index", None)
    return index() if callable(index) else id(bucket)


def _clone(tensor: Any) -> Any:
    fn = getattr(tensor, "clone", None)
    return fn() if callable(fn) else tensor


class DDPBucketProcessor:
    """Synchronous compensate -> compress -> all_reduce(payload) -> decompress -> update.

    Without an `all_reduce` payload transport the bucket only makes the local quantize / dequantize round
    trip (single-process use and tests).  Parity: ccdl_comm/communication/ddp.py:33-97.
    """

    def __init__(self, *, config: CompressionConfig, quantize, dequantize, all_reduce=None,
                 error_feedback: ErrorFeedbackState | None = None) -> None:
        self.config = config
        self.quantize, self.dequantize, self.all_reduce = quantize, dequantize, all_reduce
        self.error_feedback = error_feedback or ErrorFeedbackState()
        self._pipeline = None if all_reduce is None else CompressedAllReduce(
            config=config,
            compress=lambda t, c: coerce_payload(quantize(t, c), shape=tuple(t.shape), dtype="auto"),
            all_reduce=all_reduce, decompress=dequantize)

    @classmethod
    def from_cuda_codec(cls, config: CompressionConfig, *, extension_status: Any | None = None,
                        error_feedback: ErrorFeedbackState | None = None) -> "DDPBucketProcessor":
        """Processor over the package codec (the sm_100a kernels for CUDA buckets, the host codec otherwise)."""

        from ..ops import codec

        def quantize(tensor: Any, active: CompressionConfig) -> Any:
            return codec.quantize_tensor(tensor, active, extension_status=extension_status)

        def dequantize(payload: Any, shape: tuple[int, ...], active: CompressionConfig, dtype: str) -> Any:
            return codec.dequantize_tensor(payload, shape, active, dtype=dtype, extension_status=extension_status)

        return cls(config=config, quantize=quantize, dequantize=dequantize, error_feedback=error_feedback)

    def process(self, bucket: Any, *, dtype: str, reduce: str = "mean") -> Any:
        key = _bucket_key(bucket)
        original = bucket.buffer()
        use_ef = self.config.error_feedback
        prepared = self.error_feedback.compensate(key, original) if use_ef else original
        if self._pipeline is None:
            payload = self.quantize(prepared, self.config)
            restored = self.dequantize(payload, tuple(prepared.shape), self.config, dtype)
        else:
            restored = self._pipeline.run(prepared, shape=tuple(prepared.shape), dtype=dtype, reduce=reduce)
        if use_ef:
            self.error_feedback.update(key, original=prepared, transmitted=restored)
        return restored


class AsyncBucketPipeline:
    """gather work -> (callback thread) dequantize-reduce -> feedback -> complete the outer future."""

    def __init__(self, *, gather_work, future, dequantize_reduce, update_feedback=None, advance_policy=None,
                 completion_manager=None, synchronize_completion: bool = True) -> None:
        self.gather_work = gather_work
        self.future = future
        self.dequantize_reduce = dequantize_reduce
        self.update_feedback = update_feedback
        self.advance_policy = advance_policy
        self.completion_manager = completion_manager or CudaCompletionManager()
        self.synchronize_completion = synchronize_completion

    def run(self) -> Any:
        inner = self.gather_work.get_future() if hasattr(self.gather_work, "get_future") else None
        if inner is not None and hasattr(inner, "then"):
            inner.then(self._complete)
        else:
            self._complete()
        return self.future

    def _complete(self, _ignored: Any = None) -> Any:
        try:
            gathered = self.gather_work.wait()
            restored = self.dequantize_reduce(gathered)
            if self.update_feedback is not None:
                self.update_feedback(restored)
            if self.advance_policy is not None:
                self.advance_policy()
            completion = self.completion_manager.record_for(restored)
            completion.wait()
            if self.synchronize_completion:
                completion.synchronize()
            self.future.set_result(restored)
            return restored
        except BaseException as exc:  # surfaced by DDP when it waits on the future
            self.future.set_exception(exc)
            return None


class AsyncShardPipeline:
    """The reduced-shard counterpart of `AsyncBucketPipeline`: when the payload exchange (an all-to-all work
    object) completes, reduce this rank's shard, run the feedback and policy callbacks, hand the workspace
    leases back with the completion event of the shard, and complete the outer future with a `ReducedShard`
    whose metadata says `async_completion`.  On failure the leases are still released, behind an event, and the
    future carries the exception.  The object is itself work-like (`wait`, `query`, `get_future`, `then`).
    Parity: ccdl_comm/communication/async_shard_pipeline.py:11-129.
    """

    def __init__(self, *, communication_work, future, reduce_shard, update_feedback=None, advance_policy=None,
                 completion_manager=None, synchronize_completion: bool = False, resources=(),
                 workspace_leases=()) -> None:
        self.communication_work = communication_work
        self.future = future
        self.reduce_shard = reduce_shard
        self.update_feedback = update_feedback
        self.advance_policy = advance_policy
        self.completion_manager = completion_manager or CudaCompletionManager()
        self.synchronize_completion = synchronize_completion
        self.resources = tuple(resources)          # buffers kept alive until completion
        self._leases = list(workspace_leases)

    def run(self) -> "AsyncShardPipeline":
        getter = getattr(self.communication_work, "get_future", None)
        inner = getter() if callable(getter) else None
        if inner is not None and hasattr(inner, "then"):
            inner.then(self._complete)
        else:
            self._complete()
        return self

    # -- work protocol --------------------------------------------------------------
    def wait(self):
        waiter = getattr(self.future, "wait", None)
        if callable(waiter):
            return waiter()
        error = getattr(self.future, "exception", None)
        if error is not None and not callable(error):
            raise error
        result = getattr(self.future, "result", None)
        if result is None:
            raise RuntimeError("asynchronous shard result is not complete")
        return result

    def query(self) -> bool:
        done = getattr(self.future, "done", None)
        if callable(done):
            return bool(done())
        return getattr(self.future, "result", None) is not None or getattr(self.future, "exception", None) is not None

    def get_future(self):
        return self.future

    def then(self, callback):
        chain = getattr(self.future, "then", None)
        if not callable(chain):
            raise AttributeError("underlying future does not support then()")
        return chain(callback)

    # -- completion -------------------------------------------------------------------
    def _release(self, completion) -> None:
        while self._leases:
            self._leases.pop(0).release(completion=completion)

    def _complete(self, _ignored: Any = None):
        from dataclasses import replace

        try:
            received = self.communication_work.wait()
            shard = self.reduce_shard(received)
            shard = replace(shard, metadata={**dict(shard.metadata), "async_completion": True})
            if self.update_feedback is not None:
                self.update_feedback(shard)
            if self.advance_policy is not None:
                self.advance_policy()
            completion = self.completion_manager.record_for(shard.shard)
            completion.wait()
            self._release(completion)
            if self.synchronize_completion:
                sync = getattr(completion, "synchronize", None)
                if callable(sync):
                    sync()
            self.future.set_result(shard)
            return shard
        except BaseException as exc:  # noqa: BLE001 - the failure travels through the future
            if self._leases:
                fence = self.completion_manager.record_for(getattr(self._leases[0], "buffer", None))
                fence.wait()
                self._release(fence)
            setter = getattr(self.future, "set_exception", None)
            if callable(setter):
                setter(exc)
                return None
            raise


class _PeerEngine:
    """Lazily built peer group + fused workspaces for one hook.

    Sizing.  DDP hands the hook buckets of very different sizes (the first iteration's buckets differ from
    the rebuilt ones, and `find_unused_parameters` starts with tiny ones), so nothing is sized from the first
    bucket alone: a workspace holds the next power of two of the largest bucket seen (or `max_bucket_numel`),
    the arena is created with room for one doubling, and when a bucket outgrows both, the arena is rebuilt
    collectively (every rank sees the same bucket sizes in the same order, so every rank takes this branch in
    the same call).  An arena handed in by the caller is never rebuilt; outgrowing it is an error.
    """

    MIN_CAP = 1 << 20

    def __init__(self, *, config: CompressionConfig, process_group, peer_group, arena_bytes, max_bucket_numel,
                 max_blocks: int, ef_mode: str) -> None:
        self.config = config
        self.process_group = process_group
        self.group = peer_group
        self._own_group = peer_group is None
        self.arena_bytes = arena_bytes
        self.max_bucket_numel = max_bucket_numel
        self.max_blocks = max_blocks
        self.ef_mode = ef_mode
        self.workspaces: dict[str, Any] = {}
        self.stream = None
        self.launch_count = 0
        self.rebuilds = 0
        self._retired_launches = 0

    # seams for tests: how a group and a workspace are made
    def _make_group(self, total: int, device):
        from .peer_memory import PeerGroup

        dist = import_module("torch.distributed")
        pg = self.process_group if self.process_group is not None else dist.group.WORLD
        return PeerGroup.create(pg, total, device)

    def _make_workspace(self, dtype: str, cap: int):
        from .fused import FusedWorkspace

        ws = FusedWorkspace(self.group, dtype=dtype, config=self.config, max_numel=cap,
                            max_blocks=self.max_blocks or self._blocks_beside_backward(),
                            engine=self._engine(self.group.world_size))
        # line the ranks up before the persistent kernel takes the SMs (LBC_HOOK_GATE=0 launches it at once)
        ws.gate = ws.group.world_size > 1 and os.environ.get("LBC_HOOK_GATE", "1") != "0"
        return ws

    def _blocks_beside_backward(self) -> int:
        """Default grid cap of the hook's kernels: one block per SM.  The hook's kernels run while the backward
        pass still has GEMMs to issue; two blocks per SM (the library's default for a collective on its own) take
        all of an SM's shared memory, one leaves room for a GEMM block beside it (GPT-2 small, 2 GPUs: 28.86 ms
        per step against 29.06 with two blocks per SM and 29.13 with a block on every other SM)."""

        torch = import_module("torch")
        device = getattr(self.group, "device", None)
        try:
            return int(torch.cuda.get_device_properties(device).multi_processor_count)
        except Exception:  # noqa: BLE001 - no CUDA device behind this group (tests with stand-ins)
            return 0

    @staticmethod
    def _engine(world: int) -> str:
        """Buckets go through the single persistent kernel whatever their size and world size: the arena then holds
        that kernel's regions only (about 1.1 x the bucket's payload; the kernel sequence needs 3-7 x)."""

        return os.environ.get("LBC_ENGINE") or "pipe"

    def _need(self, world: int, dtype: str, cap: int) -> int:
        from .fused import FusedWorkspace

        engine = self._engine(world)
        return FusedWorkspace.required_bytes(world, dtype, self.config, cap, world <= 2,
                                             engine=engine if engine in ("pipe", "legacy") else "both") + (1 << 20)

    def _world(self) -> int:
        if self.group is not None:
            return self.group.world_size
        dist = import_module("torch.distributed")
        pg = self.process_group if self.process_group is not None else dist.group.WORLD
        return dist.get_world_size(pg)

    def ensure(self, tensor, dtype: str):
        ws = self.workspaces.get(dtype)
        numel = tensor.numel()
        if ws is not None and ws.max_numel >= numel:
            return ws
        cap = max(int(self.max_bucket_numel or 0), numel, self.MIN_CAP)
        cap = 1 << (cap - 1).bit_length()                 # next power of two
        world = self._world()
        need = self._need(world, dtype, cap)
        device = tensor.device
        if self.group is None:
            total = int(self.arena_bytes) if self.arena_bytes else 2 * need
            self.group = self._make_group(total, device)
        elif self.group.bytes_free < need:
            if not self._own_group:
                raise CCDLUnavailableError(
                    f"the peer arena handed to the hook has {self.group.bytes_free} bytes free, a bucket of "
                    f"{numel} elements needs {need}; create it larger or let the hook own its arena")
            # rebuild: room for every dtype's workspace at its new capacity, and for one doubling of this one
            others = sum(self._need(world, d, w.max_numel) for d, w in self.workspaces.items() if d != dtype)
            caps = {d: w.max_numel for d, w in self.workspaces.items() if d != dtype}
            self._retired_launches += sum(w.launches for w in self.workspaces.values())
            self.group.close()                            # synchronises the device and meets the peers on the host
            self.workspaces.clear()
            self.group = self._make_group(max(int(self.arena_bytes or 0), 2 * need + others), device)
            self.rebuilds += 1
            for d, c in caps.items():
                self.workspaces[d] = self._make_workspace(d, c)
        ws = self._make_workspace(dtype, cap)
        self.workspaces[dtype] = ws
        if self.stream is None:
            from .completion import comm_stream

            self.stream = comm_stream(device)
        return ws

    def check_status(self) -> None:
        if self.group is not None:
            self.group.check_status()

    def reset_after_error(self) -> None:
        """After `check_status` raised: drain the device, zero the scratch counters, clear the status word."""

        if self.group is None:
            return
        self.group.reset_after_error()
        for ws in self.workspaces.values():
            reset = getattr(ws, "reset_pipe_control", None)
            if callable(reset):
                reset()

    @property
    def launches(self) -> int:
        return self._retired_launches + sum(ws.launches for ws in self.workspaces.values())


class DDPCommHook:
    """The callable handed to `DistributedDataParallel.register_comm_hook`."""

    def __init__(self, process_bucket: Callable[[Any], Any], future_factory: Callable[[], Any]) -> None:
        self._process_bucket = process_bucket
        self._future_factory = future_factory
        self.feedback: ErrorFeedbackState | None = None
        self.policy: ErrorFeedbackPolicy | None = None
        self.peer_engine: _PeerEngine | None = None
        self.stats = {"buckets": 0, "bypassed": 0, "peer": 0, "torch": 0}
        self._layouts: dict[Any, tuple] = {}          # bucket key -> ((parameter id, numel), ...) last seen
        self._names: dict[int, str] = {}              # parameter id -> name (after bind_module)
        self._pending_named: dict[str, Any] = {}      # residuals of a name-keyed checkpoint, not yet assembled
        self._adopted: set = set()
        self._stable: dict[Any, int] = {}             # bucket key -> consecutive calls with an unchanged layout
        self._loaded_numels: dict[Any, list[int]] = {}  # segment sizes of a loaded, unnamed checkpoint, per bucket

    def __call__(self, state, bucket):  # no annotations: DDP validates them when present
        self.stats["buckets"] += 1
        self._follow_layout(bucket)
        if tracing.ENABLED:      # LBC_TRACE=1: one NVTX range per bucket on the host timeline
            with tracing.nvtx_range(f"lbc.ddp_bucket[{_bucket_key(bucket)}]"):
                result = self._process_bucket(bucket)
        else:
            result = self._process_bucket(bucket)
        if hasattr(result, "set_result") or hasattr(result, "then"):
            return result
        future = self._future_factory()
        future.set_result(result)
        return future

    # -- bucket layouts ---------------------------------------------------------------------------------
    # DDP fills a bucket with its parameters' gradients in one order during the first iteration and, after it
    # has rebuilt its buckets, in another; a residual is only meaningful in the order it was computed in.  The
    # hook therefore remembers, per bucket, which parameter owned which segment, and re-orders the residual
    # when the order changes.  With `bind_module` the parameters also have names, and checkpoints store the
    # residual per parameter name, so a resumed process, which starts in the first-iteration order again,
    # picks up exactly the residual it left with.
    def bind_module(self, module: Any) -> "DDPCommHook":
        """Give the hook the (unwrapped) model so that it can name the parameters it sees in buckets."""

        self._names = {id(p): name for name, p in module.named_parameters()}
        return self

    @staticmethod
    def _segments(bucket: Any) -> tuple[tuple[int, int], ...] | None:
        """((parameter id, numel), ...) in bucket order, or None for buckets that cannot say (fakes)."""

        params = getattr(bucket, "parameters", None)
        if not callable(params):
            return None
        try:
            return tuple((id(p), int(p.numel())) for p in params())
        except (RuntimeError, TypeError):
            return None

    _SETTLED_AFTER = 4      # DDP re-orders its buckets once, after the first iteration

    def _follow_layout(self, bucket: Any) -> None:
        if self.feedback is None:
            return
        key = _bucket_key(bucket)
        if self._stable.get(key, 0) >= self._SETTLED_AFTER and not self._pending_named:
            return                                  # seen unchanged often enough: stop asking the bucket
        layout = self._segments(bucket)
        if layout is None:
            return
        self._adopt_named_residual(key, layout, bucket)
        self._reconcile_loaded(key, layout)
        known = self._layouts.get(key)
        self._layouts[key] = layout
        self._stable[key] = self._stable.get(key, 0) + 1 if known == layout else 0
        if known is None or known == layout:
            return
        residual = self.feedback.get(key)
        if residual is None:
            return
        if sorted(known) != sorted(layout) or residual.numel() != sum(n for _, n in layout):
            self.feedback.clear(key)            # other parameters in this bucket now: the residual means nothing
            return
        pieces, at = {}, 0
        flat = residual.reshape(-1)
        for owner, numel in known:
            pieces[owner] = flat[at:at + numel]
            at += numel
        import torch

        self.feedback.set(key, torch.cat([pieces[owner] for owner, _ in layout]).reshape(residual.shape))

    def _reconcile_loaded(self, key: Any, layout) -> None:
        """A residual loaded from a checkpoint without parameter names is in the segment order of the process
        that saved it.  If this bucket's segments have other sizes in other places, the residual is re-ordered
        when the sizes identify the segments (no two alike), and dropped otherwise: losing one step of error
        feedback is harmless, adding it to the wrong parameters is not."""

        saved = self._loaded_numels.pop(key, None)
        if saved is None or self.feedback is None:
            return
        here = [numel for _, numel in layout]
        residual = self.feedback.get(key)
        if residual is None or saved == here:
            return
        if sorted(saved) != sorted(here) or len(set(saved)) != len(saved) or residual.numel() != sum(saved):
            self.feedback.clear(key)
            return
        import torch

        pieces = dict(zip(saved, residual.reshape(-1).split(saved)))
        self.feedback.set(key, torch.cat([pieces[numel] for numel in here]).reshape(residual.shape))

    def _adopt_named_residual(self, key: Any, layout, bucket: Any) -> None:
        """After `load_state_dict` of a name-keyed checkpoint: assemble this bucket's residual in its current
        order the first time the bucket is seen."""

        if not self._pending_named or key in self._adopted or not self._names:
            return
        self._adopted.add(key)
        names = [self._names.get(owner) for owner, _ in layout]
        if any(n is None or n not in self._pending_named for n in names):
            return
        import torch

        buffer = bucket.buffer()
        parts = [self._pending_named[n].reshape(-1).to(device=buffer.device, dtype=buffer.dtype) for n in names]
        if [p.numel() for p in parts] != [numel for _, numel in layout]:
            return
        self.feedback.set(key, torch.cat(parts).reshape(buffer.shape))
        self._layouts[key] = layout
        for name in names:                           # handed over: the checkpoint copy is not needed any more
            self._pending_named.pop(name, None)

    def _named_residuals(self) -> dict:
        named = {}
        if not self._names or self.feedback is None:
            return named
        for key, layout in self._layouts.items():
            residual = self.feedback.get(key)
            if residual is None or residual.numel() != sum(n for _, n in layout):
                continue
            at, flat = 0, residual.detach().reshape(-1)
            for owner, numel in layout:
                name = self._names.get(owner)
                if name is not None:
                    named[name] = flat[at:at + numel].clone()
                at += numel
        return named

    # checkpoint / resume of the error-feedback state (an addition)
    def state_dict(self) -> dict:
        return {"feedback": self.feedback.state_dict() if self.feedback else {},
                "policy": self.policy.state_dict() if self.policy else {},
                "residual_by_parameter": self._named_residuals(),
                "segment_numels": {key: [numel for _, numel in layout] for key, layout in self._layouts.items()}}

    def load_state_dict(self, state: dict) -> None:
        named = state.get("residual_by_parameter") or {}
        if self.feedback is not None and named and self._names:
            # per-parameter residuals are re-assembled bucket by bucket, in whatever order the buckets have here
            self.feedback.load_state_dict({"residuals": {}})
            self._pending_named, self._adopted, self._layouts, self._stable = dict(named), set(), {}, {}
        elif self.feedback is not None and state.get("feedback"):
            self.feedback.load_state_dict(state["feedback"])
            self._loaded_numels = {key: list(sizes) for key, sizes in (state.get("segment_numels") or {}).items()}
            self._layouts, self._stable = {}, {}
        if self.policy is not None and state.get("policy"):
            self.policy.load_state_dict(state["policy"])

    @property
    def gpu_launches(self) -> int:
        eng = self.peer_engine
        return eng.launches if eng else 0

    def check_status(self) -> None:
        """Raises `AsyncCommunicationError` when a kernel of an earlier bucket gave up waiting for a peer (its
        bucket then kept this rank's local gradient).  Reads pinned host memory, no synchronisation: call it
        after `optimizer.step()` or wherever a wrong step must not go unnoticed; the hook itself calls it
        before every bucket."""

        if self.peer_engine is not None:
            self.peer_engine.check_status()

    def reset_after_error(self) -> None:
        if self.peer_engine is not None:
            self.peer_engine.reset_after_error()


def create_ddp_comm_hook(
    config: CompressionConfig,
    *,
    dtype: str = "auto",
    strategy: str = "all_reduce",
    reduce: str = "mean",
    quantize: Callable[[Any, CompressionConfig], Any] | None = None,
    dequantize: Callable[[Any, tuple[int, ...], CompressionConfig, str], Any] | None = None,
    all_reduce: Callable[[CompressedPayload, str], CompressedPayload] | None = None,
    all_gather: Callable[[Any], GatheredPayloads] | None = None,
    async_gather: bool = False,
    async_error_feedback: bool = False,
    synchronize_async_feedback_completion: bool = True,
    async_all_gather: Callable[[Any], Any] | None = None,
    native_error_feedback_update: Callable[[Any, Any, Any], Any] | None = None,
    native_dequantize_reduce_update_feedback: Callable[..., Any] | None = None,
    native_inplace_dequantize_reduce_update_feedback: Callable[..., bool] | None = None,
    reduce_scatter_all_gather: Callable[..., Any] | None = None,
    hierarchical_all_reduce: Callable[..., Any] | None = None,
    topology_all_reduce: Callable[..., Any] | None = None,
    topology_method: str | None = None,
    allocate_dequantized_workspace: Callable[[Any, tuple[int, ...], CompressionConfig], Any] | None = None,
    workspace_cache_max_entries: int | None = 1,
    workspace_cache_max_bytes: int | None = None,
    completion_manager: Any | None = None,
    fuse_payload: bool = False,
    fuse_payload_min_numel: int = DEFAULT_FUSED_PAYLOAD_MIN_NUMEL,
    min_compress_numel: int = 0,
    bypass_all_reduce: Callable[[Any, str], Any] | None = None,
    error_feedback: ErrorFeedbackState | None = None,
    extension_status: CudaExtensionStatus | None = None,
    future_factory: Callable[[], Any] = _torch_future_factory,
    annotation_provider: Callable[[], dict[str, Any]] | None = None,
    # --- additions -------------------------------------------------------------
    process_group: Any | None = None,
    peer_group: Any | None = None,
    transport: str = "auto",
    ef_mode: str = "reference",
    arena_bytes: int | None = None,
    max_bucket_numel: int | None = None,
    max_blocks: int = 0,
    local_group_size: int | None = None,
    module: Any | None = None,
) -> Callable[[Any, Any], Any]:
    """Build the hook: `ddp_model.register_comm_hook(state=None, hook=hook)`."""

    if transport not in ("auto", "peer", "torch"):
        raise ValueError("transport must be 'auto', 'peer' or 'torch'")
    if ef_mode not in ("reference", "local"):
        raise ValueError("ef_mode must be 'reference' or 'local'")
    if topology_method not in _TOPOLOGY_METHODS:
        raise ValueError(f"unsupported topology method {topology_method!r}")
    injected = any(v is not None for v in (quantize, dequantize, all_reduce, all_gather, async_all_gather))
    world_size = _dist_fact("get_world_size", 1)
    plan = plan_ddp_compression_strategy(
        requested_strategy=strategy, world_size=world_size, rank=_dist_fact("get_rank", 0),
        local_world_size=_env_int("LOCAL_WORLD_SIZE"), node_count=_env_int("NODE_COUNT"),
        capabilities=CollectiveCapabilities(
            reduce_scatter=True, hierarchical=True, topology=True, fused_dequant_reduce=True,
            hierarchical_recommended=False))
    effective = plan.strategy
    feedback = error_feedback or ErrorFeedbackState()
    policy = ErrorFeedbackPolicy(config)
    plain_all_reduce = bypass_all_reduce or make_torch_tensor_all_reduce(group=process_group)
    manager = completion_manager or CudaCompletionManager(extension_status=extension_status)
    peer = _PeerEngine(config=config, process_group=process_group, peer_group=peer_group, arena_bytes=arena_bytes,
                       max_bucket_numel=max_bucket_numel, max_blocks=max_blocks, ef_mode=ef_mode)
    hook_ref: list[DDPCommHook] = []

    def use_peer(tensor: Any) -> bool:
        if transport == "torch" or injected or not bool(getattr(tensor, "is_cuda", False)):
            return False
        if not codec.is_fast_profile(config) or effective in ("native_nccl",):
            return False
        if effective == "hierarchical" and hierarchical_all_reduce is not None:
            return False
        status = extension_status if extension_status is not None else load_cuda_extension()
        if not status.available:
            if transport == "peer":
                raise RuntimeError(f"peer transport requested but the extension is unavailable: {status.reason}")
            raise RuntimeError("CUDA bucket but the sm_100a extension is not loaded: "
                               f"{status.reason} (refusing to fall back silently)")
        return True

    # ---------------------------------------------------------------- peer engine
    def peer_bucket(bucket: Any) -> Any:
        torch = import_module("torch")
        tensor = bucket.buffer()
        key = _bucket_key(bucket)
        name = _resolve_dtype(dtype, tensor)
        peer.check_status()                     # an earlier bucket's wait ran out: say so now, not never
        ws = peer.ensure(tensor, name)
        decision = policy.decide(key, numel=tensor.numel())
        residual = feedback.residual_for(key, tensor) if (decision.apply or decision.update) else None
        stages = {"all_gather": 1, "reduce_scatter": 2, "topology": 2}.get(effective)
        producer = torch.cuda.current_stream(tensor.device)
        peer.stream.wait_stream(producer)
        with torch.cuda.stream(peer.stream):
            ws.all_reduce(tensor, residual=residual if decision.apply else None,
                          update_residual=decision.update, op=reduce, stages=stages, ef_mode=ef_mode)
            future = torch.futures.Future(devices=[tensor.device])
            future.set_result(tensor)
        policy.advance(key)
        hook_ref[0].stats["peer"] += 1
        return future

    def peer_hierarchical_bucket(bucket: Any) -> Any:
        """strategy="hierarchical" on CUDA: the communicator's three-stage chain (reduce-scatter inside the local
        group, all-reduce of the shard across groups, gather inside the group) on the side stream, with the
        reference's error-feedback rule around it: prepared = T(gradient + residual) goes in, and the residual
        becomes T(prepared - result)."""

        torch = import_module("torch")
        from .communicator import get_communicator
        from .completion import comm_stream

        tensor = bucket.buffer()
        key = _bucket_key(bucket)
        comm = get_communicator(process_group)
        comm.check_status()
        decision = policy.decide(key, numel=tensor.numel())
        residual = feedback.residual_for(key, tensor) if (decision.apply or decision.update) else None
        if peer.stream is None:
            peer.stream = comm_stream(tensor.device)
        peer.stream.wait_stream(torch.cuda.current_stream(tensor.device))
        with torch.cuda.stream(peer.stream):
            if residual is not None and decision.apply:
                tensor.add_(residual)
            if residual is not None and decision.update:
                residual.copy_(tensor)                              # `prepared`, parked in the residual buffer
            comm.hierarchical_all_reduce(tensor, config=config, op=reduce, local_group_size=local_group_size)
            if residual is not None and decision.update:
                codec.update_error_feedback_residual(residual, tensor, residual, extension_status=extension_status)
            future = torch.futures.Future(devices=[tensor.device])
            future.set_result(tensor)
        policy.advance(key)
        hook_ref[0].stats["peer"] += 1
        hook_ref[0].stats["hierarchical"] = hook_ref[0].stats.get("hierarchical", 0) + 1
        return future

    def use_general_peer(tensor: Any) -> bool:
        """CUDA bucket with a top-k / code-book / stochastic profile: general kernels + peer-memory transport."""

        if transport == "torch" or injected or not bool(getattr(tensor, "is_cuda", False)):
            return False
        if codec.is_fast_profile(config) or effective == "native_nccl":
            return False
        status = extension_status if extension_status is not None else load_cuda_extension()
        return bool(status.available)

    def peer_general_bucket(bucket: Any) -> Any:
        torch = import_module("torch")
        from .communicator import get_communicator
        from .completion import comm_stream

        tensor = bucket.buffer()
        key = _bucket_key(bucket)
        comm = get_communicator(process_group)
        comm.check_status()
        decision = policy.decide(key, numel=tensor.numel())
        residual = feedback.residual_for(key, tensor) if (decision.apply or decision.update) else None
        if peer.stream is None:
            peer.stream = comm_stream(tensor.device)
        peer.stream.wait_stream(torch.cuda.current_stream(tensor.device))
        with torch.cuda.stream(peer.stream):
            comm.all_reduce(tensor, config=config, op=reduce, strategy="all_gather",
                            residual=residual if decision.apply else None, update_residual=decision.update)
            future = torch.futures.Future(devices=[tensor.device])
            future.set_result(tensor)
        policy.advance(key)
        hook_ref[0].stats["peer"] += 1
        hook_ref[0].stats["general"] = hook_ref[0].stats.get("general", 0) + 1
        return future

    # --------------------------------------------------------------- torch engine
    def q(tensor: Any, cfg: CompressionConfig) -> Any:
        if quantize is not None:
            return quantize(tensor, cfg)
        return codec.quantize_tensor(tensor, cfg, extension_status=extension_status)

    def dq(payload: Any, shape: tuple[int, ...], cfg: CompressionConfig, name: str) -> Any:
        if dequantize is not None:
            return dequantize(payload, shape, cfg, name)
        return codec.dequantize_tensor(payload_buffer(payload), shape, cfg, dtype=name,
                                       extension_status=extension_status)

    if all_gather is not None:
        plain_gather = fused_gather = all_gather
    else:
        base_gather = make_torch_all_gather(group=process_group)
        plain_gather = make_payload_all_gather(base_gather)
        fused_gather = make_fused_payload_all_gather(base_gather)
    async_gather_fn = async_all_gather or make_torch_async_all_gather(group=process_group)
    all_to_all = make_torch_all_to_all(group=process_group)
    restored_cache: dict[Any, Any] = {}

    def restored_buffer(key: Any, like: Any) -> Any:
        buf = restored_cache.get(key)
        if buf is None or tuple(buf.shape) != tuple(like.shape) or buf.dtype != like.dtype:
            if workspace_cache_max_entries is not None and len(restored_cache) >= max(1, workspace_cache_max_entries):
                restored_cache.pop(next(iter(restored_cache)))
            alloc = allocate_dequantized_workspace or codec.allocate_dequantized_buffer
            buf = alloc(like, tuple(like.shape), config)
            if workspace_cache_max_bytes is None or buf.numel() * buf.element_size() <= workspace_cache_max_bytes:
                restored_cache[key] = buf
        return buf

    def gather_reduce_native(key, prepared, decision, name) -> Any:
        """Native-codec all-gather strategy, synchronous or through the async pipeline."""

        payload = coerce_payload(q(prepared, config), shape=tuple(prepared.shape), dtype=name)
        needs_fb = decision.apply or decision.update
        shape = tuple(prepared.shape)

        def reduce_buffers(buffers, want_feedback: bool):
            if want_feedback and decision.update and codec.is_fast_profile(config):
                residual = feedback.residual_for(key, prepared)
                restored = restored_buffer(key, prepared)
                fused = native_inplace_dequantize_reduce_update_feedback or \
                    codec.inplace_dequantize_reduce_mean_update_error_feedback
                if fused(buffers, prepared, restored, residual, config, extension_status=extension_status,
                         reduce=reduce):
                    return restored.reshape(shape), True
            out = codec.dequantize_reduce_tensors(buffers, shape, config, dtype=name,
                                                  extension_status=extension_status, reduce=reduce)
            return out, False

        def finish(restored, fused_done: bool) -> None:
            if decision.update and not fused_done:
                latest = feedback.get(key)
                if native_error_feedback_update is not None and latest is not None:
                    native_error_feedback_update(prepared, restored, latest)
                else:
                    feedback.update(key, original=prepared, transmitted=restored)

        if async_gather and (async_error_feedback or not needs_fb):
            work = async_gather_fn(payload_buffer(payload))
            outer = future_factory()
            done = [False]

            def dequantize_reduce(gathered: GatheredPayloads):
                restored, done[0] = reduce_buffers([payload_buffer(p) for p in gathered.payloads], needs_fb)
                return restored

            return AsyncBucketPipeline(
                gather_work=work, future=outer, dequantize_reduce=dequantize_reduce,
                update_feedback=lambda restored: finish(restored, done[0]),
                advance_policy=lambda: policy.advance(key), completion_manager=manager,
                synchronize_completion=synchronize_async_feedback_completion).run()
        gather = fused_gather if should_fuse_payload(prepared, enabled=fuse_payload,
                                                     min_numel=fuse_payload_min_numel) else plain_gather
        gathered = gather(payload)
        restored, fused_done = reduce_buffers([payload_buffer(p) for p in gathered.payloads], needs_fb)
        finish(restored, fused_done)
        policy.advance(key)
        return restored

    def torch_all_gather_bucket(bucket: Any) -> Any:
        key = _bucket_key(bucket)
        original = bucket.buffer()
        decision = policy.decide(key, numel=_numel(original))
        prepared = feedback.compensate(key, original) if decision.apply else original
        name = _resolve_dtype(dtype, prepared)
        if dequantize is None and reduce in ("mean", "sum"):
            return gather_reduce_native(key, prepared, decision, name)
        gather = fused_gather if should_fuse_payload(prepared, enabled=fuse_payload,
                                                     min_numel=fuse_payload_min_numel) else plain_gather
        pipeline = CompressedAllGatherReduce(
            config=config,
            compress=lambda t, c: coerce_payload(q(t, c), shape=tuple(t.shape), dtype=name),
            all_gather=gather, decompress=dq)
        restored = pipeline.run(prepared, shape=tuple(prepared.shape), dtype=name, reduce=reduce)
        if decision.update:
            feedback.update(key, original=prepared, transmitted=restored)
        policy.advance(key)
        return restored

    def torch_reduce_scatter_bucket(bucket: Any) -> Any:
        """chunk -> quantize each -> all_to_all -> reduce own shard -> quantize -> all_gather -> decode."""

        torch = import_module("torch")
        from ..core.chunking import GroupShardPlan

        key = _bucket_key(bucket)
        original = bucket.buffer()
        if reduce_scatter_all_gather is not None:
            return reduce_scatter_all_gather(original, config=config, op=reduce, async_op=False,
                                             dtype=_resolve_dtype(dtype, original))
        decision = policy.decide(key, numel=_numel(original))
        prepared = feedback.compensate(key, original) if decision.apply else original
        name = _resolve_dtype(dtype, prepared)
        flat = prepared.reshape(-1)
        world = _dist_fact("get_world_size", 1) if process_group is None else \
            import_module("torch.distributed").get_world_size(process_group)
        plan = GroupShardPlan.build(flat.numel(), world, config.group_size, 1)
        padded = torch.nn.functional.pad(flat, (0, plan.padded_numel - flat.numel()))
        chunks = [padded[r * plan.shard_numel:(r + 1) * plan.shard_numel] for r in range(world)]
        received = all_to_all([codec.quantize_tensor(c, config, extension_status=extension_status) for c in chunks])
        shard = codec.dequantize_reduce_tensors(received, (plan.shard_numel,), config, dtype=name,
                                                extension_status=extension_status, reduce=reduce)
        gathered = plain_gather(codec.quantize_tensor(shard, config, extension_status=extension_status))
        parts = [codec.dequantize_tensor(payload_buffer(p), (plan.shard_numel,), config, dtype=name,
                                         extension_status=extension_status) for p in gathered.payloads]
        restored = torch.cat(parts)[:flat.numel()].reshape(prepared.shape)
        if decision.update:
            feedback.update(key, original=prepared, transmitted=restored)
        policy.advance(key)
        return restored

    processor = None
    if all_reduce is not None:
        processor = DDPBucketProcessor(config=config, quantize=q, dequantize=dq, all_reduce=all_reduce,
                                       error_feedback=feedback)

    def with_feedback(bucket: Any, transport: Callable[[Any, str], Any]) -> Any:
        """Error feedback around a transport that only knows how to all-reduce a tensor: what is sent is
        T(gradient + residual), and the residual becomes what the transport lost of it.  The reference leaves
        its hierarchical and topology strategies without error feedback (ccdl_comm/communication/ddp_hook.py:
        148-177); here every strategy has it, as on the peer-memory path."""

        key = _bucket_key(bucket)
        original = bucket.buffer()
        decision = policy.decide(key, numel=_numel(original))
        prepared = feedback.compensate(key, original) if decision.apply else original
        name = _resolve_dtype(dtype, prepared)
        # transports reduce in place; `prepared` is still needed for the residual
        restored = transport(_clone(prepared) if decision.update else prepared, name)
        if decision.update:
            feedback.update(key, original=prepared, transmitted=restored)
        policy.advance(key)
        return restored

    def torch_bucket(bucket: Any) -> Any:
        hook_ref[0].stats["torch"] += 1
        tensor = bucket.buffer()
        name = _resolve_dtype(dtype, tensor)
        if effective == "native_nccl":
            return plain_all_reduce(_clone(tensor), reduce)
        if effective == "hierarchical":
            from .collectives.hierarchical import compressed_hierarchical_all_reduce

            return with_feedback(bucket, lambda t, nm: compressed_hierarchical_all_reduce(
                t, config=config, op=reduce, async_op=False, dtype=nm,
                hierarchical_all_reduce=hierarchical_all_reduce, extension_status=extension_status,
                local_group_size=local_group_size))
        if effective == "topology" and topology_all_reduce is not None:
            return with_feedback(bucket, lambda t, nm: topology_all_reduce(
                t, config=config, op=reduce, async_op=False, dtype=nm, extension_status=extension_status))
        if effective == "all_reduce" and processor is not None:
            return processor.process(bucket, dtype=name, reduce=reduce)
        if effective in ("reduce_scatter", "topology"):
            return torch_reduce_scatter_bucket(bucket)
        return torch_all_gather_bucket(bucket)

    def process_bucket(bucket: Any) -> Any:
        tensor = bucket.buffer()
        if min_compress_numel > 0 and _numel(tensor) < min_compress_numel:
            hook_ref[0].stats["bypassed"] += 1
            return plain_all_reduce(_clone(tensor), reduce)
        if use_peer(tensor):
            return peer_hierarchical_bucket(bucket) if effective == "hierarchical" else peer_bucket(bucket)
        if use_general_peer(tensor) and bool(getattr(tensor, "is_contiguous", lambda: False)()):
            return peer_general_bucket(bucket)
        return torch_bucket(bucket)

    holder = DDPCommHook(process_bucket, future_factory)
    hook_ref.append(holder)
    holder.feedback, holder.policy, holder.peer_engine = feedback, policy, peer

    def hook(state, bucket):  # a plain function: DDP inspects `__name__` and the annotations
        return holder(state, bucket)

    hook.holder = holder
    hook.stats = holder.stats
    hook.feedback, hook.policy, hook.peer_engine = feedback, policy, peer
    hook.state_dict = holder.state_dict
    hook.load_state_dict = holder.load_state_dict
    hook.bind_module = holder.bind_module
    hook.check_status = holder.check_status
    hook.reset_after_error = holder.reset_after_error
    if module is not None:
        holder.bind_module(module)
    hook.gpu_launches = lambda: holder.gpu_launches
    hook._ccdl_strategy_plan = plan
    hook._ccdl_effective_strategy = effective
    hook._ccdl_topology_method = topology_method
    try:
        provider = annotation_provider or _torch_ddp_annotations
        hook.__annotations__ = dict(provider())
    except (ImportError, ModuleNotFoundError, AttributeError, TypeError):
        pass
    return hook


def _torch_ddp_annotations() -> dict[str, Any]:
    torch = import_module("torch")
    dist = import_module("torch.distributed")
    return {"state": object, "bucket": dist.GradBucket, "return": torch.futures.Future[torch.Tensor]}
