"""DDP hook logic with hand-written fakes instead of a cluster: one simulated rank, fabricated peers."""

import subprocess
import sys

import pytest
import torch

from lowbit_comm_b200 import CompressionConfig, create_ddp_comm_hook
from lowbit_comm_b200.ops import codec
from lowbit_comm_b200.ops.error_feedback import ErrorFeedbackState
from lowbit_comm_b200.parallel.ddp_hook import AsyncBucketPipeline, DDPBucketProcessor
from lowbit_comm_b200.parallel.payload import CompressedPayload, GatheredPayloads, payload_buffer


class FakeBucket:
    def __init__(self, tensor, index=0):
        self._t, self._i = tensor, index

    def buffer(self):
        return self._t

    def index(self):
        return self._i


class FakeFuture:
    def __init__(self):
        self.value, self.error = None, None

    def set_result(self, v):
        self.value = v

    def set_exception(self, e):
        self.error = e


def mirrored_gather(world):
    """Every fabricated peer sent the same payload as this rank."""

    calls = []

    def gather(payload):
        calls.append(payload)
        return GatheredPayloads(tuple(payload for _ in range(world)))

    gather.calls = calls
    return gather


def test_all_gather_strategy_with_error_feedback_matches_manual_math():
    cfg = CompressionConfig()
    gather = mirrored_gather(3)
    feedback = ErrorFeedbackState()
    hook = create_ddp_comm_hook(cfg, strategy="all_gather", all_gather=gather, error_feedback=feedback,
                                future_factory=FakeFuture)
    grad = (torch.randn(1000) * 0.01).to(torch.bfloat16)
    out = hook(None, FakeBucket(grad.clone(), 7)).value
    expect = codec.dequantize_tensor(codec.quantize_tensor(grad, cfg), grad.shape, cfg, dtype="bf16")
    assert torch.equal(out, expect) and len(gather.calls) == 1
    res1 = feedback.get(7).clone()
    assert (res1.float() - (grad.float() - expect.float())).abs().max() < 1e-3
    hook(None, FakeBucket(grad.clone(), 7))            # second step: the residual is added before quantization
    prepared = (grad.float() + res1.float()).to(torch.bfloat16)
    sent = payload_buffer(gather.calls[1])
    assert torch.equal(sent, codec.quantize_tensor(prepared, cfg))
    assert hook._ccdl_effective_strategy == "all_gather" and hook._ccdl_strategy_plan.requested_strategy == "all_gather"
    assert hook.stats["buckets"] == 2 and hook.stats["torch"] == 2
    state = hook.state_dict()
    assert 7 in state["feedback"]["residuals"] and state["policy"]["steps"][7] == 2


def test_small_bucket_bypass_and_policies():
    seen = []
    hook = create_ddp_comm_hook(CompressionConfig(), strategy="all_gather", all_gather=mirrored_gather(2),
                                min_compress_numel=100, bypass_all_reduce=lambda t, op: seen.append(op) or t * 2,
                                future_factory=FakeFuture)
    small = torch.ones(10)
    assert torch.equal(hook(None, FakeBucket(small)).value, small * 2) and seen == ["mean"]
    assert hook.stats["bypassed"] == 1
    feedback = ErrorFeedbackState()
    no_ef = create_ddp_comm_hook(CompressionConfig(error_feedback=False), strategy="all_gather",
                                 all_gather=mirrored_gather(2), error_feedback=feedback, future_factory=FakeFuture)
    no_ef(None, FakeBucket(torch.randn(128), 1))
    assert feedback.get(1) is None


def test_injected_codec_path_and_byte_sum_transport():
    log = []

    def quantize(t, cfg):
        log.append("q")
        return CompressedPayload(t * 2, tuple(t.shape), "fp32")

    def dequantize(p, shape, cfg, dtype):
        log.append("dq")
        return payload_buffer(p) / 2

    hook = create_ddp_comm_hook(CompressionConfig(error_feedback=False), strategy="all_gather", quantize=quantize,
                                dequantize=dequantize, all_gather=mirrored_gather(4), future_factory=FakeFuture)
    g = torch.arange(8, dtype=torch.float32)
    assert torch.allclose(hook(None, FakeBucket(g)).value, g) and log == ["q", "dq", "dq", "dq", "dq"]
    proc = DDPBucketProcessor(config=CompressionConfig(), quantize=quantize, dequantize=dequantize,
                              all_reduce=lambda payload, op: payload)
    assert torch.allclose(proc.process(FakeBucket(g, 3), dtype="fp32"), g)
    summed = create_ddp_comm_hook(CompressionConfig(error_feedback=False), strategy="all_reduce", quantize=quantize,
                                  dequantize=dequantize, all_reduce=lambda payload, op: payload, future_factory=FakeFuture)
    assert torch.allclose(summed(None, FakeBucket(g)).value, g)


def test_async_pipeline_orders_steps_and_reports_errors():
    order = []

    class Work:
        def wait(self):
            order.append("wait")
            return GatheredPayloads((torch.ones(2),))

        def get_future(self):
            class F:
                def then(_, cb):
                    order.append("then")
                    cb(None)
            return F()

    class Completion:
        def wait(self):
            order.append("stream-wait")

        def synchronize(self):
            order.append("host-sync")

    class Manager:
        def record_for(self, t, stream=None):
            order.append("record")
            return Completion()

    fut = FakeFuture()
    AsyncBucketPipeline(gather_work=Work(), future=fut, dequantize_reduce=lambda g: order.append("reduce") or g.payloads[0],
                        update_feedback=lambda r: order.append("feedback"), advance_policy=lambda: order.append("advance"),
                        completion_manager=Manager(), synchronize_completion=False).run()
    assert order == ["then", "wait", "reduce", "feedback", "advance", "record", "stream-wait"]
    assert torch.equal(fut.value, torch.ones(2))
    bad = FakeFuture()
    AsyncBucketPipeline(gather_work=Work(), future=bad, completion_manager=Manager(),
                        dequantize_reduce=lambda g: (_ for _ in ()).throw(RuntimeError("decode failed"))).run()
    assert isinstance(bad.error, RuntimeError) and bad.value is None


def test_async_gather_strategy_uses_the_injected_async_transport():
    cfg = CompressionConfig()

    class Work:
        def __init__(self, payload):
            self.payload = payload

        def wait(self):
            return GatheredPayloads((self.payload, self.payload))

        def get_future(self):
            return None

    hook = create_ddp_comm_hook(cfg, strategy="all_gather", async_gather=True, async_error_feedback=True,
                                async_all_gather=lambda buf: Work(buf), future_factory=FakeFuture,
                                synchronize_async_feedback_completion=False)
    grad = (torch.randn(256) * 0.01).to(torch.float16)
    fut = hook(None, FakeBucket(grad.clone(), 0))
    expect = codec.dequantize_tensor(codec.quantize_tensor(grad, cfg), grad.shape, cfg, dtype="fp16")
    assert torch.equal(fut.value, expect) and hook.feedback.get(0) is not None


def test_argument_validation_and_annotations():
    with pytest.raises(ValueError):
        create_ddp_comm_hook(CompressionConfig(), transport="carrier-pigeon")
    with pytest.raises(ValueError):
        create_ddp_comm_hook(CompressionConfig(), topology_method="moebius")
    with pytest.raises(ValueError):
        create_ddp_comm_hook(CompressionConfig(), ef_mode="psychic")
    hook = create_ddp_comm_hook(CompressionConfig(), annotation_provider=lambda: {"bucket": int, "return": str})
    assert hook.__annotations__ == {"bucket": int, "return": str} and hook.__name__ == "hook"


def test_package_import_is_torch_free():
    code = "import sys, lowbit_comm_b200 as l; l.CompressionConfig(); l.CompileCache(); assert 'torch' not in sys.modules"
    subprocess.run([sys.executable, "-c", code], check=True, cwd=str(__import__("pathlib").Path(__file__).parents[1]))


def test_bucket_processor_from_cuda_codec_round_trips_locally():
    import torch

    from lowbit_comm_b200 import CompressionConfig
    from lowbit_comm_b200.ops import oracle
    from lowbit_comm_b200.parallel.ddp_hook import DDPBucketProcessor

    class Bucket:
        def __init__(self, t):
            self._t = t

        def buffer(self):
            return self._t

        def index(self):
            return 0

    cfg = CompressionConfig()
    proc = DDPBucketProcessor.from_cuda_codec(cfg)
    assert proc.all_reduce is None and callable(proc.quantize) and callable(proc.dequantize)
    x = (torch.randn(64 * 9 + 5, generator=torch.Generator().manual_seed(2)) * 0.1).to(torch.bfloat16)
    first = proc.process(Bucket(x.clone()), dtype="bf16")
    want = oracle.decode(oracle.encode(x, cfg), x.numel(), cfg, "bf16")
    assert torch.equal(first, want)
    residual = proc.error_feedback.get(0) if proc.error_feedback.get(0) is not None else None
    second = proc.process(Bucket(x.clone()), dtype="bf16")                       # second step: residual is added first
    assert residual is None or not torch.equal(second, first) or torch.equal(residual, torch.zeros_like(residual))


def test_async_shard_pipeline_releases_leases_and_marks_the_shard():
    from lowbit_comm_b200 import ReducedShard
    from lowbit_comm_b200.parallel.ddp_hook import AsyncShardPipeline

    log = []

    class Completion:
        def __init__(self, of):
            self.of = of

        def wait(self):
            log.append(("completion.wait", self.of))

        def synchronize(self):
            log.append(("completion.synchronize", self.of))

    class Manager:
        def record_for(self, tensor, stream=None):
            log.append(("record_for", tensor))
            return Completion(tensor)

    class Lease:
        def __init__(self, name):
            self.name, self.buffer = name, f"buffer:{name}"

        def release(self, *, completion):
            log.append(("release", self.name, completion.of))

    class InnerFuture:
        def __init__(self):
            self.callbacks = []

        def then(self, cb):
            self.callbacks.append(cb)

    class Work:
        def __init__(self, fail=False):
            self.inner, self.fail = InnerFuture(), fail

        def get_future(self):
            return self.inner

        def wait(self):
            if self.fail:
                raise RuntimeError("all_to_all failed")
            return ["payload0", "payload1"]

    class Future:
        result = exception = None

        def set_result(self, value):
            self.result = value

        def set_exception(self, exc):
            self.exception = exc

        def done(self):
            return self.result is not None or self.exception is not None

    def reduce_shard(received):
        log.append(("reduce", tuple(received)))
        return ReducedShard(shard="shard-tensor", shard_index=1, shard_numel=4, original_shape=(8,), original_numel=8,
                            world_size=2, reduce="mean", metadata={"fused": True})

    work, fut = Work(), Future()
    pipe = AsyncShardPipeline(communication_work=work, future=fut, reduce_shard=reduce_shard,
                              update_feedback=lambda s: log.append(("feedback", s.shard_index)),
                              advance_policy=lambda: log.append(("advance",)), completion_manager=Manager(),
                              synchronize_completion=True, resources=("keep",),
                              workspace_leases=(Lease("send"), Lease("recv"))).run()
    assert not pipe.query() and log == [] and pipe.resources == ("keep",)      # nothing happens before the exchange ends
    work.inner.callbacks[0](None)
    assert pipe.query() and pipe.get_future() is fut
    shard = fut.result
    assert shard.metadata == {"fused": True, "async_completion": True} and shard.shard == "shard-tensor"
    assert log == [("reduce", ("payload0", "payload1")), ("feedback", 1), ("advance",), ("record_for", "shard-tensor"),
                   ("completion.wait", "shard-tensor"), ("release", "send", "shard-tensor"),
                   ("release", "recv", "shard-tensor"), ("completion.synchronize", "shard-tensor")]

    log.clear()
    work, fut = Work(fail=True), Future()
    AsyncShardPipeline(communication_work=work, future=fut, reduce_shard=reduce_shard, completion_manager=Manager(),
                       workspace_leases=(Lease("send"),)).run()
    work.inner.callbacks[0](None)
    assert isinstance(fut.exception, RuntimeError) and fut.result is None
    assert log == [("record_for", "buffer:send"), ("completion.wait", "buffer:send"), ("release", "send", "buffer:send")]


def test_cuda_stream_work_orders_streams_without_host_waits():
    from lowbit_comm_b200.parallel.completion import CudaStreamWork

    log = []

    class Stream:
        def __init__(self, name):
            self.name = name

        def wait_stream(self, other):
            log.append(("wait_stream", self.name, other.name))

    class Event:
        def record(self, stream):
            log.append(("record", stream.name))

        def wait(self):
            log.append(("event.wait",))

        def query(self):
            return True

    class Guard:
        def __init__(self, stream):
            self.stream = stream

        def __enter__(self):
            log.append(("enter", self.stream.name))

        def __exit__(self, *a):
            log.append(("exit", self.stream.name))

    event_type, stream_type = Event, Stream

    class Cuda:
        Event = event_type
        current = stream_type("compute")

        @staticmethod
        def current_stream():
            return Cuda.current

        @staticmethod
        def current_device():
            return 0

        @staticmethod
        def Stream(device):  # noqa: N802 - mirrors torch.cuda.Stream
            return stream_type(f"comm{device}")

        @staticmethod
        def stream(s):
            return Guard(s)

    class Torch:
        cuda = Cuda

    class Handle:
        def wait(self):
            log.append(("handle.wait",))

    with CudaStreamWork(torch=Torch, async_op=True, handle=Handle()) as work:
        log.append(("body",))
    assert log == [("wait_stream", "comm0", "compute"), ("enter", "comm0"), ("body",), ("exit", "comm0"),
                   ("record", "comm0")]
    assert work.query()
    work.wait()
    assert log[-2:] == [("handle.wait",), ("event.wait",)]
    log.clear()
    with CudaStreamWork(torch=Torch, async_op=False) as sync:
        pass
    assert sync.stream is Cuda.current and log[-1] == ("event.wait",) and sync.query()


class LayoutBucket(FakeBucket):
    """A bucket that also says which parameters its gradient segments belong to, like DDP's GradBucket."""

    def __init__(self, params, index=0):
        super().__init__(torch.cat([p.grad.reshape(-1) for p in params]), index)
        self._params = list(params)

    def parameters(self):
        return self._params


def test_residual_follows_the_parameters_when_the_bucket_order_changes():
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    params = list(model.parameters())
    for p in params:
        p.grad = torch.randn_like(p) * 0.01
    feedback = ErrorFeedbackState()
    hook = create_ddp_comm_hook(CompressionConfig(), strategy="all_gather", all_gather=mirrored_gather(2),
                                error_feedback=feedback, future_factory=FakeFuture, module=model)
    hook(None, LayoutBucket(params))                                   # first-iteration order
    first = feedback.get(0).clone()
    assert first.abs().max() > 0
    sizes = [p.numel() for p in params]
    by_param = dict(zip((id(p) for p in params), first.split(sizes)))
    reordered = list(reversed(params))
    hook.holder._follow_layout(LayoutBucket(reordered))                # what the next call does first
    moved = feedback.get(0)
    assert torch.equal(moved, torch.cat([by_param[id(p)] for p in reordered]))
    saved = hook.state_dict()
    names = [name for name, _ in model.named_parameters()]
    assert sorted(saved["residual_by_parameter"]) == sorted(names)
    assert torch.equal(saved["residual_by_parameter"][names[0]], by_param[id(params[0])])

    # a fresh hook on a fresh copy of the model, buckets in the original order again
    twin = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    for p, q in zip(twin.parameters(), params):
        p.grad = q.grad.clone()
    feedback2 = ErrorFeedbackState()
    hook2 = create_ddp_comm_hook(CompressionConfig(), strategy="all_gather", all_gather=mirrored_gather(2),
                                 error_feedback=feedback2, future_factory=FakeFuture)
    hook2.bind_module(twin)
    hook2.load_state_dict(saved)
    assert feedback2.get(0) is None                                    # assembled when the bucket shows up
    hook2.holder._follow_layout(LayoutBucket(list(twin.parameters())))
    assert torch.equal(feedback2.get(0), first)

    # other parameters under the same bucket index: the old residual is dropped, not misapplied
    stranger = torch.nn.Linear(3, 3)
    for p in stranger.parameters():
        p.grad = torch.zeros_like(p)
    hook.holder._follow_layout(LayoutBucket(list(stranger.parameters())))
    assert feedback.get(0) is None


def test_unnamed_checkpoint_is_reordered_by_segment_size_or_dropped():
    torch.manual_seed(4)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))         # sizes 128, 16, 64, 4: all different
    params = list(model.parameters())
    for p in params:
        p.grad = torch.randn_like(p) * 0.01

    def fresh():
        feedback = ErrorFeedbackState()
        hook = create_ddp_comm_hook(CompressionConfig(), strategy="all_gather", all_gather=mirrored_gather(2),
                                    error_feedback=feedback, future_factory=FakeFuture)
        return hook, feedback

    hook, feedback = fresh()
    hook(None, LayoutBucket(list(reversed(params))))                 # the saving process ended in this order
    saved = hook.state_dict()
    assert saved["residual_by_parameter"] == {} and saved["segment_numels"] == {0: [4, 64, 16, 128]}
    by_size = dict(zip([4, 64, 16, 128], feedback.get(0).split([4, 64, 16, 128])))

    hook2, feedback2 = fresh()
    hook2.load_state_dict(saved)
    hook2.holder._follow_layout(LayoutBucket(params))                # the resuming process starts in the other order
    assert torch.equal(feedback2.get(0), torch.cat([by_size[n] for n in (128, 16, 64, 4)]))

    twins = torch.nn.Sequential(torch.nn.Linear(4, 4, bias=False), torch.nn.Linear(4, 4, bias=False))   # 16 and 16
    for p in twins.parameters():
        p.grad = torch.randn_like(p) * 0.01
    hook3, feedback3 = fresh()
    hook3(None, LayoutBucket(list(twins.parameters())))
    state = hook3.state_dict()
    state["segment_numels"] = {0: [16, 16]}
    hook4, feedback4 = fresh()
    hook4.load_state_dict(state)
    hook4.holder._follow_layout(LayoutBucket(list(twins.parameters())))
    assert feedback4.get(0) is not None                               # same order: kept as it is
    hook5, feedback5 = fresh()
    state["segment_numels"] = {0: [8, 24]}
    hook5.load_state_dict(state)
    hook5.holder._follow_layout(LayoutBucket(list(twins.parameters())))
    assert feedback5.get(0) is None                                   # cannot tell whose residual is whose: dropped
