"""`detect()` and `CudaCompletionManager` against a fabricated torch: the CUDA branches of both run on machines
with a GPU only, so their decisions are pinned here with fakes."""

import types

import pytest

from lowbit_comm_b200.capability import detect
from lowbit_comm_b200.core.info import ExecutionCounters, ExecutionInfo
from lowbit_comm_b200.core.work import CompletionWork
from lowbit_comm_b200.parallel.completion import CudaCompletion, CudaCompletionManager, NoopCompletion


def fake_torch(*, available=True, capability=(10, 0), devices=2):
    cuda = types.SimpleNamespace(
        is_available=lambda: available, get_device_capability=lambda *a: capability,
        device_count=lambda: devices, current_device=lambda: 0)
    return types.SimpleNamespace(__version__="2.11.0-fake", cuda=cuda)


def fake_extension(*, peers=True, arch="sm_100a"):
    return types.SimpleNamespace(ARCH=arch, can_access_peer=lambda a, b: peers or a == b)


def test_detect_reports_a_usable_b200():
    report = detect(import_torch=lambda: fake_torch(), import_extension=lambda: fake_extension())
    assert report.available and report.cuda and report.cuda_arch == "sm_100" and report.compressed_collectives
    assert report.details["peer_access"] is True and report.details["device_count"] == 2
    caps = report.to_backend_capabilities()
    assert caps.available and {"peer_memory", "ddp_hook"} <= caps.features and 8 in caps.bits
    assert report.to_dict()["torch_version"] == "2.11.0-fake"


def test_detect_explains_every_way_of_not_being_usable():
    no_cuda = detect(import_torch=lambda: fake_torch(available=False))
    assert not no_cuda.available and "CUDA is not available" in no_cuda.reason and no_cuda.ddp_hook

    def broken():
        raise ImportError("no torch here")

    assert "not importable" in detect(import_torch=broken).reason

    def no_extension():
        raise OSError("cannot open shared object")

    missing = detect(import_torch=lambda: fake_torch(), import_extension=no_extension)
    assert not missing.available and missing.cuda and "extension unavailable" in missing.reason
    hopper = detect(import_torch=lambda: fake_torch(capability=(9, 0)), import_extension=lambda: fake_extension())
    assert not hopper.available and "sm_100a" in hopper.reason and hopper.cuda_arch == "sm_90"
    lonely = detect(import_torch=lambda: fake_torch(), import_extension=lambda: fake_extension(peers=False))
    assert lonely.available and lonely.details["peer_access"] is False
    assert "peer_memory" not in lonely.to_backend_capabilities().features

    def exploding_probe():
        ext = fake_extension()
        ext.can_access_peer = lambda a, b: 1 / 0
        return ext

    shaky = detect(import_torch=lambda: fake_torch(), import_extension=exploding_probe)
    assert shaky.available and shaky.details["peer_access"] is False and any("probe failed" in w for w in shaky.warnings)


class _Event:
    log = []

    def record(self, stream):
        self.log.append(("record", stream))

    def query(self):
        return True

    def wait(self):
        self.log.append(("wait", None))

    def synchronize(self):
        self.log.append(("sync", None))


class _Stream:
    def __init__(self, name):
        self.name = name

    def wait_event(self, event):
        _Event.log.append(("stream_wait", self.name))


def _manager(native=None):
    cuda = types.SimpleNamespace(Event=_Event, current_stream=lambda device=None: _Stream("current"))
    status = types.SimpleNamespace(available=native is not None, module=native, reason=None if native else "absent")
    return CudaCompletionManager(extension_status=status, torch_provider=lambda: types.SimpleNamespace(cuda=cuda))


def test_completion_manager_records_events_and_builds_work():
    _Event.log.clear()
    manager = _manager()
    host = types.SimpleNamespace(is_cuda=False)
    assert isinstance(manager.record_for(host), NoopCompletion)
    device = types.SimpleNamespace(is_cuda=True, device="cuda:0")
    side = _Stream("side")
    completion = manager.record_for(device, side)
    assert isinstance(completion, CudaCompletion) and _Event.log[-1] == ("record", side) and completion.query()
    completion.wait_stream(_Stream("consumer"))
    completion.wait_stream(None)
    completion.synchronize()
    assert [kind for kind, _ in _Event.log[-3:]] == ["stream_wait", "wait", "sync"]
    manager.record_for(device)                                     # no stream given: the tensor's current stream
    assert _Event.log[-1][0] == "record" and _Event.log[-1][1].name == "current"

    info = ExecutionInfo(requested_strategy="a", executed_strategy="a", backend="cuda", fallback_used=False,
                         fallback_reason=None, stage_names=(), original_bytes=1, compressed_bytes=1,
                         compression_ratio=1.0, workspace_cache_hit=False, async_capable=True, fast_path="native_work")
    work = manager.create_work("value", execution_info=info, execution_counters=ExecutionCounters())
    assert isinstance(work, CompletionWork) and work.wait() == "value"
    assert work.execution_info.fast_path == "python_fallback"        # no native work type behind it
    stream_work = manager.create_stream_work(device, resources=(device,), stream=side)
    assert isinstance(stream_work, CompletionWork) and stream_work.wait() is device


def test_completion_manager_prefers_the_native_work_type():
    made = []

    class Native:
        NATIVE_WORK_ABI_VERSION = 1

        @staticmethod
        def CompressedWork(*args):
            made.append(args)
            return "native-work"

    assert _manager(Native).create_work("v", resources=(1, 2)) == "native-work" and made[0][0] == "v"
    stale = type("Old", (), {"NATIVE_WORK_ABI_VERSION": 0})
    assert isinstance(_manager(stale).create_work("v"), CompletionWork)
    counted = _manager(Native).create_work("v", execution_counters=ExecutionCounters())
    assert isinstance(counted, CompletionWork)                       # counters live in the Python work object
