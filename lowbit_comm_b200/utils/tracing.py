"""Optional NVTX ranges and a tiny phase timer (off unless LBC_TRACE=1).

The reference has no tracing layer (its design document lists NVTX as a duty of
the CUDA backend, docs/SOFTWARE_DESIGN_ZH.md:319-328, without implementing it).
"""

from __future__ import annotations

import contextlib
import os
from collections import defaultdict

ENABLED = os.environ.get("LBC_TRACE", "0") not in ("", "0", "false", "False")


@contextlib.contextmanager
def nvtx_range(name: str):
    if not ENABLED:
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Records CUDA events between phases of a collective; `summary()` synchronises and reports ms."""

    def __init__(self) -> None:
        self._marks: list[tuple[str, object]] = []
        self.totals: dict[str, list[float]] = defaultdict(list)

    def mark(self, name: str, stream=None) -> None:
        import torch

        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream or torch.cuda.current_stream())
        self._marks.append((name, ev))

    def flush(self) -> None:
        if len(self._marks) < 2:
            self._marks.clear()
            return
        self._marks[-1][1].synchronize()
        for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:]):
            self.totals[name].append(a.elapsed_time(b))
        self._marks.clear()

    def summary(self) -> dict[str, float]:
        import statistics

        return {k: statistics.median(v) for k, v in self.totals.items() if v}


def kernel_names(fn, *, torch_module=None) -> dict[str, int]:
    """Runs `fn()` once under `torch.profiler` and returns {CUDA kernel name: launches}.

    Evidence, not measurement: benchmark records use it to show which kernels served an operation (the
    reference does the same with `profile.key_averages()`, tests/distributed/fused_reduced_shard_perf.py:
    244-274).  Never time anything inside this call.  On a machine without CUDA the result is empty.
    """

    torch = torch_module
    if torch is None:
        import torch
    profiler = torch.profiler
    activities = [profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        activities.append(profiler.ProfilerActivity.CUDA)
    with profiler.profile(activities=activities) as prof:
        fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    counts: dict[str, int] = {}
    for event in prof.events():
        device = getattr(event, "device_type", None)
        if device is not None and "cuda" in str(device).lower():
            counts[event.name] = counts.get(event.name, 0) + 1
    return counts
