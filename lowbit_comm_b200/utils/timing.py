"""Device-side timing helpers (CUDA events, L2 flush, max over ranks)."""

from __future__ import annotations

import statistics
from typing import Callable

import torch

L2_BYTES = 126 * 1024 * 1024


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""

    def __init__(self, device=None, nbytes: int = 2 * L2_BYTES) -> None:
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")

    def __call__(self) -> None:
        self.buf.fill_(1)


def time_cuda(fn: Callable[[], None], *, warmup: int = 3, iters: int = 10, flush: L2Flusher | None = None,
              stream: torch.cuda.Stream | None = None) -> dict:
    """Median / min / mean milliseconds of `fn`, each call bracketed by CUDA events."""

    stream = stream or torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iters):
        if flush is not None:
            flush()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        fn()
        stop.record(stream)
        stop.synchronize()
        samples.append(start.elapsed_time(stop))
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "mean_ms": statistics.fmean(samples), "samples": len(samples)}


def max_over_ranks(value: float, group=None) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
