"""Versioned benchmark result records.

Parity: tests/benchmarks/result_schema.py:13-109 of the reference (field list,
rejection of `commit == "unknown"`, identity from environment variables
`CCDL_BENCHMARK_COMMIT` / `CCDL_BENCHMARK_HOSTNAME`).  Additions: device-timed
flag, roofline fraction and per-phase timings.
"""

from __future__ import annotations

import math
import os
import socket
import subprocess
from dataclasses import asdict, dataclass, field

SCHEMA_VERSION = 2
REQUIRED = ("commit", "hostname", "gpu_name", "cuda_version", "torch_version", "world_size", "dtype", "numel",
            "strategy", "latency_ms", "effective_gbps", "peak_memory_bytes", "relative_l2", "max_abs_error", "rmse",
            "non_finite")


@dataclass(frozen=True)
class BenchmarkResult:
    commit: str
    hostname: str
    gpu_name: str
    cuda_version: str
    torch_version: str
    world_size: int
    dtype: str
    numel: int
    strategy: str
    latency_ms: float
    effective_gbps: float
    peak_memory_bytes: int
    relative_l2: float
    max_abs_error: float
    rmse: float
    non_finite: bool
    device_timed: bool = True
    roofline_fraction: float | None = None
    phases_ms: dict = field(default_factory=dict)
    schema_version: int = SCHEMA_VERSION

    def __post_init__(self) -> None:
        validate_result(asdict(self))

    def to_dict(self) -> dict:
        return asdict(self)


def validate_result(record: dict) -> dict:
    missing = [k for k in REQUIRED if k not in record]
    if missing:
        raise ValueError(f"benchmark result is missing fields: {missing}")
    if not record["commit"] or record["commit"] == "unknown":
        raise ValueError("benchmark result needs a real commit id (set CCDL_BENCHMARK_COMMIT)")
    if int(record["world_size"]) < 1 or int(record["numel"]) < 0:
        raise ValueError("world_size must be >= 1 and numel >= 0")
    for key in ("latency_ms", "effective_gbps"):
        value = float(record[key])
        if not math.isfinite(value) or value <= 0:
            raise ValueError(f"{key} must be finite and > 0")
    for key in ("relative_l2", "max_abs_error", "rmse"):
        if float(record[key]) < 0:
            raise ValueError(f"{key} must be >= 0")
    return record


def benchmark_identity(cwd: str | None = None) -> dict:
    commit = os.environ.get("CCDL_BENCHMARK_COMMIT", "")
    if not commit:
        try:
            commit = subprocess.run(["git", "rev-parse", "HEAD"], cwd=cwd, capture_output=True, text=True,
                                    timeout=10).stdout.strip()
        except (OSError, subprocess.SubprocessError):
            commit = ""
    return {"commit": commit or "unknown",
            "hostname": os.environ.get("CCDL_BENCHMARK_HOSTNAME") or socket.gethostname()}


def effective_gbps(numel: int, element_bytes: int, latency_ms: float) -> float:
    """Logical tensor bytes / latency, the reference's `effective_gbps` definition."""

    return numel * element_bytes / (latency_ms * 1e-3) / 1e9
