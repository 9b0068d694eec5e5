"""ParaScale-facing planner adapter (parity: ccdl_comm/plugin.py:9-49)."""

from __future__ import annotations

from collections.abc import Mapping
from typing import NamedTuple

from .config import CompressionConfig


class PluginDecision(NamedTuple):
    enabled: bool
    fallback: str | None
    reason: str


_REQUIREMENTS = (
    ("training_backend", "native_ddp", "CCDL only supports training_backend='native_ddp'"),
    ("device_type", "cuda", "CCDL only supports CUDA execution (sm_100a peer memory or NCCL)"),
)


class CCDLCommunicationPlugin:
    """Answers "should gradient-bucket compression be switched on here?"."""

    name = "ccdl"

    def plan(self, context: Mapping[str, object], config: CompressionConfig) -> PluginDecision:
        for key, wanted, why in _REQUIREMENTS:
            if context.get(key) != wanted:
                return PluginDecision(False, config.fallback, why)
        return PluginDecision(True, None, "CCDL can be enabled for native_ddp CUDA gradient-bucket compression")

    def explain(self, config: CompressionConfig) -> list[str]:
        return [
            "CCDL compresses native DDP gradient buckets inside fused NVLink peer-memory collectives.",
            f"It will use {config.bit}-bit {config.quant_type} quantization with group_size={config.group_size}.",
            "Training orchestration, backend selection, fallback and benchmark decisions stay with the host planner.",
        ]
