"""Error-feedback residual state and the policies that gate it.

Parity: ccdl_comm/quantization/error_feedback.py:21-54 (one residual tensor per
bucket key, bucket shape and dtype) and error_feedback_policy.py:9-63 (five
policies).  Additions: persistent residual buffers that fused kernels update in
place (`residual_for`) and `state_dict`/`load_state_dict` for bit-exact resume.
"""

from __future__ import annotations

from collections.abc import Hashable
from typing import Any, NamedTuple

from ..config import CompressionConfig


class ErrorFeedbackState:
    def __init__(self) -> None:
        self._residuals: dict[Hashable, Any] = {}

    def compensate(self, key: Hashable, tensor: Any) -> Any:
        """`tensor + residual[key]`; a residual of another shape is dropped."""

        stored = self._residuals.get(key)
        if stored is None:
            return tensor
        a, b = getattr(tensor, "shape", None), getattr(stored, "shape", None)
        if a is not None and b is not None and tuple(a) != tuple(b):
            self.clear(key)
            return tensor
        return tensor + stored

    def update(self, key: Hashable, *, original: Any, transmitted: Any) -> None:
        delta = original - transmitted
        delta = delta.detach() if hasattr(delta, "detach") else delta
        self._residuals[key] = delta.clone() if hasattr(delta, "clone") else delta

    def get(self, key: Hashable) -> Any | None:
        return self._residuals.get(key)

    def set(self, key: Hashable, residual: Any) -> None:
        self._residuals[key] = residual

    def residual_for(self, key: Hashable, like: Any) -> Any:
        """Persistent zero-initialised residual shaped like `like` (created once)."""

        stored = self._residuals.get(key)
        if stored is None or tuple(stored.shape) != tuple(like.shape) or stored.dtype != like.dtype \
                or stored.device != like.device:
            import torch

            stored = torch.zeros_like(like)
            self._residuals[key] = stored
        return stored

    def clear(self, key: Hashable | None = None) -> None:
        if key is None:
            self._residuals.clear()
        else:
            self._residuals.pop(key, None)

    def keys(self):
        return self._residuals.keys()

    def state_dict(self) -> dict:
        return {"residuals": {k: (v.detach().clone() if hasattr(v, "detach") else v)
                              for k, v in self._residuals.items()}}

    def load_state_dict(self, state: dict) -> None:
        self._residuals = {k: (v.clone() if hasattr(v, "clone") else v) for k, v in state["residuals"].items()}


class ErrorFeedbackDecision(NamedTuple):
    apply: bool
    update: bool
    reason: str


class ErrorFeedbackPolicy:
    """Per-key step counters plus the rule that turns them into decisions."""

    def __init__(self, config: CompressionConfig) -> None:
        self.config = config
        self._steps: dict[Hashable, int] = {}

    def decide(self, key: Hashable, *, numel: int) -> ErrorFeedbackDecision:
        cfg = self.config
        policy = cfg.effective_error_feedback_policy()
        step = self._steps.get(key, 0)
        if policy == "none":
            return ErrorFeedbackDecision(False, False, "error feedback disabled")
        if policy == "always":
            return ErrorFeedbackDecision(True, True, "error feedback policy always")
        if policy == "large_bucket_only":
            limit = cfg.error_feedback_min_numel
            big = numel >= limit
            verb = "reached" if big else "below"
            return ErrorFeedbackDecision(big, big, f"bucket numel {numel} {verb} error feedback threshold {limit}")
        if policy == "warmup_then_enable":
            warm = cfg.error_feedback_warmup_steps
            on = step >= warm
            verb = "reached" if on else "before"
            return ErrorFeedbackDecision(on, on, f"bucket step {step} {verb} error feedback warmup {warm}")
        if policy == "periodic":
            period = cfg.error_feedback_period
            refresh = step % period == 0
            text = (f"bucket step {step} updates error feedback every {period} steps" if refresh
                    else f"bucket step {step} skips error feedback update until period {period}")
            return ErrorFeedbackDecision(True, refresh, text)
        raise ValueError(f"unsupported error feedback policy: {policy}")

    def advance(self, key: Hashable) -> None:
        self._steps[key] = self._steps.get(key, 0) + 1

    def state_dict(self) -> dict:
        return {"steps": dict(self._steps)}

    def load_state_dict(self, state: dict) -> None:
        self._steps = dict(state["steps"])
