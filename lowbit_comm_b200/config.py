"""User compression policy.

Parity target: ccdl_comm/config.py:21-77 (same 15 fields, defaults and
validation rules).  The policy object is frozen and hashable so that it can be
part of compile-cache keys.
"""

from __future__ import annotations

from dataclasses import dataclass, fields

BITS = (4, 8)
STABLE_BITS = (8,)
GROUP_SIZES = (16, 32, 64)
TOPK_CHOICES = (0, 1, 2)
QUANT_TYPES = ("linear", "normal", "uniform", "e3m0", "e2m1")
TARGETS = ("tensor", "ddp_gradient_bucket", "collective", "p2p")
EF_POLICIES = ("none", "always", "large_bucket_only", "warmup_then_enable", "periodic")

_MEMBERSHIP = {
    "bit": BITS,
    "group_size": GROUP_SIZES,
    "topk": TOPK_CHOICES,
    "quant_type": QUANT_TYPES,
    "target": TARGETS,
    "error_feedback_policy": EF_POLICIES,
}


@dataclass(frozen=True)
class CompressionConfig:
    """How a tensor is compressed before it crosses NVLink.

    The default (linear int8, 64-element groups, no top-k, error feedback on)
    is the production profile that the fused sm_100a collectives implement;
    other combinations run through the general codec kernels.
    """

    bit: int = 8
    group_size: int = 64
    topk: int = 0
    quant_type: str = "linear"
    stochastic: bool = False
    error_feedback: bool = True
    target: str = "tensor"
    warmup_steps: int = 0
    fallback: str = "bf16_compress"
    allow_experimental: bool = False
    compact: bool = False
    error_feedback_policy: str = "always"
    error_feedback_min_numel: int = 0
    error_feedback_warmup_steps: int = 0
    error_feedback_period: int = 1

    def __post_init__(self) -> None:
        for name, allowed in _MEMBERSHIP.items():
            value = getattr(self, name)
            if value not in allowed:
                raise ValueError(f"Unsupported {name}={value!r}; expected one of {sorted(allowed)}")
        if self.bit not in STABLE_BITS and not self.allow_experimental:
            raise ValueError(f"bit={self.bit} is experimental; set allow_experimental=True to opt in")
        if self.error_feedback_min_numel < 0:
            raise ValueError("error_feedback_min_numel must be >= 0")
        if self.error_feedback_warmup_steps < 0:
            raise ValueError("error_feedback_warmup_steps must be >= 0")
        if self.error_feedback_period <= 0:
            raise ValueError("error_feedback_period must be > 0")

    def effective_error_feedback_policy(self) -> str:
        """Policy name after applying the `error_feedback` master switch."""

        return self.error_feedback_policy if self.error_feedback else "none"

    # -- helpers that the reference does not have ---------------------------
    @property
    def is_production_profile(self) -> bool:
        """True for the profile served by the fused peer-memory kernels."""

        return self.bit == 8 and self.topk == 0 and self.quant_type == "linear" and not self.stochastic

    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, values: dict) -> "CompressionConfig":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in dict(values).items() if k in known})
