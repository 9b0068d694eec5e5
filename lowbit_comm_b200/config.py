"""User compression policy.

`CompressionConfig` has the reference's 15 fields, defaults and validation rules (ccdl_comm/config.py:21-77).
It is frozen and hashable so that it can be part of compile-cache keys.  Validation is table-driven: a field
is either a member of a closed set (`_CHOICES`) or an integer with a lower bound (`_AT_LEAST`).  Additions:
named profiles (`production`, `int4`), `evolve`, `describe`, `max_code`, and dict round-tripping.
"""

from __future__ import annotations

from dataclasses import dataclass, fields, replace

BITS = (4, 8)
STABLE_BITS = (8,)
GROUP_SIZES = (16, 32, 64)
TOPK_CHOICES = (0, 1, 2)
QUANT_TYPES = ("linear", "normal", "uniform", "e3m0", "e2m1")
TARGETS = ("tensor", "ddp_gradient_bucket", "collective", "p2p")
EF_POLICIES = ("none", "always", "large_bucket_only", "warmup_then_enable", "periodic")

_CHOICES = {"bit": BITS, "group_size": GROUP_SIZES, "topk": TOPK_CHOICES, "quant_type": QUANT_TYPES,
            "target": TARGETS, "error_feedback_policy": EF_POLICIES}
_AT_LEAST = {"error_feedback_min_numel": 0, "error_feedback_warmup_steps": 0, "error_feedback_period": 1}


@dataclass(frozen=True)
class CompressionConfig:
    """How a tensor is compressed before it crosses NVLink.

    The default (linear int8, 64-element groups, no top-k, error feedback on) is the production profile that
    the fused sm_100a collectives implement; other combinations run through the general codec kernels.
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
        for name, allowed in _CHOICES.items():
            value = getattr(self, name)
            if value not in allowed:
                raise ValueError(f"Unsupported {name}={value!r}; expected one of {sorted(allowed)}")
        if self.bit not in STABLE_BITS and not self.allow_experimental:
            raise ValueError(f"bit={self.bit} is experimental; set allow_experimental=True to opt in")
        for name, minimum in _AT_LEAST.items():
            if getattr(self, name) < minimum:
                raise ValueError(f"{name} must be " + (">= 0" if minimum == 0 else f"> {minimum - 1}"))

    # -- named profiles -----------------------------------------------------------------------------
    @classmethod
    def production(cls, **changes) -> "CompressionConfig":
        """Linear int8, 64-element groups, error feedback on: what the fused peer-memory kernels serve."""

        return cls(**changes)

    @classmethod
    def int4(cls, quant_type: str = "linear", **changes) -> "CompressionConfig":
        """A 4-bit profile (opted in to experimental); `quant_type` selects linear codes or a code-book."""

        return cls(bit=4, quant_type=quant_type, allow_experimental=True, **changes)

    def evolve(self, **changes) -> "CompressionConfig":
        """A validated copy with some fields changed."""

        return replace(self, **changes)

    # -- derived facts ------------------------------------------------------------------------------
    def effective_error_feedback_policy(self) -> str:
        """Policy name after applying the `error_feedback` master switch."""

        return self.error_feedback_policy if self.error_feedback else "none"

    @property
    def is_production_profile(self) -> bool:
        """True for the profile served by the fused peer-memory kernels."""

        return self.bit == 8 and self.topk == 0 and self.quant_type == "linear" and not self.stochastic

    @property
    def max_code(self) -> int:
        """Largest magnitude of a linear code: the group's abs-max maps to this value."""

        return (1 << (self.bit - 1)) - 1

    def describe(self) -> str:
        """Short label for logs and benchmark tables, e.g. `int8 g64 linear ef=always`."""

        words = [f"int{self.bit}", f"g{self.group_size}", self.quant_type]
        if self.topk:
            words.append(f"top{self.topk}")
        words += [name for name in ("stochastic", "compact") if getattr(self, name)]
        words.append(f"ef={self.effective_error_feedback_policy()}")
        return " ".join(words)

    # -- dict round trip ----------------------------------------------------------------------------
    def to_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, values: dict) -> "CompressionConfig":
        """Unknown keys are ignored, so a dict written by a newer version still loads."""

        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in dict(values).items() if k in known})
