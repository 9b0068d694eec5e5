"""Tiny validation helpers shared by the torch-free control plane."""

from __future__ import annotations


def need_text(value: object, what: str) -> str:
    if not isinstance(value, str) or not value.strip():
        raise ValueError(f"{what} must be a non-empty string")
    return value


def is_plain_int(value: object) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def need_shape(shape, what: str = "shape") -> tuple[int, ...]:
    dims = tuple(shape)
    if any(not is_plain_int(d) or d < 0 for d in dims):
        raise ValueError(f"{what} dimensions must be non-negative integers")
    return dims


def need_optional_index(value, bound, what: str, bound_name: str) -> None:
    if value is None:
        return
    if value < 0:
        raise ValueError(f"{what} must be >= 0")
    if bound is not None and value >= bound:
        raise ValueError(f"{what} must be < {bound_name}")
