"""Validation vocabulary of the torch-free control plane.

The dataclasses of `core/` describe their invariants with these helpers instead of spelling out `if` chains;
every helper raises the exception a caller of the public API sees.
"""

from __future__ import annotations

from collections.abc import Iterable
from types import MappingProxyType
from typing import Any


def need_text(value: object, what: str) -> str:
    if not isinstance(value, str) or not value.strip():
        raise ValueError(f"{what} must be a non-empty string")
    return value


def need_texts(owner: object, *names: str) -> None:
    """`need_text` for several attributes of a (frozen) dataclass instance."""

    for name in names:
        need_text(getattr(owner, name), name)


def is_plain_int(value: object) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def need_shape(shape, what: str = "shape") -> tuple[int, ...]:
    dims = tuple(shape)
    if any(not is_plain_int(d) or d < 0 for d in dims):
        raise ValueError(f"{what} dimensions must be non-negative integers")
    return dims


def need_optional_index(value, bound, what: str, bound_name: str) -> None:
    """None, or 0 <= value (< bound when a bound is known)."""

    if value is None:
        return
    if value < 0:
        raise ValueError(f"{what} must be >= 0")
    if bound is not None and value >= bound:
        raise ValueError(f"{what} must be < {bound_name}")


def need_optional_minimum(value, minimum: int, what: str) -> None:
    """None, or value >= minimum (the message says `> minimum - 1` for a minimum of one: "must be > 0")."""

    if value is not None and value < minimum:
        raise ValueError(f"{what} must be > 0" if minimum == 1 else f"{what} must be >= {minimum}")


def text_set(values: Iterable[Any], what: str) -> frozenset[str]:
    frozen = frozenset(values)
    if any(not isinstance(v, str) or not v.strip() for v in frozen):
        raise ValueError(f"{what} must contain non-empty strings")
    return frozen


def text_tuple(values: Iterable[Any], what: str, *, message: str | None = None) -> tuple[str, ...]:
    items = tuple(values)
    if any(not isinstance(v, str) or not v.strip() for v in items):
        raise ValueError(message or f"{what} must contain non-empty strings")
    return items


def freeze(owner: object, **values: Any) -> None:
    """Assign normalised values to a frozen dataclass instance from inside `__post_init__`."""

    for name, value in values.items():
        object.__setattr__(owner, name, value)


def read_only(mapping) -> MappingProxyType:
    return MappingProxyType(dict(mapping))
