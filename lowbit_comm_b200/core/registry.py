"""Where backends announce themselves: factories under a four-part key, strategy selectors under a backend name.

Both tables are write-once (`_WriteOnce`): a second registration under the same key is a programming error and
is reported as `BackendRegistrationError`, never silently replaced.  Nothing here is touched per collective
call; the compiler consults the registry once per compile.  The public names and their behaviour follow the
reference (ccdl_comm/registry.py:13-85); `provides`, `strategies_for` and `nearest` are additions used by the
compiler's diagnostics.
"""

from __future__ import annotations

from collections.abc import Callable, Iterator
from typing import Generic, NamedTuple, TypeVar

from ..exceptions import BackendRegistrationError, UnsupportedCollective
from ._checks import need_text
from .backend import AutoStrategySelector, CommunicationBackend

K = TypeVar("K")
V = TypeVar("V")


class BackendKey(NamedTuple):
    collective: str
    strategy: str
    backend: str
    output_layout: str

    @classmethod
    def checked(cls, collective: str, strategy: str, backend: str, output_layout: str) -> "BackendKey":
        key = cls(collective, strategy, backend, output_layout)
        for name, value in zip(cls._fields, key):
            need_text(value, name)
        return key

    def distance(self, other: "BackendKey") -> int:
        """In how many of the four parts two keys differ."""

        return sum(mine != theirs for mine, theirs in zip(self, other))

    def __str__(self) -> str:
        return ":".join(self)


class _WriteOnce(Generic[K, V]):
    """Insertion-ordered map whose entries are callables and can be set exactly once."""

    def __init__(self, duplicate_message: Callable[[K], str], entry_name: str) -> None:
        self._entries: dict[K, V] = {}
        self._duplicate_message = duplicate_message
        self._entry_name = entry_name

    def put(self, key: K, entry: V) -> None:
        if not callable(entry):
            raise TypeError(f"{self._entry_name} must be callable")
        if key in self._entries:
            raise BackendRegistrationError(self._duplicate_message(key))
        self._entries[key] = entry

    def get(self, key: K) -> V | None:
        return self._entries.get(key)

    def __contains__(self, key: object) -> bool:
        return key in self._entries

    def __iter__(self) -> Iterator[K]:
        return iter(self._entries)


class BackendRegistry:
    def __init__(self) -> None:
        self._factories: _WriteOnce[BackendKey, Callable[[], CommunicationBackend]] = _WriteOnce(
            lambda key: f"backend key already registered: {key}", "factory")
        self._selectors: _WriteOnce[str, AutoStrategySelector] = _WriteOnce(
            lambda name: f"strategy selector already registered for backend {name!r}", "selector")

    # -- backend factories ------------------------------------------------------------------------
    def register(self, key: BackendKey, factory: Callable[[], CommunicationBackend]) -> None:
        if not isinstance(key, BackendKey):
            raise TypeError("key must be a BackendKey")
        self._factories.put(BackendKey.checked(*key), factory)

    def provides(self, *, collective: str, strategy: str, backend: str, output_layout: str):
        """Decorator form of `register` for a backend class or a zero-argument factory function."""

        def remember(factory):
            self.register(BackendKey(collective, strategy, backend, output_layout), factory)
            return factory

        return remember

    def resolve(self, key: BackendKey) -> CommunicationBackend:
        make = self._factories.get(key)
        if make is None:
            raise UnsupportedCollective(str(key), reason="no backend factory is registered for the requested key")
        made = make()
        if isinstance(made, CommunicationBackend):
            return made
        raise BackendRegistrationError(f"factory for {key} did not return a CommunicationBackend")

    def keys(self) -> tuple[BackendKey, ...]:
        return tuple(self._factories)

    def strategies_for(self, collective: str, backend: str, output_layout: str) -> set[str]:
        wanted = (collective, backend, output_layout)
        return {k.strategy for k in self._factories if (k.collective, k.backend, k.output_layout) == wanted}

    def nearest(self, key: BackendKey, limit: int = 3) -> tuple[BackendKey, ...]:
        """Registered keys that differ from `key` in the fewest parts (for "did you mean" diagnostics)."""

        ranked = sorted(self._factories, key=key.distance)
        return tuple(k for k in ranked[:limit] if key.distance(k) < len(BackendKey._fields))

    def __contains__(self, key: object) -> bool:
        return key in self._factories

    # -- automatic strategy selectors -------------------------------------------------------------
    def register_strategy_selector(self, backend: str, selector: AutoStrategySelector) -> None:
        self._selectors.put(need_text(backend, "backend"), selector)

    def strategy_selector(self, backend: str) -> AutoStrategySelector | None:
        return self._selectors.get(need_text(backend, "backend"))
