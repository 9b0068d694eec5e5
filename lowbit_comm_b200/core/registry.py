"""Registry of backend factories keyed by (collective, strategy, backend, layout).

Parity: ccdl_comm/registry.py:13-85.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import NamedTuple

from ..exceptions import BackendRegistrationError, UnsupportedCollective
from ._checks import need_text
from .backend import AutoStrategySelector, CommunicationBackend


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

    def __str__(self) -> str:
        return ":".join(self)


class BackendRegistry:
    def __init__(self) -> None:
        self._factories: dict[BackendKey, Callable[[], CommunicationBackend]] = {}
        self._selectors: dict[str, AutoStrategySelector] = {}

    def register(self, key: BackendKey, factory: Callable[[], CommunicationBackend]) -> None:
        if not isinstance(key, BackendKey):
            raise TypeError("key must be a BackendKey")
        BackendKey.checked(*key)
        if not callable(factory):
            raise TypeError("factory must be callable")
        if key in self._factories:
            raise BackendRegistrationError(f"backend key already registered: {key}")
        self._factories[key] = factory

    def resolve(self, key: BackendKey) -> CommunicationBackend:
        factory = self._factories.get(key)
        if factory is None:
            raise UnsupportedCollective(str(key), reason="no backend factory is registered for the requested key")
        backend = factory()
        if not isinstance(backend, CommunicationBackend):
            raise BackendRegistrationError(f"factory for {key} did not return a CommunicationBackend")
        return backend

    def register_strategy_selector(self, backend: str, selector: AutoStrategySelector) -> None:
        need_text(backend, "backend")
        if not callable(selector):
            raise TypeError("selector must be callable")
        if backend in self._selectors:
            raise BackendRegistrationError(f"strategy selector already registered for backend {backend!r}")
        self._selectors[backend] = selector

    def strategy_selector(self, backend: str) -> AutoStrategySelector | None:
        need_text(backend, "backend")
        return self._selectors.get(backend)

    def strategies_for(self, collective: str, backend: str, output_layout: str) -> set[str]:
        return {k.strategy for k in self._factories
                if (k.collective, k.backend, k.output_layout) == (collective, backend, output_layout)}

    def keys(self) -> tuple[BackendKey, ...]:
        return tuple(self._factories)

    def __contains__(self, key: object) -> bool:
        return key in self._factories
