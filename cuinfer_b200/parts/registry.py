"""Registries from a ``kind`` string to the class that builds that part.

One table per role.  A new mixer, feed-forward, norm, position encoding or block arrangement
is added by decorating its class; nothing else in the package has to change, and no part
looks at which model it is in.
"""
from __future__ import annotations

from typing import Callable, Dict, TypeVar

T = TypeVar("T")


class Registry:
    def __init__(self, role: str) -> None:
        self.role = role
        self._table: Dict[str, type] = {}

    def register(self, kind: str, *, replace: bool = False) -> Callable[[T], T]:
        def deco(cls: T) -> T:
            if kind in self._table and not replace:
                raise ValueError(f"{self.role} kind {kind!r} is already registered")
            self._table[kind] = cls  # type: ignore[assignment]
            return cls

        return deco

    def unregister(self, kind: str) -> None:
        self._table.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._table[kind]
        except KeyError:
            known = ", ".join(sorted(self._table)) or "(none)"
            raise KeyError(f"unknown {self.role} kind {kind!r}; registered: {known}") from None

    def kinds(self) -> list[str]:
        return sorted(self._table)

    def __contains__(self, kind: str) -> bool:
        return kind in self._table


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
