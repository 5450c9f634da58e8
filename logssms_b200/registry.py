"""Name -> object registries.

Every pluggable kind of thing in the engine (architectures, mixers, feed-forwards,
norms, position encodings, blocks, embeddings, output heads) lives in one `Registry`.  A test or a user
package adds an entry with `registry.register("name")(cls)`; nothing inside the
framework has to change.  The same shape as the reference's `Registry[T]`
(python/logssms/utils/registry.py:5-37) and its architecture table
(python/logssms/models/register.py:7-17).
"""
from __future__ import annotations

from typing import Callable, Generic, Iterator, TypeVar

T = TypeVar("T")


class Registry(Generic[T]):
    def __init__(self, kind: str):
        self.kind = kind
        self._entries: dict[str, T] = {}

    def register(self, name: str, *, replace: bool = False) -> Callable[[T], T]:
        def deco(obj: T) -> T:
            if name in self._entries and not replace:
                raise KeyError(f"{self.kind} {name!r} is already registered")
            self._entries[name] = obj
            return obj
        return deco

    def unregister(self, name: str) -> None:
        self._entries.pop(name, None)

    def get(self, name: str) -> T:
        try:
            return self._entries[name]
        except KeyError:
            raise ValueError(
                f"{self.kind} {name} not supported; known: {sorted(self._entries)}"
            ) from None

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def names(self) -> list[str]:
        return sorted(self._entries)

    def __iter__(self) -> Iterator[str]:
        return iter(self.names())


ARCHITECTURES: Registry = Registry("Model architecture")
MIXERS: Registry = Registry("Mixer")
FEED_FORWARDS: Registry = Registry("Feed-forward")
NORMS: Registry = Registry("Norm")
POSITION_ENCODINGS: Registry = Registry("Position encoding")
BLOCKS: Registry = Registry("Block")
EMBEDDINGS: Registry = Registry("Embedding")
HEADS: Registry = Registry("Output head")
