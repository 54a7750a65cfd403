"""One registry per family of parts: a kind name to the class that builds it.

The reference extends itself by ``RegisterArchitecture`` (models/llm/arch.go:60-64);
here every family can be extended the same way, from outside the package, so a
new mixer, feed-forward, norm, position encoding or block arrangement needs no
change to the framework's files.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

from ..config.spec import PartSpec


class PartRegistry:
    def __init__(self, family: str):
        self.family = family
        self._kinds: Dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
        if kind in self._kinds and not replace:
            raise ValueError(f"{self.family} kind {kind!r} is already registered")
        self._kinds[kind] = factory

    def kinds(self) -> list[str]:
        return sorted(self._kinds)

    def build(self, spec: PartSpec) -> Any:
        try:
            factory = self._kinds[spec.kind]
        except KeyError:
            raise KeyError(
                f"unknown {self.family} kind {spec.kind!r}; registered: {', '.join(self.kinds()) or '(none)'}"
            ) from None
        return factory(**dict(spec.params))


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
BLOCKS = PartRegistry("block")
EMBEDDINGS = PartRegistry("embedding")
HEADS = PartRegistry("head")


def register_mixer(kind: str, factory: Callable[..., Any], **kw: Any) -> None:
    MIXERS.register(kind, factory, **kw)


def register_feed_forward(kind: str, factory: Callable[..., Any], **kw: Any) -> None:
    FEED_FORWARDS.register(kind, factory, **kw)


def register_norm(kind: str, factory: Callable[..., Any], **kw: Any) -> None:
    NORMS.register(kind, factory, **kw)


def register_position_encoding(kind: str, factory: Callable[..., Any], **kw: Any) -> None:
    POSITION_ENCODINGS.register(kind, factory, **kw)


def register_block(kind: str, factory: Callable[..., Any], **kw: Any) -> None:
    BLOCKS.register(kind, factory, **kw)
