"""Registries that turn a ``PartSpec`` (kind name + parameters) into a part.

One registry per role.  Registering a new kind needs no change to any file of
the framework: call ``register_mixer("my_kind", MyMixer)`` (or the decorator
form) before the model is built, and name ``"my_kind"`` in a ``PartSpec``.
"""

from __future__ import annotations

from typing import Any, Callable

from .base import Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PartSpec, PositionEncoding


class UnknownPartError(KeyError):
    pass


class _Registry:
    def __init__(self, role: str, base: type):
        self.role = role
        self.base = base
        self._kinds: dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, factory: Callable[..., Part] | None = None):
        def _add(f: Callable[..., Part]):
            self._kinds[kind] = f
            return f
        return _add(factory) if factory is not None else _add

    def build(self, spec: PartSpec, **extra: Any) -> Part:
        try:
            factory = self._kinds[spec.kind]
        except KeyError:
            raise UnknownPartError(
                f"no {self.role} of kind {spec.kind!r} is registered; known: {sorted(self._kinds)}"
            ) from None
        part = factory(**spec.params, **extra)
        if not isinstance(part, self.base):
            raise TypeError(f"{self.role} kind {spec.kind!r} built a {type(part).__name__}, "
                            f"which is not a {self.base.__name__}")
        return part

    def kinds(self) -> list[str]:
        return sorted(self._kinds)


MIXERS = _Registry("mixer", Mixer)
FEED_FORWARDS = _Registry("feed-forward", FeedForward)
NORMS = _Registry("norm", Norm)
POSITION_ENCODINGS = _Registry("position encoding", PositionEncoding)
BLOCKS = _Registry("block", Block)
EMBEDDINGS = _Registry("embedding", Embedding)
HEADS = _Registry("output head", Head)

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
