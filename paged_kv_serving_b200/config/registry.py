"""Registries: architecture name -> model builder, and part kind/name -> part class.

The reference has one hard-wired model class (src/paged_kv_serving/engine/model.py:224);
here the ``architecture`` key of ``config.json`` selects the builder, and each layer of a
model names its parts, so that a test (or a later architecture) can add a mixer, a
feed-forward, a norm or a position encoding without touching the framework's files.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

__all__ = [
    "PART_KINDS", "architecture", "known_architectures", "known_parts", "part",
    "register_architecture", "register_part",
]

PART_KINDS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")

_ARCHITECTURES: dict[str, Any] = {}
_PARTS: dict[str, dict[str, Any]] = {kind: {} for kind in PART_KINDS}


def register_architecture(name: str) -> Callable[[Any], Any]:
    """Class decorator: make ``name`` in ``config.json["architecture"]`` build this class."""

    def decorate(cls: Any) -> Any:
        if name in _ARCHITECTURES and _ARCHITECTURES[name] is not cls:
            raise ValueError(f"architecture {name!r} is already registered")
        _ARCHITECTURES[name] = cls
        return cls

    return decorate


def architecture(name: str) -> Any:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ValueError(f"unknown architecture {name!r}; known architectures: {known}") from None


def known_architectures() -> tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def register_part(kind: str, name: str) -> Callable[[Any], Any]:
    """Class decorator: register a part class under ``(kind, name)``."""
    if kind not in PART_KINDS:
        raise ValueError(f"unknown part kind {kind!r}; kinds: {', '.join(PART_KINDS)}")

    def decorate(cls: Any) -> Any:
        if name in _PARTS[kind] and _PARTS[kind][name] is not cls:
            raise ValueError(f"{kind} part {name!r} is already registered")
        _PARTS[kind][name] = cls
        return cls

    return decorate


def part(kind: str, name: str) -> Any:
    _load_builtin()
    try:
        return _PARTS[kind][name]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(kind, {}))) or "(none)"
        raise ValueError(f"unknown {kind} part {name!r}; known: {known}") from None


def known_parts(kind: str) -> tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_PARTS[kind]))


def _load_builtin() -> None:
    """Import the modules whose decorators fill the registries (idempotent)."""
    import paged_kv_serving_b200.models  # noqa: F401
    import paged_kv_serving_b200.parts  # noqa: F401
