"""Registries of part kinds and block kinds.  `make_part(spec)` builds the
implementation that `spec.kind` names; a new mixer, feed-forward, norm,
position encoding or block becomes available to every architecture by one
`register_part` / `register_block` call."""
from __future__ import annotations

from typing import Callable

from ..config import ConfigError, LayerSpec, PartSpec

_PARTS: dict[str, Callable] = {}
_BLOCKS: dict[str, Callable] = {}


def register_part(kind: str, factory: Callable, *, replace: bool = False) -> None:
    if kind in _PARTS and not replace:
        raise ValueError(f"part kind '{kind}' is already registered")
    _PARTS[kind] = factory


def unregister_part(kind: str) -> None:
    _PARTS.pop(kind, None)


def register_block(kind: str, factory: Callable, *, replace: bool = False) -> None:
    if kind in _BLOCKS and not replace:
        raise ValueError(f"block kind '{kind}' is already registered")
    _BLOCKS[kind] = factory


def part_kinds() -> list[str]:
    return sorted(_PARTS)


def make_part(spec: PartSpec):
    try:
        factory = _PARTS[spec.kind]
    except KeyError:
        raise ConfigError(f"no part of kind '{spec.kind}' is registered (known: {part_kinds()})") from None
    return factory(spec)


def make_block(spec: LayerSpec):
    try:
        factory = _BLOCKS[spec.block]
    except KeyError:
        raise ConfigError(f"no block of kind '{spec.block}' is registered (known: {sorted(_BLOCKS)})") from None
    return factory(spec)
