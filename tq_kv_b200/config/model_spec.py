"""Architecture-neutral description of a decoder: which parts each layer is
made of, with which sizes, and in which order the layers run.

A typed architecture configuration (one per architecture, read from that
architecture's config.json) is turned into a `ModelSpec` by the builder that
the registry holds for the architecture's name.  Everything below the
registry (parts, cache, engine) sees only the `ModelSpec`; no part knows which
model it belongs to.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


class ConfigError(ValueError):
    """A config.json that cannot be read, lacks a key, or contradicts itself."""


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` selects the implementation in the part registry,
    `params` are its sizes and constants (all of them; a part reads nothing
    else).  `weights_prefix` is prepended to the part's own tensor names."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    weights_prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (`block` kind) and the parts it arranges."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block_params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer.  `layer` indexes `ModelSpec.layers`; a layer may be
    named by several entries (it then runs twice with the same weights).
    `cache_of` names the schedule entry whose cache this entry's mixer reads;
    None means the entry owns a cache of its own and writes to it."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: tuple[int, ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, but there are {n} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ConfigError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns no cache itself")
