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
    """One layer: the arrangement (`block` kind) and the parts it arranges, by
    name.  The four names that the pre-norm residual block uses are fields of
    their own; a block kind with other slots (norms after the parts, a second
    feed-forward, ...) finds them in `extra_parts` and leaves unset what it
    does not use.  Which names a layer needs is the block kind's business:
    `part(name)` raises for one that is missing."""
    block: str
    mixer: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    block_params: dict[str, Any] = field(default_factory=dict)
    extra_parts: dict[str, PartSpec] = field(default_factory=dict)

    def parts(self) -> dict[str, PartSpec]:
        """Every part the layer names, by slot name."""
        named = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "feed_forward_norm": self.feed_forward_norm,
                 "feed_forward": self.feed_forward}
        out = {k: v for k, v in named.items() if v is not None}
        for k, v in self.extra_parts.items():
            if k in out:
                raise ConfigError(f"layer names the part '{k}' twice")
            out[k] = v
        return out

    def part(self, name: str) -> PartSpec:
        try:
            return self.parts()[name]
        except KeyError:
            raise ConfigError(f"a block of kind '{self.block}' needs a part named '{name}'; "
                              f"the layer has {sorted(self.parts())}") from None


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
