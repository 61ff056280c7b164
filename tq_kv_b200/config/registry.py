"""The one registry from an architecture's name to its model.

An entry holds the typed configuration class that reads the architecture's
config.json and the builder that turns a configuration into a `ModelSpec`.
`resolve()` picks the entry from config.json's `architectures[0]` (or, failing
that, from `model_type`).  Adding an architecture = one `register_architecture`
call; nothing else in the package names an architecture.

Reference: the engine has no dispatch by class name (src/engine.rs:234 ignores
its `_arch`; src/models/turbo_generic.rs:2028-2029 uses `model_type` only to
pick the rotary layout); src/catalog.rs:17-82 maps model names to files.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_spec import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: Any                      # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve(config_dict: dict) -> Architecture:
    """The registry entry for a config.json (given as a dict)."""
    names = config_dict.get("architectures")
    if isinstance(names, list) and names:
        name = names[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(
            f"config.json: architecture '{name}' is not registered (registered: {registered_architectures()})")
    mt = config_dict.get("model_type")
    for arch in _ARCHITECTURES.values():
        if mt is not None and arch.model_type == mt:
            return arch
    raise ConfigError(
        "config.json: neither 'architectures' nor a known 'model_type' is given "
        f"(registered: {registered_architectures()})")


def spec_from_config_dict(config_dict: dict) -> tuple[Architecture, Any, ModelSpec]:
    arch = resolve(config_dict)
    cfg = arch.config_class.from_dict(config_dict)
    return arch, cfg, arch.build_spec(cfg)
