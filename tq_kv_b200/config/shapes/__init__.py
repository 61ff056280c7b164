"""Named shapes: config.json files kept as data beside this module.

Reference: src/catalog.rs:17-82 maps `name:tag` to a downloadable file; there
is no network here, so a name maps to a config.json only, to be used with the
random-weights mode.
"""
from __future__ import annotations

import json
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def shape_names() -> list[str]:
    return sorted(f[:-5] for f in os.listdir(_HERE) if f.endswith(".json"))


def named_shape(name: str) -> dict:
    path = os.path.join(_HERE, name + ".json")
    if not os.path.exists(path):
        raise KeyError(f"unknown shape '{name}' (known: {shape_names()})")
    with open(path) as f:
        return json.load(f)
