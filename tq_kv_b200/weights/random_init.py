"""The random-weights mode: from a configuration and a seed to tensors, and to
a model folder (config.json + model.safetensors) that the loader reads back.

Init rules by role: matrices and embeddings N(0, 0.02^2); biases N(0, 0.02^2);
norm scales 1 + N(0, 0.1^2).  Each tensor has a generator of its own, seeded
from (seed, tensor name), so a tensor's values do not depend on which other
tensors exist; the values do depend on the device that generates them (CPU
and CUDA generators differ).  The reference has no such mode.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Iterator

import torch

from .safetensors_io import write_safetensors

_STD = {"matrix": 0.02, "embedding": 0.02, "bias": 0.02, "norm_scale": 0.1}


def storage_dtype(name: str) -> torch.dtype:
    try:
        return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[name]
    except KeyError:
        raise ValueError(f"unsupported torch_dtype '{name}' for random weights") from None


def random_tensor(name: str, shape: tuple[int, ...], role: str, seed: int, dtype: torch.dtype, device) -> torch.Tensor:
    if role not in _STD:
        raise ValueError(f"no random-init rule for role '{role}' (tensor {name})")
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * _STD[role]
    if role == "norm_scale":
        t += 1.0
    return t.to(dtype)


def random_tensors(weight_specs, seed: int, dtype: torch.dtype, device) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (name, tensor) for `weight_specs` (objects with name, shape, role)."""
    for ws in weight_specs:
        yield ws.name, random_tensor(ws.name, tuple(ws.shape), ws.role, seed, dtype, device)


def write_model_folder(config_dict: dict, folder: str, seed: int, *, device="cpu") -> str:
    """Writes config.json and model.safetensors for `config_dict` (an
    architecture's config.json content) with random weights in the
    configuration's `torch_dtype`."""
    from ..config import spec_from_config_dict
    from ..engine.model import DecoderModel

    arch, cfg, spec = spec_from_config_dict(config_dict)
    model = DecoderModel(spec)
    specs = list(model.weight_specs().values())
    dtype = storage_dtype(config_dict.get("torch_dtype", "bfloat16"))
    os.makedirs(folder, exist_ok=True)
    full = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config_dict)
    full["architectures"] = [arch.name]          # the name the registry resolved, not the config class's own
    full["model_type"] = arch.model_type
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(full, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(ws.name, dtype, tuple(ws.shape)) for ws in specs],
                      random_tensors(specs, seed, dtype, device),
                      metadata={"format": "pt", "seed": seed})
    return folder
