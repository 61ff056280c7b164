"""The random-weights mode: from a configuration and a seed to tensors, and to
a model folder (config.json + model.safetensors) that the loader reads back.

Init rules by role: matrices and embeddings N(0, 0.02^2); biases N(0, 0.02^2);
norm scales 1 + N(0, 0.1^2).  The generator is counter-based: element i of a
tensor depends on (seed, tensor name, i) only, so a tensor's values depend
neither on which other tensors exist nor on where they are made.  The host
twin below (numpy) and the device kernel (csrc/random_fill.cu) do the same
single IEEE float32 operations in the same order and give the same bits; a
model folder written on the CPU and an engine filled on the GPU from the same
seed therefore hold the same weights.  Values are rounded to bfloat16 once,
from float32.  The reference has no such mode.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Iterator

import numpy as np
import torch

from .safetensors_io import write_safetensors

_STD = {"matrix": 0.02, "embedding": 0.02, "bias": 0.02, "norm_scale": 0.1}
_OFFSET = {"norm_scale": 1.0}
_MASK = (1 << 64) - 1
_CHUNK = 1 << 15          # elements generated at a time on the host (stays in the cache)


def storage_dtype(name: str) -> torch.dtype:
    try:
        return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[name]
    except KeyError:
        raise ValueError(f"unsupported torch_dtype '{name}' for random weights") from None


def _mix_int(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream."""
    return _mix_int(_mix_int(int(seed) & _MASK) ^ ((zlib.crc32(name.encode()) * 0xA0761D6478BD642F) & _MASK))


def _f(x) -> np.float32:
    return np.float32(x)


_ONE = _f(1.0)
_SQRT2 = _f(float.fromhex("0x1.6a09e6p+0"))
_LN2 = _f(float.fromhex("0x1.62e43p-1"))
_QUARTER_PI = _f(float.fromhex("0x1.921fb6p-1"))
_LOG_COEF = [_ONE / _f(d) for d in (11.0, 9.0, 7.0, 5.0, 3.0)] + [_ONE]
_SIN_COEF = [_ONE / _f(362880.0), -_ONE / _f(5040.0), _ONE / _f(120.0), -_ONE / _f(6.0), _ONE]
_COS_COEF = [-_ONE / _f(3628800.0), _ONE / _f(40320.0), -_ONE / _f(720.0), _ONE / _f(24.0), _f(-0.5), _ONE]


def _horner(coef, x2: np.ndarray) -> np.ndarray:
    p = np.full_like(x2, coef[0])
    for c in coef[1:]:
        p = p * x2 + c              # two float32 roundings: numpy never fuses them
    return p


def standard_normal_host(key: int, start: int, count: int) -> np.ndarray:
    """Elements start .. start+count-1 of the stream `key` as float32; the
    same operations, in the same order, as rf_normal() in csrc/random_fill.cu."""
    with np.errstate(over="ignore"):
        i = np.arange(start, start + count, dtype=np.uint64)
        z = np.uint64(key) ^ (i * np.uint64(0xD6E8FEB86659FD93))
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    k1 = (z >> np.uint64(40)).astype(np.uint32)
    k2 = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.uint32)

    fb = (k1 + np.uint32(1)).astype(np.float32).view(np.uint32)
    e = (fb >> np.uint32(23)).astype(np.int32) - 127
    m = ((fb & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(np.float32)
    big = m > _SQRT2
    m = np.where(big, m * _f(0.5), m)
    e = np.where(big, e + 1, e)
    s = (m + _f(-1.0)) / (m + _ONE)
    ln_m = (_f(2.0) * s) * _horner(_LOG_COEF, s * s)
    ln_u = (e - 24).astype(np.float32) * _LN2 + ln_m
    radius = np.sqrt(_f(-2.0) * ln_u)

    octant = k2 >> np.uint32(21)
    r = k2 & np.uint32(0x1FFFFF)
    rr = np.where(octant & np.uint32(1), np.uint32(0x200000) - r, r)
    x = (rr.astype(np.float32) * (_ONE / _f(2097152.0))) * _QUARTER_PI
    x2 = x * x
    sn = _horner(_SIN_COEF, x2) * x
    cs = _horner(_COS_COEF, x2)
    use_sin = (octant == 1) | (octant == 2) | (octant == 5) | (octant == 6)
    c = np.where(use_sin, sn, cs)
    c = np.where((octant >= 2) & (octant <= 5), -c, c)
    out = radius * c
    assert out.dtype == np.float32
    return out


def _host_tensor(key: int, n: int, std: float, offset: float) -> torch.Tensor:
    out = np.empty(n, dtype=np.float32)
    for a in range(0, n, _CHUNK):
        c = min(_CHUNK, n - a)
        out[a:a + c] = _f(offset) + standard_normal_host(key, a, c) * _f(std)
    return torch.from_numpy(out)


def random_tensor(name: str, shape: tuple[int, ...], role: str, seed: int, dtype: torch.dtype, device) -> torch.Tensor:
    """The tensor `name` of the model seeded with `seed`, made on `device`
    (the same values on any device)."""
    if role not in _STD:
        raise ValueError(f"no random-init rule for role '{role}' (tensor {name})")
    key, std, offset = tensor_key(seed, name), _STD[role], _OFFSET.get(role, 0.0)
    n = 1
    for d in shape:
        n *= int(d)
    dev = torch.device(device)
    if dev.type == "cuda":
        from .. import kernels
        made = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        t = torch.empty(shape, dtype=made, device=dev)
        kernels.random_fill(t, key, std, offset)
        return t if made == dtype else t.to(dtype)
    return _host_tensor(key, n, std, offset).reshape(shape).to(dtype)


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
