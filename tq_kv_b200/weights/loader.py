"""Loading a model folder's tensors by name.

The model says which tensors it expects (name, shape); the loader compares
that list with what the safetensors files hold and raises ONE error that
lists every missing tensor, every unexpected tensor and every wrong shape.
Then it copies the tensors to the device under this dtype policy:
  serving (bfloat16):  bfloat16 stays, float16 becomes bfloat16, a tensor
                       stored in 32-bit stays 32-bit, integers become int32;
  all-32-bit path:     every floating tensor becomes float32.

Reference: src/models/turbo_generic.rs:2038-2066 — every *.safetensors of the
folder, lookup by name with "Missing tensor: {name}" on the first miss,
BF16 widened to F32.
"""
from __future__ import annotations

from typing import Iterable

import torch

from .safetensors_io import SafetensorsError, open_model_files


class WeightsError(ValueError):
    """Checkpoint and model disagree.  The lists are kept as attributes."""

    def __init__(self, folder: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple, tuple]]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"weights in {folder} do not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


def target_dtype(stored: torch.dtype, mode: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if mode == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_tensors(folder: str, expected: dict[str, tuple[int, ...]], ignored: Iterable[str], *, mode: torch.dtype,
                 device) -> dict[str, torch.Tensor]:
    """The expected tensors of `folder` on `device`.  `expected` maps tensor
    name to shape; names in `ignored` may be present without being loaded."""
    files, where = open_model_files(folder)
    try:
        ignored = set(ignored)
        missing = sorted(n for n in expected if n not in where)
        unexpected = sorted(n for n in where if n not in expected and n not in ignored)
        wrong = [(n, where[n].entries[n].shape, tuple(shape)) for n, shape in sorted(expected.items())
                 if n in where and tuple(where[n].entries[n].shape) != tuple(shape)]
        if missing or unexpected or wrong:
            raise WeightsError(folder, missing, unexpected, wrong)
        out: dict[str, torch.Tensor] = {}
        for name in expected:
            t = where[name].read(name)
            out[name] = t.to(device=device, dtype=target_dtype(t.dtype, mode), copy=True)
        return out
    finally:
        for f in files:
            f.close()


__all__ = ["SafetensorsError", "WeightsError", "load_tensors", "target_dtype"]
