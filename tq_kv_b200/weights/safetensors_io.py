"""Reading and writing the safetensors file format.

Layout of a file: an 8-byte little-endian header length N, N bytes of JSON
{tensor name: {"dtype", "shape", "data_offsets": [begin, end]}} (plus an
optional "__metadata__" entry), then the raw little-endian tensor data;
offsets are relative to the end of the header.

Reference: src/models/turbo_generic.rs:2038-2053 loads every *.safetensors of
the model folder into one map from tensor name to tensor.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable, Iterator

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    file: str
    begin: int          # absolute byte offset in the file
    end: int


class SafetensorsFile:
    """One memory-mapped file; `entries` lists its tensors, `read(name)`
    returns a CPU tensor that views the mapping (copy it before the file
    object goes away)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"Cannot read {path}: {e}") from e
        head = self._f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.fstat(self._f.fileno()).st_size
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file size {size}")
        try:
            header = json.loads(self._f.read(n))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        base = 8 + n
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = _DTYPES.get(meta.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {meta.get('dtype')!r}")
            shape = tuple(int(s) for s in meta["shape"])
            a, b = meta["data_offsets"]
            numel = 1
            for s in shape:
                numel *= s
            if b - a != numel * torch.empty((), dtype=dt).element_size() or base + b > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has offsets {a}:{b} that do not match shape {shape}")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + a, base + b)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def read(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._mm)[e.begin:e.end]
        # frombuffer warns about non-writable buffers; the result is only read.
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=e.dtype)
        return t.reshape(e.shape)

    def close(self) -> None:
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass  # a tensor still views the mapping; the OS unmaps at exit
        self._f.close()


INDEX_NAME = "model.safetensors.index.json"


def open_model_files(folder: str) -> tuple[list[SafetensorsFile], dict[str, SafetensorsFile]]:
    """All safetensors files of a model folder and the map from tensor name to
    the file that holds it.  A name found in two files is an error.  If the
    folder has a `model.safetensors.index.json`, its `weight_map` decides:
    only the files it names are opened (a stray file beside them is not
    read), and a tensor that the map places in a file that does not hold it is
    an error.  (The reference scans the folder and ignores the index:
    src/models/turbo_generic.rs:2038-2053.)"""
    try:
        present = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
    except OSError as e:
        raise SafetensorsError(f"Cannot read model dir: {e}") from e
    weight_map = None
    index_path = os.path.join(folder, INDEX_NAME)
    if os.path.isfile(index_path):
        try:
            with open(index_path) as f:
                weight_map = json.load(f)["weight_map"]
            if not isinstance(weight_map, dict):
                raise TypeError("weight_map is no object")
        except (OSError, ValueError, KeyError, TypeError) as e:
            raise SafetensorsError(f"Invalid {INDEX_NAME}: {e}") from e
        names = sorted(set(weight_map.values()))
        lost = [n for n in names if n not in present]
        if lost:
            raise SafetensorsError(f"{INDEX_NAME} names files that are not in {folder}: {', '.join(lost)}")
    else:
        names = present
    if not names:
        raise SafetensorsError(f"No .safetensors files found in {folder}")
    files = [SafetensorsFile(os.path.join(folder, n)) for n in names]
    where: dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.entries:
            if weight_map is not None and weight_map.get(name) != os.path.basename(f.path):
                continue                      # the index places this tensor elsewhere (or nowhere)
            if name in where:
                raise SafetensorsError(f"tensor '{name}' is stored twice: in {where[name].path} and in {f.path}")
            where[name] = f
    if weight_map is not None:
        wrong = sorted(n for n in weight_map if n not in where)
        if wrong:
            raise SafetensorsError(f"{INDEX_NAME} places tensors in files that do not hold them: "
                                   + ", ".join(f"{n} -> {weight_map[n]}" for n in wrong))
    return files, where


def write_safetensors(path: str, specs: list[tuple[str, torch.dtype, tuple[int, ...]]],
                      tensors: Iterable[tuple[str, torch.Tensor]], metadata: dict | None = None) -> None:
    """Writes `tensors` (an iterable that yields them in the order of `specs`,
    so that a large model never sits in memory whole)."""
    header: dict = {}
    off = 0
    for name, dt, shape in specs:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dt).element_size()
        header[name] = {"dtype": _NAMES[dt], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        it: Iterator = iter(tensors)
        for name, dt, shape in specs:
            got_name, t = next(it)
            if got_name != name or t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(
                    f"write_safetensors: expected '{name}' {dt} {shape}, got '{got_name}' {t.dtype} {tuple(t.shape)}")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() < (1 << 26)
                        else memoryview(t.view(torch.uint8).numpy()))
