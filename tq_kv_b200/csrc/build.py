"""Builds the native libraries of this package and loads them with ctypes: the
CUDA kernels with nvcc for sm_100a, the host runtime (plain C++, no CUDA) with
the system's C++ compiler.

A library is a named group of .cu (or .cpp) files of this folder.  The shared object is
written beside the sources as `_build/libtqkv_<group>_<hash>.so`, where the
hash covers the sources, the headers and the flags, so that a stale build is
never loaded.  If the folder cannot be written to, a per-user folder under
the system's temporary directory is used.  A group is compiled the first time
something asks for it; progress lines go to stderr.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))

GROUPS: dict[str, list[str]] = {
    # everything a model needs in either precision
    "core": ["elementwise.cu", "attention.cu", "flash_decode.cu", "flash_prefill.cu", "flash_prefill_tc.cu", "gemm.cu", "skinny_gemm.cu",
             "gemm_tc.cu", "decode_gemm_tc.cu", "sampling.cu", "random_fill.cu"],
    # decode attention for callers that cannot allocate: a library of its own (flash_decode_static.h)
    "noalloc": ["flash_decode_static.cu"],
    # the host side of a step: cache bookkeeping, checks and packing (C++, no CUDA: builds and runs without a GPU)
    "host": ["host_runtime.cpp"],
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[tq-kv-b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of this package cannot be built")


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); "
                     "the host runtime of this package cannot be built")


def _is_host(group: str) -> bool:
    return all(src.endswith(".cpp") for src in GROUPS[group])


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def group_hash(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(HOST_FLAGS if _is_host(group) else NVCC_FLAGS).encode())
    included = sorted(f for f in os.listdir(_HERE) if f.endswith(".cu") and f not in GROUPS[group]
                      and any(f'#include "{f}"' in open(os.path.join(_HERE, src)).read() for src in GROUPS[group]))
    for name in GROUPS[group] + included + _headers():
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    return h.hexdigest()[:12]


def _build_dirs() -> list[str]:
    dirs = [os.path.join(_HERE, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"tq_kv_b200_build_{uid}"))
    return dirs


def library_path(group: str) -> str | None:
    """Path of an up-to-date build of `group`, or None."""
    name = f"libtqkv_{group}_{group_hash(group)}.so"
    for d in _build_dirs():
        p = os.path.join(d, name)
        if os.path.exists(p):
            return p
    return None


def _writable_build_dir() -> str:
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {_build_dirs()}")


def _run(cmd: list[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed ({p.returncode}):\n{' '.join(cmd)}\n{p.stdout}")


def build(group: str, verbose_ptxas: bool = False) -> str:
    """Compiles `group` if no up-to-date build exists; returns the .so path."""
    have = library_path(group)
    if have:
        return have
    if _is_host(group):
        return _build_host(group)
    nvcc = find_nvcc()
    out_dir = _writable_build_dir()
    tag = group_hash(group)
    final = os.path.join(out_dir, f"libtqkv_{group}_{tag}.so")
    work = tempfile.mkdtemp(prefix=f"{group}_{tag}_", dir=out_dir)
    sources = GROUPS[group]
    _say(f"compiling CUDA library '{group}' for sm_100a ({len(sources)} files) into {out_dir} ...")
    t0 = time.time()
    done = [0]

    def compile_one(src: str) -> str:
        obj = os.path.join(work, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
        if verbose_ptxas:
            cmd[1:1] = ["-Xptxas", "-v"]
        _run(cmd, f"nvcc {src}")
        done[0] += 1
        _say(f"  compiled {src} ({done[0]}/{len(sources)}, {time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            objs = list(pool.map(compile_one, sources))
        tmp_so = os.path.join(work, "lib.so")
        _run([nvcc, "-shared", "-o", tmp_so, *objs, "-Xcompiler", "-fPIC", "-lcuda"], f"link {group}")
        os.replace(tmp_so, final)      # atomic: concurrent builders end with the same file
        for old in os.listdir(out_dir):  # builds of older sources are of no use any more
            if old.startswith(f"libtqkv_{group}_") and old.endswith(".so") and old != os.path.basename(final):
                try:
                    os.remove(os.path.join(out_dir, old))
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {os.path.basename(final)} in {time.time() - t0:.0f} s")
    return final


def _build_host(group: str) -> str:
    cxx = find_cxx()
    out_dir = _writable_build_dir()
    final = os.path.join(out_dir, f"libtqkv_{group}_{group_hash(group)}.so")
    tmp_so = os.path.join(out_dir, f".{os.path.basename(final)}.{os.getpid()}")
    t0 = time.time()
    try:
        _run([cxx, *HOST_FLAGS, "-shared", "-I", _HERE, "-o", tmp_so, *(os.path.join(_HERE, s) for s in GROUPS[group])],
             f"{os.path.basename(cxx)} {group}")
        os.replace(tmp_so, final)
    finally:
        if os.path.exists(tmp_so):
            os.remove(tmp_so)
    for old in os.listdir(out_dir):
        if old.startswith(f"libtqkv_{group}_") and old.endswith(".so") and old != os.path.basename(final):
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    _say(f"built {os.path.basename(final)} in {time.time() - t0:.1f} s")
    return final


def load(group: str) -> ctypes.CDLL:
    """The ctypes handle of `group`, built first if need be."""
    with _lock:
        lib = _loaded.get(group)
        if lib is None:
            lib = ctypes.CDLL(build(group))
            _loaded[group] = lib
        return lib


def build_all() -> list[str]:
    return [build(g) for g in GROUPS]
