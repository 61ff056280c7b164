"""Python entry point of the sampling kernel (csrc/sampling.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import KernelError, check, core, need_contiguous, ptr, stream


def sample(logits: torch.Tensor, out: torch.Tensor, *, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           uniforms: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None,
           repeat_penalty: float = 1.0, requests: Optional[torch.Tensor] = None, seed: int = 0,
           index: int = 0) -> torch.Tensor:
    """One token per row of float32 logits [R, V] into out (int32 [R]).
    temperature <= 0: arg-max (lowest id on ties).  Else softmax(logits /
    temperature) restricted by top_k (0: off) and top_p (>= 1: off), drawn
    with one uniform in [0, 1) per row: uniforms[r] if given, else generated
    on the device from (seed, requests[r], index) — the request index of each
    row (int32 [R] on the device) and the index of the token being sampled
    (sampling/rng.py is the same generator on the host).  `counts` (int32
    [R, V]) holds how often each token was generated so far; the repeat penalty
    is applied once per occurrence and the chosen token's count is incremented."""
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [R, V], contiguous along V")
    R, V = logits.shape
    if out.dtype != torch.int32 or out.shape[0] < R:
        raise KernelError("sample: out must be int32 [R]")
    if temperature > 0:
        if uniforms is not None:
            if uniforms.dtype != torch.float32 or uniforms.shape[0] < R:
                raise KernelError("sample: uniforms must be float32 [R]")
        elif requests is None or requests.dtype != torch.int32 or requests.shape[0] < R:
            raise KernelError("sample: temperature > 0 needs float32 uniforms [R] or int32 requests [R]")
    if counts is not None and (counts.dtype != torch.int32 or tuple(counts.shape) != (R, V)):
        raise KernelError("sample: counts must be int32 [R, V]")
    need_contiguous(out=out, uniforms=uniforms, counts=counts, requests=requests)
    scratch = None
    if temperature <= 0 or 0 < top_k <= FAST_TOP_K_MAX:
        scratch = _sample_scratch(logits.device, R)
    n_kernels = 2 if scratch is not None else 1
    if temperature > 0 and uniforms is None:
        check(core().tq_sample_seeded(ptr(logits), logits.stride(0), R, V, float(temperature), int(top_k), float(top_p),
                                      ptr(requests), int(seed) & ((1 << 64) - 1), int(index), ptr(counts),
                                      float(repeat_penalty), ptr(out), ptr(scratch), stream()), "sample", n_kernels)
        return out
    check(core().tq_sample(ptr(logits), logits.stride(0), R, V, float(temperature), int(top_k), float(top_p),
                           ptr(uniforms), ptr(counts), float(repeat_penalty), ptr(out), ptr(scratch), stream()),
          "sample", n_kernels)
    return out


FAST_TOP_K_MAX = 64
_scratch: dict = {}


def _sample_scratch(device, rows: int) -> torch.Tensor:
    """Candidates of the two-step kernels (arg-max parts, top-k parts): kept per device, grown on demand."""
    lib = core()
    lib.tq_sample_scratch_bytes.restype = ctypes.c_size_t
    lib.tq_sample_scratch_bytes.argtypes = [ctypes.c_int]
    need = int(lib.tq_sample_scratch_bytes(max(rows, 64)))
    t = _scratch.get(device)
    if t is None or t.numel() < need:
        t = _scratch[device] = torch.empty(need, dtype=torch.uint8, device=device)
    return t
