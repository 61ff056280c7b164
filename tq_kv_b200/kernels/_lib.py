"""ctypes bindings of the CUDA libraries: argument types, pointer and stream
helpers, the error check.  No kernel has a CPU fallback: a tensor that is not
on a CUDA device is an error, and so is a library that cannot be built."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only (this package has no CPU path)")
    return t.data_ptr()


def need_contiguous(**tensors: torch.Tensor | None) -> None:
    for name, t in tensors.items():
        if t is not None and not t.is_contiguous():
            raise KernelError(f"'{name}' must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current CUDA stream's handle (asked of torch at every launch: a capture runs on a stream of its own)."""
    if _raw_stream is not None:            # a tenth of the cost of building a torch.cuda.Stream object per launch
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# How many kernels of this package were launched (a claim the benchmark reports).
launches = [0]


class Timeline:
    """Device time by class of work.  While a timeline is the module's `timeline`, the parts call `mark(label)`
    after the kernels of a class (q/k/v product, attention, ...), which records a CUDA event; `totals()` then
    gives the time between consecutive marks, summed by label.  The marks sit between kernels, so a kernel does
    not start under its predecessor's tail across a mark (dependent launch); the sum of the classes is therefore
    a little more than the step takes when it is replayed as a graph.  The caller must keep the device busy
    ahead of the step (see bench.py), or the marks measure the host's launch pace instead of the kernels."""

    def __init__(self):
        self.marks: list = []

    def mark(self, label: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((label, ev))

    def totals(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for (_, a), (label, b) in zip(self.marks, self.marks[1:]):
            out[label] = out.get(label, 0.0) + a.elapsed_time(b) * 1e3        # microseconds
        return out


timeline = None          # a Timeline while one is recording


def mark(label: str) -> None:
    """Ends a class of work on the recording timeline, if there is one."""
    if timeline is not None:
        timeline.mark(label)


def check(status: int, what: str, n_kernels: int = 1) -> None:
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status}" + (" (invalid argument)" if status == 1 else ""))
    launches[0] += n_kernels


# ---- the report buffer: the status word of the tcgen05 kernels and the sampled ids --
# One int32 buffer per device.  Word 0 is the status word: the mbarrier waits of the tcgen05 kernels are bounded,
# and a wait that runs out raises a bit here instead of hanging (2: a matrix product, 4: the prompt attention,
# 8: its shared memory was not aligned).  Words 1.. take the token ids the sampler chooses, so that one small
# device-to-host copy per step brings both the ids and the status to the host.
REPORT_ROWS = 4096
_report: dict = {}                  # device -> int32[1 + REPORT_ROWS]
_tc_launched = [0]


def report_buffer(device) -> torch.Tensor:
    t = _report.get(device)
    if t is None:
        t = _report[device] = torch.zeros(1 + REPORT_ROWS, dtype=torch.int32, device=device)
    return t


def tc_status_word(device) -> torch.Tensor:
    """The device word a tcgen05 kernel launched now reports into; notes that one was launched."""
    _tc_launched[0] += 1
    return report_buffer(device)[:1]


def mark_tc_launched() -> None:
    """Replayed graphs launch tcgen05 kernels without passing through tc_status_word(): the caller says so."""
    _tc_launched[0] += 1


def raise_on_status(value: int, device) -> None:
    """Raises for a non-zero status word that the caller has read (and clears the word on the device)."""
    if value:
        report_buffer(device)[:1].zero_()
        raise KernelError(f"a tcgen05 kernel on {device}: a pipeline wait ran out (status {value}); "
                          "results are invalid")


def check_tc_status() -> None:
    """Raises if a tcgen05 kernel launched since the last check gave up on a
    pipeline wait (its output is then invalid).  Synchronises with the device."""
    if not _tc_launched[0]:
        return
    _tc_launched[0] = 0
    for dev, t in _report.items():
        raise_on_status(int(t[0].item()), dev)


_SIGNATURES = {
    "tq_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "tq_select_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "tq_random_fill": [c_void_p, c_int, c_size_t, ctypes.c_ulonglong, c_float, c_float, c_void_p],
    "tq_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    "tq_qkv_rope_cache": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tq_swiglu": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "tq_add_into": [c_void_p, c_void_p, c_int, c_size_t, c_void_p],
    "tq_attention": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                     c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                     c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tq_gemm_tiled": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_void_p],
    "tq_gemv_rows": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, c_int, c_int, c_void_p],
    "tq_skinny_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                       c_int, c_int, c_void_p],
    "tq_skinny_gemm_norm": [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_void_p],
    "tq_decode_gemm_tc_norm": [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tq_gemm_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_void_p, c_void_p],
    "tq_gemm_tc_mode": [c_int],
    "tq_decode_gemm_tc_adds_shares": [c_int, c_int],
    "tq_decode_gemm_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_void_p, c_void_p],
    "tq_flash_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                        c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tq_flash_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                         c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "tq_flash_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int,
                            c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int,
                            c_void_p, c_void_p],
    "tq_attention_merge": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tq_sample": [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_float, c_void_p,
                  c_void_p, c_void_p],
    "tq_sample_seeded": [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, ctypes.c_ulonglong, c_int,
                         c_void_p, c_float, c_void_p, c_void_p, c_void_p],
}

_core = None


def core() -> ctypes.CDLL:
    """The 'core' library, built at first use."""
    global _core
    if _core is None:
        lib = _build.load("core")
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _core = lib
    return _core
