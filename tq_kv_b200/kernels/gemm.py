"""Matrix products: y = x · W^T with W stored [out, in].

`linear()` picks the kernel from the operands:
  * up to 16 rows of bfloat16 and small weights (decoding a small model; the
    limits are in `_tc_takes`): the weight-streaming mma.sync kernel of
    csrc/skinny_gemm.cu, which reads the weight once and fuses bias, SwiGLU
    gating and the float32 accumulation into the residual stream;
  * up to 64 rows of bfloat16 otherwise: the same job on tcgen05 with swapped
    operands, TMA-fed (csrc/decode_gemm_tc.cu);
  * up to 16 rows of anything else: the float32 row kernel of csrc/gemm.cu
    with the same epilogues;
  * many rows, bfloat16 × bfloat16: the TMA + tcgen05 kernels of
    csrc/gemm_tc.cu (pairs of SMs from 129 rows on) with the same fused epilogues; with USE_TCGEN05 off, the
    library matrix product (cuBLAS through torch.mm with float32 output), as
    the reference engine does for all its products
    (src/models/turbo_generic.rs:68-91 -> candle -> cuBLAS);
  * everything else (the float32 path, mixed operands): the tiled float32
    FMA kernel of csrc/gemm.cu — never a reduced-precision mode.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import elementwise
from ._lib import (KernelError, check, check_tc_status, core, dtype_code, mark, need_contiguous, ptr, stream,
                   tc_status_word)

class PendingNorm:
    """An RMS norm that has not run yet: the float32 rows `h`, the norm's
    float32 weights and eps, and the dtype its result would have.  `linear()`
    takes it in place of activations and, where a decode kernel can, folds
    the norm into the product (the kernel reads h, multiplies with the
    weights while it builds its operand and scales its sums by each row's
    1 / sqrt(mean(h^2) + eps)); otherwise `materialize()` runs the norm's own
    kernel.  (src/models/turbo_generic.rs:41-51 is the norm.)"""

    def __init__(self, h: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype):
        self.h, self.weight, self.eps, self.out_dtype = h, weight, float(eps), out_dtype
        self._done: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.h.shape

    @property
    def device(self):
        return self.h.device

    @property
    def dtype(self):
        return self.out_dtype

    def materialize(self) -> torch.Tensor:
        if self._done is None:
            out = torch.empty(self.h.shape, dtype=self.out_dtype, device=self.h.device)
            self._done = elementwise.rmsnorm(self.h, self.weight, self.eps, out)
            mark("norms")               # a recording timeline books the kernel under the norms, not the product
        return self._done


# Fold a pending norm into the decode products: True wherever a kernel can, False nowhere, "auto" where it was
# measured to pay (see _fused_norm).  TQ_FUSE_NORM=1 / 0 set True / False.
FUSE_NORM = {"1": True, "0": False}.get(os.environ.get("TQ_FUSE_NORM", ""), "auto")
FUSED_NORM_MAX_ROWS = 16
ROW_KERNEL_MAX_ROWS = 16
SKINNY_MAX_ROWS = 64
# Weights from which a decode product of up to 16 rows runs on the tcgen05 kernel (see _tc_takes)
TC_DECODE_MIN_WEIGHT_BYTES = 24 << 20      # the product after a pending norm
TC_DECODE_MIN_GATED_BYTES = 64 << 20       # gated products
TC_DECODE_MIN_ADDED_BYTES = 4 << 20        # float32 results of given rows, which leave as shares of K
TC_DECODE_ADDED_ROWS = 8                   # ... and these from 9 rows on at any size


def _tc_takes(rows: int, w: torch.Tensor, swiglu: bool, after_norm: bool, float32_out: bool) -> bool:
    """Which of the two decode kernels gets a bfloat16 product that both can run: True for the TMA-fed
    tcgen05 kernel, False for the mma.sync one.  Over 16 rows always the former.  Below that by the weight's
    size, with limits that were measured (each product alone in a replayed graph, and the whole decode step
    of the 7B and 0.5B shapes): the product after a pending norm from 24 MB on (below it the mma.sync kernel
    with the norm folded in wins: 6 MB q|k|v 4.4 against 3.8 + a norm kernel); gated products from 64 MB on
    (55 MB at 8 rows: 12.8 against 14.3 us; 90 MB: 21.0 against 20.1); float32 results of rows that are
    given, which the tcgen05 kernel cuts into shares of K that meet in the L2, from 4 MB on and from 9 rows on
    at any size (9 MB with K = 4,864 at 8 rows: 6.1 against 4.5 us, at 16 rows 8.6 against 4.8; 5 MB with
    K = 1,536: 4.5 against 3.2; 1.6 MB at 8 rows: 2.9 against 2.7, a tie left where it was)."""
    if rows > ROW_KERNEL_MAX_ROWS or w.shape[1] % 32:
        return True
    size = w.numel() * 2
    if swiglu:
        return size >= TC_DECODE_MIN_GATED_BYTES
    if after_norm or not float32_out:
        return size >= TC_DECODE_MIN_WEIGHT_BYTES
    return size >= TC_DECODE_MIN_ADDED_BYTES or rows > TC_DECODE_ADDED_ROWS


def skinny_gemm(x, w, out, bias=None, accumulate=False, swiglu=False):
    """bfloat16 x [M <= 64, K] times bfloat16 w [N, K]^T on the tensor cores,
    streaming w once (csrc/skinny_gemm.cu).  K must be a multiple of 32."""
    M, K = x.shape
    N = out.shape[1]
    check(core().tq_skinny_gemm(ptr(x), ptr(w), ptr(bias), ptr(out), dtype_code(out), M, N, K, x.stride(0),
                                w.stride(0), out.stride(0), int(accumulate), int(swiglu), stream()), "skinny_gemm")
    return out


# ---- tcgen05 + TMA product for many rows (csrc/gemm_tc.cu) -----------------------
USE_TCGEN05 = True                  # False: the library product (cuBLAS) takes the many-row bfloat16 case
EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2


def set_gemm_tc_mode(mode: int) -> None:
    """0: products of more than 128 rows run on pairs of SMs (tcgen05 cta_group::2, 256-row tiles), smaller
    ones on single SMs; 1: single SMs always; 2: pairs always.  The default is 0 (or TQ_GEMM_TC_MODE)."""
    if mode not in (0, 1, 2):
        raise KernelError(f"gemm_tc mode {mode}: 0, 1 or 2")
    core().tq_gemm_tc_mode(mode)


def gemm_tc(x, w, out, bias=None, epilogue=EPI_STORE):
    """out (=, +=) x · w^T on the tcgen05 tensor cores; with EPI_SWIGLU w holds
    gate rows then up rows and out = silu(gate) * up.  bfloat16 operands, K a
    multiple of 8, 16-byte aligned rows."""
    M, K = x.shape
    N = out.shape[1]
    check(core().tq_gemm_tc(ptr(x), ptr(w), ptr(bias), ptr(out), dtype_code(out), M, N, K, x.stride(0), w.stride(0),
                            out.stride(0), epilogue, ptr(tc_status_word(x.device)), stream()), "gemm_tc")
    return out


def decode_gemm_tc(x, w, out, bias=None, accumulate=False, swiglu=False):
    """bfloat16 x [M <= 64, K] times w [N, K]^T on the tcgen05 tensor cores
    with the operands swapped (csrc/decode_gemm_tc.cu): the weight streams once
    through TMA, K is split over a thread-block cluster where tiles are few."""
    M, K = x.shape
    N = out.shape[1]
    check(core().tq_decode_gemm_tc(ptr(x), ptr(w), ptr(bias), ptr(out), dtype_code(out), M, N, K, x.stride(0),
                                   w.stride(0), out.stride(0), int(accumulate), int(swiglu),
                                   ptr(tc_status_word(x.device)), stream()), "decode_gemm_tc")
    return out


def _fused_norm(x: "PendingNorm", w, out, bias, accumulate, swiglu) -> bool:
    """Runs out (=, +=) norm(h) . w^T with the norm folded into a decode product; False if none takes it."""
    h, g = x.h, x.weight
    M, K = h.shape
    big = _tc_takes(M, w, bool(swiglu), True, out.dtype == torch.float32)     # the tcgen05 kernel's case
    # Measured inside whole decode steps: the tcgen05 kernel gains from the folded norm where it runs in its
    # cluster form anyway (gated products: 7B shape -0.8 % of a step) and loses where the norm costs it the
    # form with independent shares of K (float32 results: +8 %); the mma.sync kernel gains for plain products
    # (0.5B shape -1.5 %) and loses for gated ones, whose registers are scarce (+2 %).
    if FUSE_NORM == "auto" and big != bool(swiglu):
        return False
    if not (FUSE_NORM and USE_TCGEN05 and x.out_dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and h.dtype == torch.float32 and g.dtype == torch.float32 and 0 < M <= FUSED_NORM_MAX_ROWS
            and h.stride(1) == 1 and h.stride(0) % 4 == 0 and h.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0
            and g.is_contiguous() and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 and K % 8 == 0
            and out.dtype in (torch.float32, torch.bfloat16) and (not accumulate or out.dtype == torch.float32)
            and (not swiglu or w.shape[0] % 2 == 0)):
        return False
    N = out.shape[1]
    args = (ptr(h), ptr(g), x.eps, ptr(w), ptr(bias), ptr(out), dtype_code(out), M, N, K, h.stride(0), w.stride(0),
            out.stride(0), int(accumulate), int(swiglu))
    if big:
        check(core().tq_decode_gemm_tc_norm(*args, ptr(tc_status_word(h.device)), stream()), "decode_gemm_tc_norm")
    else:
        check(core().tq_skinny_gemm_norm(*args, stream()), "skinny_gemm_norm")
    return True


def product_adds_shares(rows: int, w: torch.Tensor, after_norm: bool = True) -> bool:
    """Whether linear() of `rows` bfloat16 rows (the result of a pending norm, or given rows) with `w` and a
    float32 result would run the decode product that cuts K into independent shares and adds them into the
    result (which it clears first, unless told to accumulate).  A caller that keeps a buffer of zeros can then
    ask for accumulation and save the clearing."""
    N, K = w.shape
    if not (USE_TCGEN05 and w.dtype == torch.bfloat16 and 0 < rows <= SKINNY_MAX_ROWS and K % 8 == 0
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0):
        return False
    if not _tc_takes(rows, w, False, after_norm, True):
        return False                                   # the mma.sync kernel takes it
    return bool(core().tq_decode_gemm_tc_adds_shares(N, K))


def _tc_ok(x, w, out, swiglu) -> bool:
    return (USE_TCGEN05 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (not swiglu or out.shape[1] % 2 == 0) and out.dtype in (torch.float32, torch.bfloat16)
            # the result leaves through TMA: 16-byte aligned base and row stride
            and out.data_ptr() % 16 == 0 and (out.stride(0) * out.element_size()) % 16 == 0)


def _skinny_ok(x, w) -> bool:
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_ROWS
            and K % 32 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tiled(x, w, out, bias=None, accumulate=False):
    M, K = x.shape
    N = w.shape[0]
    check(core().tq_gemm_tiled(ptr(x), dtype_code(x), ptr(w), dtype_code(w), ptr(bias), ptr(out), dtype_code(out),
                               M, N, K, x.stride(0), w.stride(0), out.stride(0), int(accumulate), stream()),
          "gemm_tiled")
    return out


def gemv_rows(x, w, out, bias=None, accumulate=False, swiglu=False):
    M, K = x.shape
    N = out.shape[1]
    check(core().tq_gemv_rows(ptr(x), dtype_code(x), ptr(w), dtype_code(w), ptr(bias), ptr(out), dtype_code(out),
                              M, N, K, x.stride(0), w.stride(0), out.stride(0), int(accumulate), int(swiglu),
                              stream()), "gemv_rows")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           accumulate: bool = False, swiglu: bool = False) -> torch.Tensor:
    """y = x · w^T (+ bias); with `swiglu`, w holds gate rows then up rows and
    y = silu(x · gate^T) * (x · up^T); with `accumulate`, `out` (float32) gets
    y added to it.  x [M, K], w [N, K] (or [2N, K]); float32 accumulation
    throughout."""
    pending = x if isinstance(x, PendingNorm) else None
    if len(x.shape) != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not multiply")
    if (pending is None and x.stride(1) != 1) or w.stride(1) != 1:
        raise KernelError("linear: operands must be contiguous along the inner dimension")
    M, K = x.shape
    rows_w = w.shape[0]
    if swiglu and rows_w % 2:
        raise KernelError("linear: a SwiGLU weight needs an even number of rows")
    N = rows_w // 2 if swiglu else rows_w
    if accumulate:
        if out is None or out.dtype != torch.float32:
            raise KernelError("linear: accumulate needs a float32 `out`")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)      # (a pending norm has both too)
    if tuple(out.shape) != (M, N) or out.stride(1) != 1:
        raise KernelError(f"linear: out has shape {tuple(out.shape)}, expected {(M, N)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != rows_w):
        raise KernelError("linear: bias must be float32 with one entry per weight row")
    if M == 0:
        return out
    if pending is not None:
        if _fused_norm(pending, w, out, bias, accumulate, swiglu):
            return out
        x = pending.materialize()

    # decoding: the TMA-fed tcgen05 kernel or the mma.sync kernel (_tc_takes says which, where both can)
    if (USE_TCGEN05 and M <= SKINNY_MAX_ROWS and _tc_ok(x, w, out, swiglu)
            and (not accumulate or out.dtype == torch.float32)
            and (not _skinny_ok(x, w)
                 or _tc_takes(M, w, bool(swiglu), pending is not None, out.dtype == torch.float32))):
        return decode_gemm_tc(x, w, out, bias, accumulate, swiglu)
    if _skinny_ok(x, w):
        return skinny_gemm(x, w, out, bias, accumulate, swiglu)
    if M <= ROW_KERNEL_MAX_ROWS:
        return gemv_rows(x, w, out, bias, accumulate, swiglu)

    if _tc_ok(x, w, out, swiglu) and (not accumulate or out.dtype == torch.float32):
        return gemm_tc(x, w, out, bias, EPI_SWIGLU if swiglu else (EPI_ACCUM if accumulate else EPI_STORE))

    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and bias is None:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)          # library product, float32 out
        if swiglu:
            return elementwise.swiglu(y, out)
        if accumulate:
            return elementwise.add_into(out, y)
        if out.dtype == torch.float32:
            out.copy_(y)
        else:
            out.copy_(y)
        return out

    if swiglu:
        y = torch.empty((M, rows_w), dtype=torch.float32, device=x.device)
        gemm_tiled(x, w, y, bias, False)
        return elementwise.swiglu(y, out)
    return gemm_tiled(x, w, out, bias, accumulate)
