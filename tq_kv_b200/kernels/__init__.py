"""Python entry points of the hand-written CUDA kernels (sources in ../csrc)."""
from . import _lib
from ._lib import KernelError, Timeline, launches, mark, mark_tc_launched
from .attention import attention, check_head_geometry, plan_splits, split_scratch_floats
from .elementwise import add_into, embed, qkv_rope_cache, random_fill, rmsnorm, select_tokens, swiglu
from .gemm import (PendingNorm, check_tc_status, decode_gemm_tc, gemm_tc, gemm_tiled, gemv_rows, linear, product_adds_shares, set_gemm_tc_mode,
                   skinny_gemm)
from .sampling import sample

__all__ = ["KernelError", "PendingNorm", "Timeline", "mark", "add_into", "attention", "check_head_geometry", "check_tc_status", "decode_gemm_tc", "embed", "launches", "mark_tc_launched", "gemm_tc", "gemm_tiled", "set_gemm_tc_mode", "gemv_rows",
           "linear", "plan_splits", "product_adds_shares", "qkv_rope_cache", "random_fill", "rmsnorm", "select_tokens", "sample", "skinny_gemm", "split_scratch_floats", "swiglu"]
