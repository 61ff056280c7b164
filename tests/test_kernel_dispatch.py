"""Which decode kernel `kernels.linear` hands a bfloat16 product to (no GPU needed: the rule only looks at sizes)."""
import pytest
import torch

from tq_kv_b200.kernels import gemm


def _w(n, k):
    return torch.empty(n, k, dtype=torch.bfloat16, device="meta")


@pytest.mark.parametrize("rows,n,k,swiglu,after_norm,f32,want", [
    # the 7B shape: everything on the tcgen05 kernel
    (8, 4608, 3584, False, True, True, True),
    (8, 3584, 3584, False, False, True, True),
    (8, 2 * 18944, 3584, True, True, False, True),
    (8, 3584, 18944, False, False, True, True),
    # the 0.5B shape at 8 rows: q|k|v (norm folded in), o and gate|up stay on the mma.sync kernel, down does not
    (8, 1152, 896, False, True, True, False),
    (8, 896, 896, False, False, True, False),
    (8, 2 * 4864, 896, True, True, False, False),
    (8, 896, 4864, False, False, True, True),
    # from 9 rows on the float32 results of given rows leave the mma.sync kernel at any size
    (9, 896, 896, False, False, True, True),
    (9, 1152, 896, False, True, True, False),
    # a 55 MB gated product stays, a 90 MB one does not
    (8, 2 * 8960, 1536, True, True, False, False),
    (8, 2 * 11008, 2048, True, True, False, True),
    # over 16 rows, or with K no multiple of 32, only the tcgen05 kernel can
    (17, 896, 896, False, False, True, True),
    (4, 64, 40, False, False, True, True),
])
def test_which_decode_kernel_takes_a_product(rows, n, k, swiglu, after_norm, f32, want):
    assert gemm._tc_takes(rows, _w(n, k), swiglu, after_norm, f32) is want
