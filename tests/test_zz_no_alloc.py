"""The allocation-free decode-attention entry point, called through its
exported C symbol (GPU).

Some hosts of these kernels may not allocate device memory while they run:
a loop with a hard deadline, a plugin whose host application owns every byte
of the device, a process that gave its whole budget to another allocator.
`tq_flash_decode_static` serves them: the scratch for the split key range is
a fixed array inside the library, the caller passes inputs and outputs only.
This test calls it several times in a row (each call finds the leftovers of
the one before in the shared scratch; one of them leaves huge values there on
purpose) and compares every result with two others that share nothing with
it but the inputs: the ordinary entry point routed to the general attention
kernel (another kernel, scratch from the caller), and a float64 computation
on the host over the keys gathered through the block table.  It also checks
that a call too large for the fixed scratch is refused with a clear message.

The file sorts last on purpose, so that a run that stops at the first failure
has run every other test before it.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOO_LARGE, UNSUPPORTED = -2, -3


def _lib():
    from tq_kv_b200.csrc import build
    lib = ctypes.CDLL(build.build("noalloc"))
    lib.tq_flash_decode_static.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                           c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p]
    lib.tq_flash_decode_static.restype = c_int
    lib.tq_flash_decode_static_error.restype = ctypes.c_char_p
    return lib


def _case(seed, B, nh, nkv, hd, lengths):
    g = torch.Generator().manual_seed(seed)
    P, width = 64, 12
    n_pages = B * width
    kp = (torch.randn(n_pages, nkv, P, hd, generator=g)).to(torch.bfloat16).to(DEV)
    vp = (torch.randn(n_pages, nkv, P, hd, generator=g)).to(torch.bfloat16).to(DEV)
    table = torch.randperm(n_pages, generator=g).reshape(B, width).to(torch.int32).to(DEV)
    q = torch.randn(B, nh * hd, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    return q, kp, vp, table, width, pos, seq


def _ordinary(q, kp, vp, table, width, pos, seq, nh, nkv, hd, window, n_splits):
    from tq_kv_b200 import kernels
    B = q.shape[0]
    out = torch.empty_like(q)
    scratch = torch.empty(kernels.split_scratch_floats(B, nh, hd, n_splits), device=DEV) if n_splits > 1 else None
    kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=pos, tok_seq=seq,
                      cu_seqlens=torch.arange(B + 1, dtype=torch.int32, device=DEV), start_pos=pos, window=window,
                      k_pages=kp, v_pages=vp, block_table=table, table_width=width, n_splits=n_splits,
                      scratch=scratch, use_flash=False)       # the general kernel, not the one under test
    return out


def _float64(q, kp, vp, table, width, pos, seq, nh, nkv, hd, window):
    """softmax(q k^T / sqrt(hd)) v in float64 on the host, keys found through the block table."""
    import math
    q, kp, vp, table = q.cpu().double(), kp.cpu().double(), vp.cpu().double(), table.cpu()
    out = torch.zeros_like(q)
    for b, p in enumerate(pos.tolist()):
        n = p + 1
        lo = max(0, n - window) if window else 0
        pages = table[b, :-(-n // 64)].long()
        k = kp[pages].transpose(0, 1).reshape(nkv, -1, hd)[:, lo:n]          # [nkv, keys, hd]
        v = vp[pages].transpose(0, 1).reshape(nkv, -1, hd)[:, lo:n]
        qb = q[b].reshape(nkv, nh // nkv, hd)
        w = torch.softmax(qb @ k.transpose(1, 2) / math.sqrt(hd), -1)
        out[b] = (w @ v).reshape(-1)
    return out


def _static(lib, q, kp, vp, table, width, pos, seq, nh, nkv, hd, window, n_splits):
    out = torch.zeros_like(q)
    st = lib.tq_flash_decode_static(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), width, 0, 64,
                                    pos.data_ptr(), seq.data_ptr(), int(window or 0), 1.0 / hd ** 0.5,
                                    out.data_ptr(), q.shape[0], nh, nkv, hd, n_splits,
                                    torch.cuda.current_stream().cuda_stream)
    return st, out


def test_calls_in_a_row_match_another_kernel_and_a_float64_computation():
    lib = _lib()
    # different sizes and split counts, so that a call reads scratch rows the one before wrote differently; the
    # second call's values are scaled up a thousandfold and it uses more splits than the third, which then finds
    # those large numbers in every scratch row it does not overwrite first
    calls = [dict(seed=1, B=5, nh=28, nkv=4, hd=128, lengths=[700, 64, 1, 511, 333], window=None, n_splits=6),
             dict(seed=6, B=4, nh=6, nkv=2, hd=64, lengths=[600, 768, 129, 640], window=None, n_splits=8, scale=1e3),
             dict(seed=2, B=3, nh=6, nkv=2, hd=64, lengths=[300, 768, 129], window=200, n_splits=3),
             dict(seed=3, B=2, nh=8, nkv=8, hd=32, lengths=[40, 500], window=None, n_splits=1)]
    for c in calls:
        args = list(_case(c["seed"], c["B"], c["nh"], c["nkv"], c["hd"], c["lengths"]))
        if "scale" in c:
            args[2] = (args[2].float() * c["scale"]).to(torch.bfloat16)        # the values
        shape = (c["nh"], c["nkv"], c["hd"], c["window"], c["n_splits"])
        st, got = _static(lib, *args, *shape)
        torch.cuda.synchronize()
        assert st == 0, lib.tq_flash_decode_static_error()
        for what, want in (("the general kernel", _ordinary(*args, *shape).float().cpu()),
                           ("float64 on the host", _float64(*args, *shape[:4]).float())):
            err = float((got.float().cpu() - want).abs().max())
            assert err <= 8e-3 * max(1.0, float(want.abs().max())), (what, c, err)


def test_a_call_beyond_the_fixed_scratch_is_refused_and_launches_nothing():
    lib = _lib()
    args = _case(4, 64, 28, 4, 128, [700] * 64)
    st, out = _static(lib, *args, 28, 4, 128, None, 8)          # 64*28*8*130 floats > 2^20
    torch.cuda.synchronize()
    assert st == TOO_LARGE and float(out.float().abs().sum()) == 0.0
    msg = lib.tq_flash_decode_static_error().decode()
    assert "1863680 floats" in msg and "1048576" in msg
    st, _ = _static(lib, *_case(5, 2, 6, 2, 48, [10, 20]), 6, 2, 48, None, 1)
    assert st == UNSUPPORTED and "head_dim 48" in lib.tq_flash_decode_static_error().decode()
