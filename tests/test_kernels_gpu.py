"""Each CUDA kernel alone against a plain float32 PyTorch computation of the
same operation, at sizes other than the tiny models' (GPU)."""
import math

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all(), what
    err = float((got - want).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: {err:.3e}"


# ---- embedding, norm, gating --------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    from tq_kv_b200 import kernels
    table = rnd(1000, 200, dtype=dtype)
    toks = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embed(toks, table, out, status)
    assert torch.equal(out, table[toks.long()].float()) and int(status) == 0
    kernels.embed(torch.tensor([3, 1000], dtype=torch.int32, device=DEV), table, out[:2], status)
    assert int(status) == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("H,out_dtype", [(1000, torch.float32), (72, torch.bfloat16), (3584, torch.bfloat16),
                                         (896, torch.bfloat16), (5120, torch.bfloat16), (8192, torch.float32),
                                         (8196, torch.float32), (1001, torch.bfloat16)])
def test_rmsnorm(H, out_dtype):
    from tq_kv_b200 import kernels
    x, w = rnd(7, H, scale=3.0), rnd(H) + 1.0
    out = torch.empty(7, H, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, w, 1e-5, out)
    want = pm.rms_norm(x.cpu(), w.cpu(), 1e-5)
    close(out, want, 1e-6 if out_dtype == torch.float32 else 4e-3, "rmsnorm")
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    out = torch.empty(3, H, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, w, 1e-5, out, rows)
    close(out, want[[6, 0, 6]], 1e-6 if out_dtype == torch.float32 else 4e-3, "rmsnorm rows")


@pytest.mark.parametrize("H,out_dtype", [(72, torch.float32), (1000, torch.bfloat16), (1536, torch.bfloat16),
                                         (3584, torch.bfloat16), (5120, torch.float32), (8192, torch.bfloat16),
                                         (8200, torch.bfloat16), (70, torch.float32)])
def test_rmsnorm_many_rows(H, out_dtype):
    """A prompt's rows go through the variant that holds a row in registers (widths up to 8192 in steps of
    four); wider or odd rows fall to the general kernel.  Both give the plain result."""
    from tq_kv_b200 import kernels
    x, w = rnd(200, H, scale=3.0), rnd(H) + 1.0
    x[17] *= 40.0                                            # rows of very different size
    out = torch.empty(200, H, dtype=out_dtype, device=DEV)
    kernels.rmsnorm(x, w, 1e-6, out)
    want = pm.rms_norm(x.cpu(), w.cpu(), 1e-6)
    close(out, want, 2e-6 if out_dtype == torch.float32 else 4e-3, "rmsnorm many rows")
    rows = torch.arange(199, -1, -1, dtype=torch.int32, device=DEV)
    kernels.rmsnorm(x, w, 1e-6, out, rows)
    close(out, want.flip(0), 2e-6 if out_dtype == torch.float32 else 4e-3, "rmsnorm many rows, gathered")


def test_swiglu_and_add_into():
    from tq_kv_b200 import kernels
    gu = rnd(5, 2 * 203, scale=2.0)
    out = torch.empty(5, 203, dtype=torch.bfloat16, device=DEV)
    kernels.swiglu(gu, out)
    want = torch.nn.functional.silu(gu[:, :203]) * gu[:, 203:]
    close(out, want, 4e-3, "swiglu")
    acc, x = rnd(9, 77), rnd(9, 77, dtype=torch.bfloat16, seed=1)
    want = acc + x.float()
    kernels.add_into(acc, x)
    assert torch.equal(acc, want)


# ---- matrix products ------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(70, 130, 50), (1, 64, 16), (129, 65, 203)])
@pytest.mark.parametrize("dts", [(torch.float32,) * 3, (torch.bfloat16, torch.bfloat16, torch.float32),
                                 (torch.bfloat16, torch.float32, torch.bfloat16)])
def test_gemm_tiled(M, N, K, dts):
    from tq_kv_b200 import kernels
    a, w, bias = rnd(M, K, dtype=dts[0]), rnd(N, K, dtype=dts[1], seed=1), rnd(N, seed=2)
    out = torch.empty(M, N, dtype=dts[2], device=DEV)
    kernels.gemm_tiled(a, w, out, bias)
    want = a.double() @ w.double().T + bias.double()
    tol = 2e-6 if dts[2] == torch.float32 else 4e-3
    close(out, want, tol, "gemm_tiled")
    if dts[2] == torch.float32:
        kernels.gemm_tiled(a, w, out, None, accumulate=True)
        close(out, 2 * want - bias.double(), tol, "gemm_tiled accumulate")


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("K,dt", [(200, torch.bfloat16), (203, torch.bfloat16), (100, torch.float32),
                                  (3584, torch.bfloat16)])
def test_gemv_rows(M, K, dt):
    from tq_kv_b200 import kernels
    N = 37
    a, w, bias = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt, seed=1), rnd(N, seed=2)
    out = rnd(M, N, seed=3)
    base = out.clone()
    kernels.gemv_rows(a, w, out, bias, accumulate=True)
    want = base.double() + a.double() @ w.double().T + bias.double()
    close(out, want, 3e-6 * math.sqrt(K / 100), "gemv accumulate")
    w2 = rnd(2 * N, K, dtype=dt, seed=4, scale=0.2)
    out = torch.empty(M, N, dtype=dt, device=DEV)
    kernels.gemv_rows(a, w2, out, swiglu=True)
    y = a.double() @ w2.double().T
    want = torch.nn.functional.silu(y[:, :N]) * y[:, N:]
    close(out, want, 1e-5 if dt == torch.float32 else 4e-3, "gemv swiglu")


@pytest.mark.parametrize("M", [5, 16, 17, 300])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tcgen05", [False, True])
def test_linear_picks_a_kernel_for_every_shape(M, dt, tcgen05, monkeypatch):
    from tq_kv_b200 import kernels
    monkeypatch.setattr(kernels.gemm, "USE_TCGEN05", tcgen05)
    K, N = 136, 210
    x, w = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt, seed=1, scale=0.1)
    want = x.double() @ w.double().T
    close(kernels.linear(x, w, out_dtype=torch.float32), want, 5e-6, "linear")
    res = rnd(M, N, seed=5)
    want_acc = res.double() + want
    kernels.linear(x, w, out=res, accumulate=True)
    close(res, want_acc, 5e-6, "linear accumulate")
    w2 = rnd(2 * N, K, dtype=dt, seed=2, scale=0.1)
    y = x.double() @ w2.double().T
    close(kernels.linear(x, w2, swiglu=True, out_dtype=dt), torch.nn.functional.silu(y[:, :N]) * y[:, N:],
          1e-5 if dt == torch.float32 else 4e-3, "linear swiglu")
    if dt == torch.bfloat16:        # a 32-bit weight under 16-bit activations stays 32-bit
        wf = rnd(N, K, seed=3, scale=0.1)
        close(kernels.linear(x, wf, out_dtype=torch.float32), x.double() @ wf.double().T, 5e-6, "mixed")


@pytest.mark.parametrize("M", [1, 7, 8, 9, 16, 31, 33, 64])
@pytest.mark.parametrize("N,K", [(37, 64), (100, 96), (512, 3584), (33, 18944)])
def test_skinny_gemm(M, N, K):
    from tq_kv_b200 import kernels
    x, w, bias = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1), rnd(N, seed=2)
    want = x.double() @ w.double().T
    out = rnd(M, N, seed=3)
    base = out.clone()
    kernels.skinny_gemm(x, w, out, bias, accumulate=True)
    close(out, base.double() + want + bias.double(), 1e-5 * math.sqrt(K / 64), "skinny accumulate")
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.skinny_gemm(x, w, out)
    close(out, want, 4e-3, "skinny bf16 out")
    w2, b2 = rnd(2 * N, K, dtype=torch.bfloat16, seed=4, scale=2.0 / math.sqrt(K)), rnd(2 * N, seed=5)
    y = x.double() @ w2.double().T + b2.double()
    out = torch.empty(M, N, device=DEV)
    kernels.skinny_gemm(x, w2, out, b2, swiglu=True)
    close(out, torch.nn.functional.silu(y[:, :N]) * y[:, N:], 1e-5 * math.sqrt(K / 64), "skinny swiglu")
    # a view with a row stride (columns of a wider matrix)
    wide = rnd(M, K + 64, dtype=torch.bfloat16, seed=6)
    out = torch.empty(M, N, device=DEV)
    kernels.skinny_gemm(wide[:, 32:32 + K], w, out)
    close(out, wide[:, 32:32 + K].double() @ w.double().T, 1e-5 * math.sqrt(K / 64), "skinny strided")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (1, 8, 8), (2048, 512, 3584), (257, 1000, 1096),
                                   (512, 4608, 3584), (100, 3584, 2048)])
@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_tc(M, N, K, mode):
    """The TMA + tcgen05 product on single SMs (128-row tiles) and on pairs of SMs (cta_group::2, 256-row
    tiles): whole tiles, ragged edges in M, N and K, a long K; tiles fewer than the SMs, which the float32
    products cut along K (the plain store then clears C first and sums the shares)."""
    from tq_kv_b200 import kernels
    kernels.set_gemm_tc_mode(mode)
    try:
        _check_gemm_tc(kernels, M, N, K)
    finally:
        kernels.set_gemm_tc_mode(0)


def _check_gemm_tc(kernels, M, N, K):
    x, w, bias = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1), rnd(N, seed=2)
    want = x.double() @ w.double().T
    tol = 2e-6 * math.sqrt(K)
    out = torch.full((M, N), 7.0, device=DEV)
    kernels.gemm_tc(x, w, out, bias)
    kernels.check_tc_status()
    close(out, want + bias.double(), tol, "tc store")
    base = rnd(M, N, seed=3)
    out = base.clone()
    kernels.gemm_tc(x, w, out, None, kernels.gemm.EPI_ACCUM)
    close(out, base.double() + want, tol, "tc accumulate")
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(x, w, out)
    close(out, want, 4e-3, "tc bf16 out")
    if N % 2 == 0:
        w2 = rnd(2 * N, K, dtype=torch.bfloat16, seed=4, scale=2.0 / math.sqrt(K))
        y = x.double() @ w2.double().T
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        kernels.gemm_tc(x, w2, out, None, kernels.gemm.EPI_SWIGLU)
        close(out, torch.nn.functional.silu(y[:, :N]) * y[:, N:], 4e-3, "tc swiglu")
    # operands that are views with a row stride
    wide = rnd(M, K + 64, dtype=torch.bfloat16, seed=6)
    out = torch.empty(M, N, device=DEV)
    kernels.gemm_tc(wide[:, 32:32 + K], w, out)
    close(out, wide[:, 32:32 + K].double() @ w.double().T, tol, "tc strided")
    kernels.check_tc_status()


@pytest.mark.parametrize("M", [17, 32, 33, 50, 64, 3])
@pytest.mark.parametrize("N,K", [(37, 64), (100, 96), (512, 3584), (130, 18944), (3584, 512)])
def test_decode_gemm_tc(M, N, K):
    """Swapped-operand tcgen05 product for decode batches: ragged N, short and long K (cluster split-K)."""
    from tq_kv_b200 import kernels
    x, w, bias = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1), rnd(N, seed=2)
    want = x.double() @ w.double().T
    out = rnd(M, N, seed=3)
    base = out.clone()
    kernels.decode_gemm_tc(x, w, out, bias, accumulate=True)
    close(out, base.double() + want + bias.double(), 1e-5 * math.sqrt(K / 64), "accumulate")
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.decode_gemm_tc(x, w, out)
    close(out, want, 4e-3, "bf16 out")
    w2, b2 = rnd(2 * N, K, dtype=torch.bfloat16, seed=4, scale=2.0 / math.sqrt(K)), rnd(2 * N, seed=5)
    y = x.double() @ w2.double().T + b2.double()
    out = torch.empty(M, N, device=DEV)
    kernels.decode_gemm_tc(x, w2, out, b2, swiglu=True)
    # float32 accumulation over K terms: the rounding error grows with sqrt(K), as in the check above
    close(out, torch.nn.functional.silu(y[:, :N]) * y[:, N:], 1e-5 * math.sqrt(K / 64), "swiglu")
    kernels.check_tc_status()


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K,big", [(37, 64, False), (100, 96, False), (512, 3584, False), (200, 1000, True),
                                     (4608, 3584, True), (129, 7168, True), (640, 8, True)])
def test_decode_products_with_the_norm_folded_in(M, N, K, big, monkeypatch):
    """kernels.linear() given a pending RMS norm instead of activations: the mma.sync kernel (small weights) and
    the tcgen05 kernel (large weights, or K no multiple of 32) read the float32 rows, multiply with the norm's
    weights while they build their operand and scale their sums by each row's 1/rms.  The reference rounds
    h * g to bfloat16 as the kernels do, so the bound is that of float32 summation alone; plain, accumulating
    and gated epilogues; then against the norm run as a kernel of its own."""
    from tq_kv_b200 import kernels
    if big:
        monkeypatch.setattr(kernels.gemm, "TC_DECODE_MIN_WEIGHT_BYTES", 0)       # send it to the tcgen05 kernel
    monkeypatch.setattr(kernels.gemm, "FUSE_NORM", True)                         # wherever a kernel can
    eps = 1e-5
    h, g = rnd(M, K, seed=7, scale=3.0), 1.0 + rnd(K, seed=8, scale=0.2)
    w, bias = rnd(N, K, dtype=torch.bfloat16, seed=1), rnd(N, seed=2)
    x = (h * g).to(torch.bfloat16).double()
    rms = torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    want = (x @ w.double().T) / rms
    tol = 1e-5 * math.sqrt(max(K, 64) / 64)
    n0 = kernels.launches[0]
    out = kernels.linear(kernels.PendingNorm(h, g, eps, torch.bfloat16), w, bias=bias, out_dtype=torch.float32)
    assert kernels.launches[0] - n0 == 1                                        # one kernel: no norm of its own
    close(out, want + bias.double(), tol, "folded norm")
    res = rnd(M, N, seed=3)
    base = res.clone()
    kernels.linear(kernels.PendingNorm(h, g, eps, torch.bfloat16), w, out=res, accumulate=True)
    close(res, base.double() + want, tol, "folded norm, accumulate")
    w2, b2 = rnd(2 * N, K, dtype=torch.bfloat16, seed=4, scale=2.0 / math.sqrt(K)), rnd(2 * N, seed=5)
    y = (x @ w2.double().T) / rms + b2.double()
    out = kernels.linear(kernels.PendingNorm(h, g, eps, torch.bfloat16), w2, bias=b2, swiglu=True,
                         out_dtype=torch.float32)
    close(out, torch.nn.functional.silu(y[:, :N]) * y[:, N:], tol, "folded norm, gated")
    out = kernels.linear(kernels.PendingNorm(h, g, eps, torch.bfloat16), w2, swiglu=True, out_dtype=torch.bfloat16)
    y = (x @ w2.double().T) / rms
    close(out, torch.nn.functional.silu(y[:, :N]) * y[:, N:], 4e-3, "folded norm, gated, bf16 out")
    # the same through the norm's own kernel: rounding of the normed rows to bfloat16 is the only difference
    monkeypatch.setattr(kernels.gemm, "FUSE_NORM", False)
    n0 = kernels.launches[0]
    apart = kernels.linear(kernels.PendingNorm(h, g, eps, torch.bfloat16), w, bias=bias, out_dtype=torch.float32)
    assert kernels.launches[0] - n0 >= 2
    close(apart, want + bias.double(), 8e-3, "norm as a kernel of its own")
    kernels.check_tc_status()


def test_a_pending_norm_runs_as_its_own_kernel_where_no_product_takes_it():
    """More rows than the decode products fold a norm for, float32 weights, a float32 result dtype: the norm's
    kernel runs first and the product follows; the result is the same either way."""
    from tq_kv_b200 import kernels
    eps = 1e-6
    for M, wdt, odt in ((17, torch.bfloat16, torch.bfloat16), (200, torch.bfloat16, torch.bfloat16),
                        (4, torch.float32, torch.float32)):
        h, g = rnd(M, 256, seed=9, scale=2.0), 1.0 + rnd(256, seed=10, scale=0.1)
        w = rnd(300, 256, dtype=wdt, seed=11, scale=0.1)
        x = (h.double() / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)) * g.double()
        out = kernels.linear(kernels.PendingNorm(h, g, eps, odt), w, out_dtype=torch.float32)
        close(out, x @ w.double().T, 8e-3 if odt == torch.bfloat16 else 1e-5, f"pending norm, {M} rows")


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_tc_accumulate_with_a_short_last_round(mode):
    """More tiles than SMs with a remainder: the residual product cuts the last round's tiles along K and the
    shares add up in C (16 x 14 = 224 tiles of 128 x 256, as o_proj at 2,048 tokens of the 7B shape)."""
    from tq_kv_b200 import kernels
    M, N, K = 2048, 3584, 1024
    x, w, bias = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1), rnd(N, seed=2)
    base = rnd(M, N, seed=3)
    out = base.clone()
    kernels.set_gemm_tc_mode(mode)
    try:
        kernels.gemm_tc(x, w, out, bias, kernels.gemm.EPI_ACCUM)
        kernels.check_tc_status()
    finally:
        kernels.set_gemm_tc_mode(0)
    want = base.double() + x.double() @ w.double().T + bias.double()
    close(out, want, 2e-6 * math.sqrt(K), "accumulate, split last round")


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_tc_under_load(mode):
    """Thousands of tiles per launch, several launches: every block walks many tiles through its stages, its two
    accumulators and its epilogue buffers, which is where a mistake in the order of waits would show."""
    from tq_kv_b200 import kernels
    M, K = 8192, 5120
    x = rnd(M, K, dtype=torch.bfloat16)
    kernels.set_gemm_tc_mode(mode)
    try:
        for rep in range(2):
            for N, epi in ((5120, kernels.gemm.EPI_ACCUM), (7168, kernels.gemm.EPI_STORE), (6912, kernels.gemm.EPI_SWIGLU)):
                rows = 2 * N if epi == kernels.gemm.EPI_SWIGLU else N
                w = rnd(rows, K, dtype=torch.bfloat16, seed=7 * rep + N, scale=1.0 / math.sqrt(K))
                y = x.float() @ w.float().T
                if epi == kernels.gemm.EPI_ACCUM:
                    base = rnd(M, N, seed=3)
                    out, want, tol = base.clone(), base + y, 2e-4
                elif epi == kernels.gemm.EPI_STORE:
                    out, want, tol = torch.full((M, N), 7.0, device=DEV), y, 2e-4
                else:
                    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
                    want, tol = torch.nn.functional.silu(y[:, :N]) * y[:, N:], 4e-2
                kernels.gemm_tc(x, w, out, None, epi)
                kernels.check_tc_status()
                err = float((out.float() - want).abs().max())
                assert err <= tol, f"mode {mode}, N {N}, epilogue {epi}, launch {rep}: {err:.3e}"
    finally:
        kernels.set_gemm_tc_mode(0)


def test_a_wait_that_ran_out_is_reported_by_the_host_check():
    """The tcgen05 kernels bound every mbarrier wait and raise a status bit instead of hanging.  No wait is made
    to run out here (that would need a kernel that misbehaves on purpose); the status word is set by hand and the
    host-side check must turn it into an error and clear it."""
    from tq_kv_b200 import kernels
    x, w = rnd(128, 64, dtype=torch.bfloat16), rnd(256, 64, dtype=torch.bfloat16, seed=1)
    out = torch.empty(128, 256, device=DEV)
    kernels.gemm_tc(x, w, out)
    kernels.check_tc_status()                                        # a healthy launch passes
    kernels.gemm_tc(x, w, out)
    kernels._lib.tc_status_word(x.device).fill_(2)
    with pytest.raises(kernels.KernelError, match="wait ran out"):
        kernels.check_tc_status()
    kernels.gemm_tc(x, w, out)
    kernels.check_tc_status()                                        # the word was cleared


# ---- rotary encoding and cache append ----------------------------------------------
@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(5, 5, 48, 48), (6, 2, 80, 32), (3, 1, 16, 16)])
def test_qkv_rope_cache(cache_dtype, nh, nkv, hd, rot):
    from tq_kv_b200 import kernels
    lens, starts = [70 + 128, 3, 1], [0, 130, 64]      # row 0: a prompt; rows 1, 2: continuations
    T, B = sum(lens), 3
    width = (nh + 2 * nkv) * hd
    qkv, bias = rnd(T, width), rnd(width, seed=1)
    cos, sin = pm.rope_tables(rot, 50000.0, 256)
    # (over 128 tokens, so that the 16-byte kernel for many tokens runs where its conditions hold)
    tok_seq = torch.tensor(sum(([b] * n for b, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    pos = sum((list(range(s, s + n)) for s, n in zip(starts, lens)), [])
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    new_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=DEV)
    pages, P = 10, 64
    table = torch.tensor([[4, 7, 0, 9], [1, 8, 2, 9], [3, 5, 6, 9]], dtype=torch.int32, device=DEV)
    kp = torch.zeros(pages, nkv, P, hd, dtype=cache_dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q = torch.empty(T, nh * hd, dtype=cache_dtype, device=DEV)
    k = torch.empty(T, nkv * hd, dtype=cache_dtype, device=DEV)
    v = torch.empty_like(k)
    kernels.qkv_rope_cache(qkv, bias, cos.to(DEV), sin.to(DEV), tok_pos, tok_seq, new_lens, q, n_heads=nh,
                           n_kv_heads=nkv, head_dim=hd, rotary_dim=rot, k_out=k, v_out=v, k_pages=kp, v_pages=vp,
                           block_table=table, table_width=4, ring_pages=0, page_tokens=P)
    x = (qkv + bias).cpu()
    xq = x[:, :nh * hd].reshape(T, nh, hd)
    xk = x[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    xv = x[:, (nh + nkv) * hd:].reshape(T, nkv, hd)

    def rope(t):       # [T, heads, hd] with each token at its own position
        r = torch.stack([pm.rope_halved(t[i:i + 1, :, :rot].transpose(0, 1), cos[p:p + 1], sin[p:p + 1])[:, 0]
                         for i, p in enumerate(pos)])
        return torch.cat([r, t[:, :, rot:]], dim=-1)

    tol = 1e-6 if cache_dtype == torch.float32 else 4e-3
    wq, wk = rope(xq), rope(xk)
    close(q, wq.reshape(T, -1), tol, "q")
    close(k, wk.reshape(T, -1), tol, "k packed")
    close(v, xv.reshape(T, -1), tol, "v packed")
    tbl = table.cpu()
    for i, (b, p) in enumerate(zip(tok_seq.tolist(), pos)):
        page = int(tbl[b, p // P])
        close(kp[page, :, p % P], wk[i], tol, "k cache")
        close(vp[page, :, p % P], xv[i], tol, "v cache")
    written = sum(lens) * nkv * hd
    assert int((vp != 0).sum()) == written               # nothing else was touched
    # the same with the input cleared behind the kernel: equal results, and zeros where qkv was
    q2, kp2, vp2, keep = torch.empty_like(q), torch.zeros_like(kp), torch.zeros_like(vp), qkv.clone()
    kernels.qkv_rope_cache(qkv, bias, cos.to(DEV), sin.to(DEV), tok_pos, tok_seq, new_lens, q2, n_heads=nh,
                           n_kv_heads=nkv, head_dim=hd, rotary_dim=rot, k_pages=kp2, v_pages=vp2,
                           block_table=table, table_width=4, ring_pages=0, page_tokens=P, clear_input=True)
    assert float(qkv.abs().sum()) == 0.0 and float(keep.abs().sum()) > 0
    tight = 0.0 if T < 128 else tol                      # under 128 tokens both calls ran the same kernel
    close(q2, q, tight, "q, input cleared")
    close(kp2, kp, tight, "k cache, input cleared")
    close(vp2, vp, tight, "v cache, input cleared")


def test_ring_keeps_only_the_last_positions_of_a_long_prompt():
    from tq_kv_b200 import kernels
    nh = nkv = 1
    hd, P, ring = 16, 64, 2
    n = 300                                              # 300 tokens onto a ring of 128
    qkv = rnd(n, 3 * hd)
    cos, sin = pm.rope_tables(hd, 1e4, 512)
    tok_pos = torch.arange(n, dtype=torch.int32, device=DEV)
    tok_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
    new_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    table = torch.tensor([[2, 0]], dtype=torch.int32, device=DEV)
    kp = torch.zeros(3, 1, P, hd, device=DEV)
    vp = torch.zeros_like(kp)
    q = torch.empty(n, hd, device=DEV)
    kernels.qkv_rope_cache(qkv, None, cos.to(DEV), sin.to(DEV), tok_pos, tok_seq, new_lens, q, n_heads=1,
                           n_kv_heads=1, head_dim=hd, rotary_dim=hd, k_pages=kp, v_pages=vp, block_table=table,
                           table_width=2, ring_pages=ring, page_tokens=P)
    for p in range(n - ring * P, n):
        page = [2, 0][(p // P) % ring]
        assert torch.equal(vp[page, 0, p % P], qkv[p, 2 * hd:]), p
    assert float(vp[1].abs().sum()) == 0.0


# ---- attention ----------------------------------------------------------------------
def plain_attention(q, k, v, nh, nkv, hd, window, q_pos):
    """q [Tq, nh*hd] at absolute positions q_pos over keys 0..Tk-1, float64."""
    Tq, Tk = q.shape[0], k.shape[0]
    q = q.double().reshape(Tq, nh, hd).transpose(0, 1)
    k = pm.repeat_kv(k.double().reshape(Tk, nkv, hd).transpose(0, 1), nh // nkv)
    v = pm.repeat_kv(v.double().reshape(Tk, nkv, hd).transpose(0, 1), nh // nkv)
    att = q @ k.transpose(1, 2) / math.sqrt(hd)
    i = torch.tensor(q_pos).reshape(-1, 1)
    j = torch.arange(Tk).reshape(1, -1)
    masked = j > i
    if window:
        masked = masked | (j < i - window + 1)
    att = torch.where(masked.unsqueeze(0), torch.full_like(att, float("-inf")), att)
    return (pm.softmax_last_dim(att) @ v).transpose(0, 1).reshape(Tq, nh * hd)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(7, 1, 128, None), (6, 3, 48, 20), (5, 5, 16, None), (16, 2, 256, 33),
                                              (24, 2, 80, None), (4, 2, 64, 70), (3, 3, 96, None), (2, 1, 32, 5),
                                              (14, 2, 128, 129)])
@pytest.mark.parametrize("lens", [[1, 37, 90], [200, 64, 3, 129], [300]])
@pytest.mark.parametrize("flash", ["tcgen05", "mma", "general"])
def test_attention_over_packed_prompts(dtype, nh, nkv, hd, window, lens, flash, monkeypatch):
    """Three kernels for prompts: tcgen05 (heads of 64 and 128), mma.sync (32..128), the general one."""
    from tq_kv_b200 import kernels
    import importlib
    att = importlib.import_module("tq_kv_b200.kernels.attention")   # (the package exports a function of that name)
    monkeypatch.setattr(att, "USE_TC_ATTENTION", flash == "tcgen05")
    flash = flash != "general"
    T = sum(lens)
    q, k, v = rnd(T, nh * hd, dtype=dtype), rnd(T, nkv * hd, dtype=dtype, seed=1), rnd(T, nkv * hd, dtype=dtype, seed=2)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    tok_seq = torch.tensor(sum(([b] * n for b, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(sum((list(range(n)) for n in lens), []), dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=tok_pos, tok_seq=tok_seq,
                      cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=DEV),
                      start_pos=torch.zeros(len(lens), dtype=torch.int32, device=DEV), window=window, k_packed=k,
                      v_packed=v, use_flash=flash)
    for b, n in enumerate(lens):
        a, e = cu[b], cu[b + 1]
        want = plain_attention(q[a:e].cpu(), k[a:e].cpu(), v[a:e].cpu(), nh, nkv, hd, window, list(range(n)))
        close(out[a:e], want, 2e-6 if dtype == torch.float32 else 8e-3, f"row {b}")


def test_tcgen05_prompt_attention_under_load_agrees_with_the_mma_kernel(monkeypatch):
    """A full machine of long chains (40 q heads, eight prompts of 2,048 tokens: 5,120 blocks of up to 32 key
    tiles), several times over: buffers in tensor memory are reused tile after tile, and a mistake in the order
    of the MMAs and waits that share them shows only under load and only sometimes (two such mistakes were
    found this way).  The mma.sync kernel is the reference here (checked against the plain attention above);
    every run must agree with it."""
    from tq_kv_b200 import kernels
    import importlib
    att = importlib.import_module("tq_kv_b200.kernels.attention")
    nh, nkv, hd, lens = 40, 8, 128, [2048] * 8
    T = sum(lens)
    cu = (torch.arange(9, device=DEV) * 2048).int()
    tok_seq = torch.arange(8, device=DEV).repeat_interleave(2048).int()
    tok_pos = torch.arange(2048, device=DEV).repeat(8).int()
    start = torch.zeros(8, dtype=torch.int32, device=DEV)

    def run(q, k, v, tc):
        monkeypatch.setattr(att, "USE_TC_ATTENTION", tc)
        out = torch.empty_like(q)
        kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=tok_pos, tok_seq=tok_seq,
                          cu_seqlens=cu, start_pos=start, window=None, k_packed=k, v_packed=v)
        return out

    for rep in range(6):
        # every other run with a wide spread of scores: rows' maxima then grow late and by a lot, and the
        # blocks' warps take different paths (rescaling the output or not) at different speeds
        q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=10 * rep, scale=3.0 if rep % 2 else 1.0)
        k = rnd(T, nkv * hd, dtype=torch.bfloat16, seed=10 * rep + 1)
        v = rnd(T, nkv * hd, dtype=torch.bfloat16, seed=10 * rep + 2)
        want = run(q, k, v, False).float()
        got = run(q, k, v, True).float()
        kernels.check_tc_status()
        assert torch.isfinite(got).all(), f"run {rep}: non-finite output"
        # both are rounded to bfloat16 at the end: a step of 2^-8 of the value, beside the 8e-3 of the small values
        excess = (got - want).abs() - (8e-3 + 2.0 ** -6 * want.abs())
        assert float(excess.max()) <= 0, f"run {rep}: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("window", [1000, 64, 129])
def test_tcgen05_prompt_attention_with_a_window_over_long_prompts(window, monkeypatch):
    """A window far shorter than the prompt: most key tiles of a block lie outside its range and are never
    loaded, the first and last tiles of the range are cut by the window's edge and by the diagonal."""
    from tq_kv_b200 import kernels
    import importlib
    att = importlib.import_module("tq_kv_b200.kernels.attention")
    nh, nkv, hd, lens = 8, 2, 128, [4096, 3001]
    T = sum(lens)
    cu = torch.tensor([0, 4096, T], dtype=torch.int32, device=DEV)
    tok_seq = torch.cat([torch.zeros(4096), torch.ones(3001)]).int().to(DEV)
    tok_pos = torch.cat([torch.arange(4096), torch.arange(3001)]).int().to(DEV)
    start = torch.zeros(2, dtype=torch.int32, device=DEV)
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=1, scale=2.0)
    k, v = rnd(T, nkv * hd, dtype=torch.bfloat16, seed=2), rnd(T, nkv * hd, dtype=torch.bfloat16, seed=3)
    outs = []
    for tc in (False, True):
        monkeypatch.setattr(att, "USE_TC_ATTENTION", tc)
        out = torch.empty_like(q)
        kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=tok_pos, tok_seq=tok_seq,
                          cu_seqlens=cu, start_pos=start, window=window, k_packed=k, v_packed=v)
        outs.append(out.float())
    kernels.check_tc_status()
    # the mma.sync kernel against the plain attention on a few rows of each prompt, then the two kernels on all
    for b, n in enumerate(lens):
        a = int(cu[b])
        rows = [0, 63, 64, window - 1, window, window + 1, n // 2, n - 1]
        want = plain_attention(q[a:a + n].cpu()[rows], k[a:a + n].cpu(), v[a:a + n].cpu(), nh, nkv, hd, window, rows)
        close(outs[0][a:a + n][rows], want, 1.6e-2, f"mma, prompt {b}")
    excess = (outs[1] - outs[0]).abs() - (8e-3 + 2.0 ** -6 * outs[0].abs())
    assert float(excess.max()) <= 0, f"{float((outs[1] - outs[0]).abs().max()):.3e}"


def _paged(k, v, nkv, hd, table_row, P=64):
    """Scatters [Tk, nkv*hd] keys/values into pages per `table_row`."""
    n_pages = max(table_row) + 2
    kp = torch.full((n_pages, nkv, P, hd), 1e4, dtype=k.dtype, device=DEV)    # unwritten rows hold junk, not zeros
    vp = torch.full_like(kp, 1e4)
    for j in range(k.shape[0]):
        kp[table_row[j // P], :, j % P] = k[j].reshape(nkv, hd)
        vp[table_row[j // P], :, j % P] = v[j].reshape(nkv, hd)
    return kp, vp


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window,n_splits", [(28, 4, 128, None, 1), (28, 4, 128, None, 5),
                                                       (3, 1, 32, 100, 3), (6, 6, 48, None, 7),
                                                       (12, 2, 96, None, 4), (32, 2, 64, 50, 2), (9, 9, 128, 1, 1),
                                                       (8, 2, 64, None, 40)])       # more splits than a warp has lanes
@pytest.mark.parametrize("flash", [True, False])
def test_attention_over_the_paged_cache_with_splits(dtype, nh, nkv, hd, window, n_splits, flash):
    from tq_kv_b200 import kernels
    Tk = 700
    k, v = rnd(Tk, nkv * hd, dtype=dtype, seed=1), rnd(Tk, nkv * hd, dtype=dtype, seed=2)
    table_row = [9, 3, 0, 11, 5, 7, 2, 10, 1, 6, 4]
    kp, vp = _paged(k, v, nkv, hd, table_row)
    q_pos = [699, 64, 0, 511]                          # four "sequences" sharing the pages, of different lengths
    B = len(q_pos)
    q = rnd(B, nh * hd, dtype=dtype)
    table = torch.tensor([table_row] * B, dtype=torch.int32, device=DEV)
    scratch = torch.empty(kernels.split_scratch_floats(B, nh, hd, n_splits), device=DEV) if n_splits > 1 else None
    out = torch.empty_like(q)
    kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                      tok_pos=torch.tensor(q_pos, dtype=torch.int32, device=DEV),
                      tok_seq=torch.arange(B, dtype=torch.int32, device=DEV),
                      cu_seqlens=torch.arange(B + 1, dtype=torch.int32, device=DEV),
                      start_pos=torch.tensor(q_pos, dtype=torch.int32, device=DEV), window=window,
                      k_pages=kp, v_pages=vp, block_table=table, table_width=len(table_row),
                      n_splits=n_splits, scratch=scratch, use_flash=flash)
    want = torch.cat([plain_attention(q[b:b + 1].cpu(), k[:p + 1].cpu(), v[:p + 1].cpu(), nh, nkv, hd, window, [p])
                      for b, p in enumerate(q_pos)])
    close(out, want, 2e-6 if dtype == torch.float32 else 8e-3, "paged")


@pytest.mark.parametrize("n_splits", [1, 6])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_among_hundreds_is_found(n_splits, dtype):
    """Random scores are nearly flat, so a dropped key would hardly show.  Here
    one key far back (position 3 of 700) matches the query strongly and its
    value is distinct: the output must be that value."""
    from tq_kv_b200 import kernels
    nh, nkv, hd, Tk = 4, 2, 64, 700
    k, v = rnd(Tk, nkv * hd, scale=0.1, seed=1, dtype=dtype), rnd(Tk, nkv * hd, scale=0.1, seed=2, dtype=dtype)
    q = rnd(1, nh * hd, scale=0.1, dtype=dtype)
    k[3] = 0
    k[3, :hd] = 8.0
    k[3, hd:] = 8.0
    q[:] = 8.0
    v[3] = 5.0
    table_row = list(range(11))
    kp, vp = _paged(k, v, nkv, hd, table_row)
    scratch = torch.empty(kernels.split_scratch_floats(1, nh, hd, n_splits), device=DEV) if n_splits > 1 else None
    out = torch.empty_like(q)
    args = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=torch.tensor([699], dtype=torch.int32, device=DEV),
                tok_seq=torch.zeros(1, dtype=torch.int32, device=DEV),
                cu_seqlens=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                start_pos=torch.tensor([699], dtype=torch.int32, device=DEV), k_pages=kp, v_pages=vp,
                block_table=torch.tensor([table_row], dtype=torch.int32, device=DEV), table_width=11,
                n_splits=n_splits, scratch=scratch)
    kernels.attention(q, out, window=None, **args)
    assert float((out.float() - 5.0).abs().max()) < 1e-3
    # the window's edge: with 697 keys in view key 3 is the oldest one seen, with 696 it is out
    kernels.attention(q, out, window=697, **args)
    assert float((out.float() - 5.0).abs().max()) < 1e-3
    kernels.attention(q, out, window=696, **args)
    assert float(out.float().abs().max()) < 1.0


def test_prompt_chunks_attend_over_the_paged_cache():
    dtype = torch.bfloat16
    # Two sequences continued by 70 and 9 tokens at positions 130 and 64: the
    # 64-query kernel reads earlier keys (and the chunk's own) from the pages.
    from tq_kv_b200 import kernels
    nh, nkv, hd, P = 6, 2, 64, 64
    starts, lens = [130, 64], [70, 9]
    ks = [rnd(s + n, nkv * hd, dtype=dtype, seed=10 + i) for i, (s, n) in enumerate(zip(starts, lens))]
    vs = [rnd(s + n, nkv * hd, dtype=dtype, seed=20 + i) for i, (s, n) in enumerate(zip(starts, lens))]
    tables = [[5, 2, 7, 0], [1, 6, 3, 4]]
    kp = torch.full((8, nkv, P, hd), 1e4, dtype=dtype, device=DEV)
    vp = torch.full_like(kp, 1e4)
    for b in range(2):
        for j in range(ks[b].shape[0]):
            kp[tables[b][j // P], :, j % P] = ks[b][j].reshape(nkv, hd)
            vp[tables[b][j // P], :, j % P] = vs[b][j].reshape(nkv, hd)
    T = sum(lens)
    q = rnd(T, nh * hd, dtype=dtype)
    pos = sum((list(range(s, s + n)) for s, n in zip(starts, lens)), [])
    import importlib
    att = importlib.import_module("tq_kv_b200.kernels.attention")
    for window in (None, 100):
        for flash in ("tcgen05", "mma", "general"):
            att.USE_TC_ATTENTION = flash == "tcgen05"
            flash = flash != "general"
            out = torch.empty_like(q)
            kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                              tok_pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
                              tok_seq=torch.tensor([0] * 70 + [1] * 9, dtype=torch.int32, device=DEV),
                              cu_seqlens=torch.tensor([0, 70, 79], dtype=torch.int32, device=DEV),
                              start_pos=torch.tensor(starts, dtype=torch.int32, device=DEV), window=window,
                              k_pages=kp, v_pages=vp, block_table=torch.tensor(tables, dtype=torch.int32, device=DEV),
                              table_width=4, use_flash=flash)
            a = 0
            for b in range(2):
                want = plain_attention(q[a:a + lens[b]].cpu(), ks[b].cpu(), vs[b].cpu(), nh, nkv, hd, window,
                                       list(range(starts[b], starts[b] + lens[b])))
                close(out[a:a + lens[b]], want, 8e-3, f"row {b}, window {window}, flash {flash}")
                a += lens[b]
    att.USE_TC_ATTENTION = True
    kernels.check_tc_status()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
def test_ring_cache_decoding_reads_the_right_rows(dtype, tol):
    """A window of 100 on a ring of 2 pages: position 300 sees 201..300, which
    lie in ring rows (p % 128) of two physical pages."""
    from tq_kv_b200 import kernels
    nh, nkv, hd, W, P, ring = 2, 1, 32, 100, 64, 2
    n = 301
    k, v = rnd(n, hd, seed=1, dtype=dtype), rnd(n, hd, seed=2, dtype=dtype)
    kp = torch.full((4, 1, P, hd), 1e4, device=DEV, dtype=dtype)
    vp = torch.full_like(kp, 1e4)
    phys = [3, 1]
    for p in range(n - ring * P, n):
        kp[phys[(p // P) % ring], 0, p % P] = k[p]
        vp[phys[(p // P) % ring], 0, p % P] = v[p]
    q = rnd(1, nh * hd, dtype=dtype)
    out = torch.empty_like(q)
    kernels.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                      tok_pos=torch.tensor([300], dtype=torch.int32, device=DEV),
                      tok_seq=torch.zeros(1, dtype=torch.int32, device=DEV),
                      cu_seqlens=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                      start_pos=torch.tensor([300], dtype=torch.int32, device=DEV), window=W, k_pages=kp, v_pages=vp,
                      block_table=torch.tensor([phys], dtype=torch.int32, device=DEV), table_width=2,
                      ring_pages=ring)
    want = plain_attention(q.cpu(), k.cpu(), v.cpu(), nh, nkv, hd, W, [300])
    close(out, want, tol, "ring")


def test_sizes_outside_the_kernels_reach_are_refused():
    from tq_kv_b200 import kernels
    with pytest.raises(kernels.KernelError, match="head_dim"):
        kernels.check_head_geometry(4, 2, 24)
    with pytest.raises(kernels.KernelError, match="head_dim"):
        kernels.check_head_geometry(4, 2, 272)
    with pytest.raises(kernels.KernelError, match="shared"):
        kernels.check_head_geometry(5, 2, 64)
    with pytest.raises(kernels.KernelError, match="CUDA"):
        kernels.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-6, torch.zeros(2, 8))


# ---- sampling -----------------------------------------------------------------------
@pytest.mark.parametrize("V", [1000, 50257])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.0, 0, 1.0), (0.8, 0, 1.0), (1.0, 40, 1.0), (0.7, 0, 0.9),
                                                     (0.7, 40, 0.9), (1.5, 5, 0.5), (1.0, 1, 1.0)])
def test_sample_follows_the_plain_sampler(V, temperature, top_k, top_p):
    from tq_kv_b200 import kernels
    R = 6
    logits = rnd(R, V, scale=3.0, seed=V)
    top_p32 = float(torch.tensor(top_p, dtype=torch.float32))
    us = [0.0, 0.13, 0.5, 0.77, 0.999, 0.31]
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    kernels.sample(logits, out, temperature=temperature, top_k=top_k, top_p=top_p,
                   uniforms=torch.tensor(us, device=DEV))
    want = [pm.sample(logits[r].cpu(), temperature, top_k, top_p32, us[r]) for r in range(R)]
    assert out.tolist() == want


@pytest.mark.parametrize("top_k", [0, 40])
def test_draws_made_on_the_device_are_the_host_generators(top_k):
    """With request indices instead of uniforms the kernel generates each row's draw from (seed, request, index
    of the sampled token): the same tokens as with the host generator's numbers, whatever row a request sits in."""
    from tq_kv_b200 import kernels
    from tq_kv_b200.sampling import uniform
    R, V = 7, 3000
    logits = rnd(R, V, scale=2.0, seed=11)
    requests = [12, 0, 5, 1000003, 7, 3, 2 ** 31 - 1]
    for seed, index in [(0, 0), (1234567890123, 5), (2 ** 64 - 1, 70000)]:
        us = torch.tensor([uniform(seed, r, index) for r in requests], dtype=torch.float32, device=DEV)
        want = torch.zeros(R, dtype=torch.int32, device=DEV)
        kernels.sample(logits, want, temperature=0.9, top_k=top_k, top_p=0.95, uniforms=us)
        got = torch.zeros(R, dtype=torch.int32, device=DEV)
        kernels.sample(logits, got, temperature=0.9, top_k=top_k, top_p=0.95, seed=seed, index=index,
                       requests=torch.tensor(requests, dtype=torch.int32, device=DEV))
        assert got.tolist() == want.tolist()
    assert len(set(want.tolist())) > 1


def test_argmax_ties_go_to_the_lowest_id():
    from tq_kv_b200 import kernels
    logits = torch.zeros(2, 5000, device=DEV)
    logits[0, [4321, 77, 3000]] = 2.0
    logits[1, 4999] = 1.0
    out = torch.zeros(2, dtype=torch.int32, device=DEV)
    kernels.sample(logits, out)
    assert out.tolist() == [77, 4999]


def test_repeat_penalty_counts_every_occurrence():
    from tq_kv_b200 import kernels
    V = 300
    logits = rnd(2, V, scale=2.0, seed=3)
    counts = torch.zeros(2, V, dtype=torch.int32, device=DEV)
    hist = [[5, 9, 5, 200], [17]]
    for r, h in enumerate(hist):
        for t in h:
            counts[r, t] += 1
    before = counts.clone()
    out = torch.zeros(2, dtype=torch.int32, device=DEV)
    us = [0.4, 0.9]
    kernels.sample(logits, out, temperature=0.9, top_k=50, top_p=0.95, uniforms=torch.tensor(us, device=DEV),
                   counts=counts, repeat_penalty=1.3)
    p95 = float(torch.tensor(0.95, dtype=torch.float32))
    want = [pm.sample(pm.apply_repeat_penalty(logits[r].cpu(), hist[r], 1.3), 0.9, 50, p95, us[r]) for r in range(2)]
    assert out.tolist() == want
    before[0, want[0]] += 1
    before[1, want[1]] += 1
    assert torch.equal(counts, before)                   # the chosen tokens were counted
    # greedy with a penalty strong enough to dethrone the best token
    best = int(logits[0].argmax())
    counts.zero_()
    counts[0, best] = 3
    kernels.sample(logits, out, counts=counts, repeat_penalty=50.0)
    assert out.tolist()[0] == pm.greedy(pm.apply_repeat_penalty(logits[0].cpu(), [best] * 3, 50.0)) != best
