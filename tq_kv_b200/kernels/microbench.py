"""Times single kernels with CUDA events: `python -m tq_kv_b200.kernels.microbench <what> ...`.

  gemm        the many-row product (csrc/gemm_tc.cu) at one shape, on single SMs and on pairs, alternating
  decode-gemm the decode products (csrc/decode_gemm_tc.cu, csrc/skinny_gemm.cu) of a layer shape at one batch size
  attention   the prompt attention (csrc/flash_prefill_tc.cu) for prompts of given lengths
  decode-attention  the attention of one decoded token per sequence over the paged cache
              (csrc/flash_decode.cu and the merge of its splits) at one batch size and context

Every timing loops over several copies of the large operand, so that it is read from memory and not from the L2,
after three warm-up launches.  The numbers explain bench.py's; they are not a benchmark of the engine.
"""
from __future__ import annotations

import argparse

import torch

from . import gemm
from ._lib import check_tc_status

DEV = "cuda"


def _time(fn, n_variants: int, reps: int, graph: bool = False) -> float:
    """Mean microseconds of fn(i) over reps * n_variants launches.  With `graph`, one round over the variants
    is captured into a CUDA graph and replayed, so that kernels of a few microseconds are not timed at the
    pace of their launches from Python."""
    for i in range(min(3, n_variants)):
        fn(i)
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_variants):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        if g is not None:
            g.replay()
            continue
        for i in range(n_variants):
            fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * n_variants)


def _copies(rows: int, cols: int, scale: float) -> list[torch.Tensor]:
    n = max(2, min(12, int(600e6 // (rows * cols * 2)) + 1))        # > 600 MB in all: far more than the L2
    return [torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16) * scale for _ in range(n)]


def bench_gemm(args) -> None:
    M, N, K = args.rows, args.out, args.inner
    epi = {"store": gemm.EPI_STORE, "accumulate": gemm.EPI_ACCUM, "swiglu": gemm.EPI_SWIGLU}[args.epilogue]
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    ws = _copies(2 * N if epi == gemm.EPI_SWIGLU else N, K, 0.02)
    out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16 if epi == gemm.EPI_SWIGLU else torch.float32)
    flop = 2.0 * M * ws[0].shape[0] * K
    for turn in range(args.turns):
        for mode, name in ((1, "single SMs"), (2, "pairs of SMs")):
            gemm.set_gemm_tc_mode(mode)
            us = _time(lambda i: gemm.gemm_tc(x, ws[i], out, epilogue=epi), len(ws), args.reps)
            print(f"gemm_tc {M} x {N} x {K} {args.epilogue:10s} {name:12s} {us:8.1f} us  {flop / us / 1e6:7.1f} TFLOP/s")
    gemm.set_gemm_tc_mode(0)
    check_tc_status()


def bench_decode_gemm(args) -> None:
    M, H, I, V = args.batch, args.hidden, args.intermediate, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("q|k|v", qkv, H, False, False), ("o", H, args.heads * args.head_dim, True, False),
              ("gate|up", I, H, False, True), ("down", H, I, True, False), ("lm head", V, H, False, False)]
    for name, N, K, acc, swiglu in shapes:
        ws = _copies(2 * N if swiglu else N, K, 0.02)
        x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16 if swiglu else torch.float32)
        us = _time(lambda i: gemm.linear(x, ws[i], out=out, accumulate=acc, swiglu=swiglu), len(ws), args.reps,
                   graph=True)         # small products are otherwise timed at the pace of Python's launches
        print(f"{name:8s} {M} x {N} x {K}  {us:8.1f} us  {ws[0].numel() * 2 / us / 1e6:5.2f} TB/s of weights")
    check_tc_status()


def bench_attention(args) -> None:
    from . import attention                     # the package's function of that name
    nh, nkv, hd, lens = args.heads, args.kv_heads, args.head_dim, args.lengths
    T = sum(lens)
    q = torch.randn(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, nkv * hd, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, nkv * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    start = torch.zeros(len(lens), dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(n) for n in lens]).int().to(DEV)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().to(DEV)
    us = _time(lambda i: attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=pos, tok_seq=seq,
                                   cu_seqlens=cu, start_pos=start, window=None, k_packed=k, v_packed=v), 1, args.reps)
    flop = sum(4.0 * nh * hd * n * (n + 1) / 2 for n in lens)
    print(f"attention {nh} q / {nkv} kv heads of {hd}, prompts {lens}: {us:8.1f} us  {flop / us / 1e6:7.1f} TFLOP/s (causal)")
    check_tc_status()


def bench_decode_attention(args) -> None:
    import importlib
    att = importlib.import_module(__package__ + ".attention")   # (the package also exports a function of that name)
    B, T, nh, nkv, hd = args.batch, args.context, args.heads, args.kv_heads, args.head_dim
    width = -(-T // 64)
    n_pages = B * width
    copy_bytes = 2 * n_pages * nkv * 64 * hd * 2
    n = max(2, min(16, int(600e6 // copy_bytes) + 1))
    caches = [(torch.randn(n_pages, nkv, 64, hd, device=DEV, dtype=torch.bfloat16),
               torch.randn(n_pages, nkv, 64, hd, device=DEV, dtype=torch.bfloat16)) for _ in range(n)]
    table = torch.randperm(n_pages, device=DEV).reshape(B, width).to(torch.int32)
    q = torch.randn(B, nh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.full((B,), T - 1, dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = att.plan_splits(B, nkv, args.plan_context or T, sms)
    scratch = torch.empty(att.split_scratch_floats(B, nh, hd, splits), device=DEV) if splits > 1 else None

    def run(i):
        k, v = caches[i]
        att.attention(q, out, n_heads=nh, n_kv_heads=nkv, head_dim=hd, tok_pos=pos, tok_seq=seq, cu_seqlens=cu,
                      start_pos=pos, window=None, k_pages=k, v_pages=v, block_table=table, table_width=width,
                      n_splits=splits, scratch=scratch)

    us = _time(run, n, args.reps, graph=True)
    read = B * T * nkv * hd * 2 * 2
    print(f"decode attention, batch {B}, {T} cached tokens, {nh}/{nkv} heads of {hd}, {splits} splits: {us:8.1f} us, "
          f"{read / 1e6:.1f} MB of keys and values, {read / us / 1e3:.0f} GB/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tq_kv_b200.kernels.microbench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--rows", type=int, default=2048)
    g.add_argument("--out", type=int, default=18944)
    g.add_argument("--inner", type=int, default=3584)
    g.add_argument("--epilogue", choices=["store", "accumulate", "swiglu"], default="swiglu")
    g.add_argument("--turns", type=int, default=2, help="how often the two forms take turns")
    g.add_argument("--reps", type=int, default=5)
    g.set_defaults(fn=bench_gemm)
    d = sub.add_parser("decode-gemm")
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--hidden", type=int, default=3584)
    d.add_argument("--intermediate", type=int, default=18944)
    d.add_argument("--vocab", type=int, default=152064)
    d.add_argument("--heads", type=int, default=28)
    d.add_argument("--kv-heads", type=int, default=4)
    d.add_argument("--head-dim", type=int, default=128)
    d.add_argument("--reps", type=int, default=5)
    d.set_defaults(fn=bench_decode_gemm)
    a = sub.add_parser("attention")
    a.add_argument("--heads", type=int, default=28)
    a.add_argument("--kv-heads", type=int, default=4)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--lengths", type=int, nargs="+", default=[2048])
    a.add_argument("--reps", type=int, default=20)
    a.set_defaults(fn=bench_attention)
    da = sub.add_parser("decode-attention")
    da.add_argument("--batch", type=int, default=8)
    da.add_argument("--context", type=int, default=3072)
    da.add_argument("--plan-context", type=int, default=4096,
                    help="the context the splits are planned for, as a replayed graph plans them (0: --context)")
    da.add_argument("--heads", type=int, default=28)
    da.add_argument("--kv-heads", type=int, default=4)
    da.add_argument("--head-dim", type=int, default=128)
    da.add_argument("--reps", type=int, default=20)
    da.set_defaults(fn=bench_decode_attention)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    args.fn(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
