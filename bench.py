"""Benchmark of the decode step (and of a 2,048-token prefill) of the
Qwen2.5-7B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
                    [--shape qwen2.5-7b|qwen2.5-0.5b|qwen2.5-32b] [--workload equal|unequal]

Prints ONE JSON line.  `value` is decoded tokens per second at the default
batch, timed on the device with CUDA events around K decode steps that are
launched back to back (tokens are given, nothing waits for the host).  `e2e`
is the same through the Python entry point `Engine.generate()`: prompts go in
as host token ids and every step's token ids come back to the host (the loop
reads them one step late, while the device runs the next step); it runs for
at least 128 timed steps whatever K is, after warm-up steps as the device-timed
run has them (`e2e.steps`, `e2e.warmup`).  `prefill`
is one step over a 2,048-token prompt (timed the second time: like every single prompt from position 0 it then
replays the graph captured the first time, the same kernels without the host's launches between them); `roofline` relates the decode step's
necessary bytes (every weight it uses once, the cache of the live sequences)
to its time; `points` hold decode at batch 1 and 64, device-timed and end to
end, and the time to the first token of a 32- and a 2,048-token prompt through
`Engine.generate()` (`ttft_ms_p32`, `ttft_ms_p2048`); `kernels` holds the device time of one decode step and of the prefill by
class of kernel (launched one by one behind a head start of other work, with
events between the classes) and what each class achieves of the measured
peak.  `--workload unequal` is the second benchmark configuration: a batch of
64 prompts with seeded lengths uniform in 64..4,096, prefilled in ONE step,
then 256 decode steps.  Peaks come from MEASURED_PEAKS.json beside this file
if it exists, else from an earlier measurement on the same kind of machine
(6.65 TB/s, 1.59 PFLOP/s).

The reference arm (`--impl reference`) cannot run here: the reference is a
Rust workspace and no Rust toolchain is installed, so it prints its
`unavailable` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if k in d and d[k]:
                    out[k] = float(d[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.samples.append([x.strip() for x in out.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self) -> dict:
        mhz = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        reasons = sorted({n for s in self.samples for n, v in zip(self.NAMES, s[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def model_numbers(cfg: dict, n_layers: int) -> dict:
    """Parameters in matrix products per layer, bytes a decode step must read,
    flops of a step, and the same by class of kernel."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, I, V = cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    per_class = {"qkv": (nh + 2 * nkv) * hd * H, "o": H * nh * hd, "gate_up": 2 * I * H, "down": I * H}
    layer_mm = sum(per_class.values())
    layer_small = (nh + 2 * nkv) * hd + 2 * H
    weight_bytes = 2 * (n_layers * (layer_mm + layer_small) + V * H + H)     # the embedding table is not read
    kv_bytes_per_token = 2 * nkv * hd * 2 * n_layers
    return {"layer_mm": layer_mm, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "head_mm": V * H, "attn_flops_per_key": 4 * nh * hd * n_layers,
            "class_params": {k: v * n_layers for k, v in per_class.items()}}


CLASSES = ["embed", "norms", "qkv", "rotary", "attention", "o", "gate_up", "down", "head", "sampler"]


def class_table(totals_us: dict, prefix: str, nums: dict, pk: dict, *, tokens: int, cached_tokens: float,
                wanted_rows: int, decode: bool, attn_flops: float = 0.0) -> dict:
    """Flat `kernels` entries of one step: microseconds per class, and for the classes with a roofline what
    they reach of it: GB/s over the measured copy bandwidth for a decode step (weights once, the cache),
    TFLOP/s over the measured bf16 peak for a prompt."""
    out = {}
    for c in CLASSES:
        us = totals_us.get(c)
        if us is None:
            continue
        out[f"{prefix}.{c}.us"] = round(us, 1)
        params = nums["class_params"].get(c) if c != "head" else nums["head_mm"]
        if decode:
            nbytes = 2 * params if params else (cached_tokens * nums["kv_bytes_per_token"] if c == "attention" else 0)
            if nbytes:
                gbs = nbytes / (us * 1e-6) / 1e9
                out[f"{prefix}.{c}.gbs"] = round(gbs, 1)
                out[f"{prefix}.{c}.frac"] = round(gbs / pk["hbm_gbs"], 3)
        else:
            rows = wanted_rows if c == "head" else tokens
            flops = 2 * rows * params if params else (attn_flops if c == "attention" else 0)
            if flops and c != "head":
                tf = flops / (us * 1e-6) / 1e12
                out[f"{prefix}.{c}.tflops"] = round(tf, 1)
                out[f"{prefix}.{c}.frac"] = round(tf / pk["bf16_tflops"], 3)
    out[f"{prefix}.sum.us"] = round(sum(v for k, v in totals_us.items() if k in CLASSES), 1)
    return out


def timed_by_class(run, reps: int = 3) -> dict:
    """Median device time by class of `run()` (a step launched kernel by kernel).  The device is first given
    some tens of milliseconds of other work, so that the host has launched the whole step before the device
    reaches it and the events between the classes see the kernels back to back, not the host's pace."""
    import torch
    from tq_kv_b200 import kernels
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    runs = []
    for _ in range(reps):
        torch.cuda.synchronize()
        tl = kernels.Timeline()
        for _ in range(48):
            torch.mm(a, a)
        kernels._lib.timeline = tl
        try:
            tl.mark("start")
            run()
        finally:
            kernels._lib.timeline = None
        runs.append(tl.totals())
    return {k: statistics.median(r.get(k, 0.0) for r in runs) for k in runs[0]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="default 8 (64 with --workload unequal)")
    ap.add_argument("--shape", default="qwen2.5-7b")
    ap.add_argument("--workload", default="equal", choices=["equal", "unequal"],
                    help="equal: prompts of --prompt tokens; unequal: seeded lengths uniform in 64..4096, one prefill step")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--context", type=int, default=None, help="default 4096 (8192 with --workload unequal)")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--e2e-steps", type=int, default=128, help="the end-to-end run takes at least this many steps")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for profiler captures)")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-class kernel times")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prefill alone (profiler captures)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode kernels one by one (for profiler captures)")
    ap.add_argument("--gemm", default=None, choices=["tcgen05", "library"],
                    help="many-row bfloat16 products: this package's tcgen05 kernel or the library (default: the package's choice)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py/pyproject.toml; pip: 'not installable') "
                          "and no cargo/rustc is installed"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    unequal = args.workload == "unequal"
    if args.batch is None:
        args.batch = 64 if unequal else 8
    if args.context is None:
        args.context = 8192 if unequal else 4096

    import torch
    import tq_kv_b200 as tq
    from tq_kv_b200 import kernels
    from tq_kv_b200.engine import StepRow
    from tq_kv_b200.sampling import Sampler

    if args.gemm is not None:
        kernels.gemm.USE_TCGEN05 = args.gemm == "tcgen05"
    cfg = dict(tq.named_shape(args.shape))
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    cfg["max_window_layers"] = n_layers
    V = cfg["vocab_size"]
    pk, pk_src = peaks()
    nums = model_numbers(cfg, n_layers)
    K, W = args.steps, args.warmup
    gen = torch.Generator().manual_seed(0)
    if unequal:
        lengths = torch.randint(64, 4097, (args.batch,), generator=gen).tolist()
        max_b = args.batch
        room = max(K + W, max(args.e2e_steps, K) + max(W, 48) + 1) + 2
        max_tokens = sum(-(-(n + room) // 64) * 64 for n in lengths)
    else:
        lengths = None
        max_b = args.batch if args.no_points else max(args.batch, 64)
        # the cache a full batch of full contexts needs, cut to what fits beside the weights where it must be
        max_tokens = max_b * args.context
        free = torch.cuda.mem_get_info()[0] - nums["weight_bytes"] - 2 * V * cfg["hidden_size"] - (12 << 30)
        fit = int(free // nums["kv_bytes_per_token"]) // 64 * 64
        max_tokens = max(64 * max_b, min(max_tokens, fit))
    # the timed steps sit in the middle of a run from `prompt` to `context` tokens
    span = args.context - args.prompt
    start_ctx = args.prompt + max(0, (span - K - W) // 2)
    if start_ctx + K + W > args.context:
        start_ctx = max(1, args.context - K - W)

    engine = tq.Engine.from_random(cfg, seed=0, dtype="bfloat16", max_slots=max_b, max_context=args.context,
                                   max_tokens=max_tokens)
    engine.use_graphs = not args.no_graphs
    dev = engine.runtime.device

    def fill(ctx_lens: list[int]) -> list[int]:
        """Slots holding that many random tokens each, prefilled a few rows at a time."""
        slots = [engine.new_sequence() for _ in ctx_lens]
        for a in range(0, len(slots), 4):
            rows = [StepRow(s, torch.randint(0, V, (n,), generator=gen).tolist(), [])
                    for s, n in zip(slots[a:a + 4], ctx_lens[a:a + 4])]
            engine.step(rows)
        return slots

    def decode_run(ctx_lens: list[int], steps: int, warmup: int):
        """Device time of `steps` decode steps launched back to back."""
        batch = len(ctx_lens)
        slots = fill(ctx_lens)
        sampler = Sampler(tq.GenerationParams.greedy(1), batch, V, dev)
        toks = torch.randint(0, V, (steps + warmup, batch), generator=gen).tolist()

        def one(i):
            logits = engine.step([StepRow(s, [toks[i][r]], [0]) for r, s in enumerate(slots)], keep_logits=False)
            kernels.sample(logits, sampler.out)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        n0 = kernels.launches[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        engine.check_status()
        ms = e0.elapsed_time(e1)
        launches = kernels.launches[0] - n0
        for s in slots:
            engine.release(s)
        return ms, launches

    e2e_warmup = max(W, 48)

    def e2e_run(prompts: list[list[int]], steps: int):
        """Tokens per second through Engine.generate(): host token ids in, every step's ids back on the host.
        As in the device-timed run, the first steps after the prompts are warm-up and are not timed (right
        after prompts of thousands of tokens the first dozen or two of decode steps run at the lower clocks
        that the prompts' matrix products left behind: 4.2 instead of 3.2 ms at batch 8); then `steps` steps are timed between the arrivals of their
        tokens on the host."""
        stamps: list[float] = []
        B = len(prompts)

        def on_token(i, t):
            stamps.append(time.perf_counter())             # the token is on the host now

        h2d0, stats = engine.h2d_bytes, {}
        engine.generate(prompts, tq.GenerationParams.greedy(e2e_warmup + steps + 1, stop_token_ids=()),
                        on_token=on_token, stats=stats)
        # every request yields the same number of tokens, a round of the batch at a time: the clock starts with
        # the last token of the last warm-up round
        first = e2e_warmup * B - 1
        n_timed = len(stamps) - 1 - first
        value = n_timed / (stamps[-1] - stamps[first])
        rounds = len(stamps) / B
        h2d = (engine.h2d_bytes - h2d0 + stats.get("h2d_bytes", 0)) / rounds
        return value, int(h2d), int(stats.get("d2h_bytes", 0) / rounds), n_timed // B

    def e2e_prompt(steps: int) -> int:
        """Prompt length at which `steps` generated tokens see the same mean context as the device-timed steps."""
        want = start_ctx + W + K / 2 - steps / 2 - e2e_warmup
        return int(max(args.prompt, min(want, args.context - steps - e2e_warmup - 2)))

    def prefill_run(prompt_lens: list[int]):
        """One step over prompts of these lengths, logits at each prompt's last place; after one warm-up."""
        ms = 0.0
        for _ in range(2):
            slots = [engine.new_sequence() for _ in prompt_lens]
            rows = [StepRow(s, torch.randint(0, V, (n,), generator=gen).tolist(), [n - 1])
                    for s, n in zip(slots, prompt_lens)]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step(rows)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            for s in slots:
                engine.release(s)
        T = sum(prompt_lens)
        attn = nums["attn_flops_per_key"] * sum(n * (n + 1) / 2 for n in prompt_lens)
        flops = 2 * T * n_layers * nums["layer_mm"] + attn + 2 * len(prompt_lens) * nums["head_mm"]
        return ms, T, flops, attn

    if args.prefill_only:
        ms, T, _, _ = prefill_run([args.prompt])
        print(json.dumps({"prefill_ms": round(ms, 3), "tokens": T, "layers": n_layers}))
        return 0

    ctx_lens = [n + 1 for n in lengths] if unequal else [start_ctx] * args.batch
    with ClockSampler() as clocks:
        ms, launches = decode_run(ctx_lens, K, W)
    ms_step = ms / K
    value = args.batch * K / (ms / 1e3)
    mean_cached = sum(ctx_lens) + args.batch * (W + K / 2)          # tokens in the cache, mean over the timed steps
    step_bytes = nums["weight_bytes"] + mean_cached * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    rec = {
        "metric": f"decode tok/s ({args.shape} shape, bf16 random weights)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "gpu_launches": launches,
        "config": {"model": args.shape, "layers": n_layers, "layers_full": full_layers,
                   "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": V, "global_batch": args.batch,
                   "seq_len": args.context,
                   "prompt_len": "uniform 64..4096, seed 0" if unequal else args.prompt,
                   "decode_ctx_start": round(sum(ctx_lens) / args.batch) + W,
                   "cache_tokens": engine.cache.groups[0].book.n_pages * 64,
                   "parallelism": "single GPU", "weights": "random N(0,0.02) bf16",
                   "l2": f"a step reads {step_bytes / 1e9:.1f} GB of weights and cache, more than the 126 MB L2",
                   "peaks": pk_src},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks.summary(),
    }

    # end to end through the Python entry point
    e2e_steps = max(args.e2e_steps, K)
    if not args.no_e2e:
        if unequal:
            prompts = [torch.randint(0, V, (n,), generator=gen).tolist() for n in lengths]
        else:
            e2e_steps = min(e2e_steps, args.context - args.prompt - e2e_warmup - 2)
            prompts = [torch.randint(0, V, (e2e_prompt(e2e_steps),), generator=gen).tolist()
                       for _ in range(args.batch)]
        ev, h2d, d2h, n = e2e_run(prompts, e2e_steps)
        rec["e2e"] = {"value": round(ev, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "steps": n, "warmup": e2e_warmup}
    else:
        rec["e2e"] = {"value": 0.0, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "steps": 0}

    peak_tf = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])
    if not args.no_points:
        # prefill: one 2,048-token prompt in one step (or, unequal workload, the whole batch's prompts in one step)
        plens = lengths if unequal else [2048]
        pms, T, flops, attn_flops = prefill_run(plens)
        rec["prefill"] = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / 1e12 / peak_tf, 4)}
        if not unequal:
            points = {}
            for b in (1, 64):
                steps_b = max(64, min(K, 128))
                ms_b, _ = decode_run([start_ctx] * b, steps_b, max(W, 16))      # (the clocks settle, as for e2e)
                points[f"decode_b{b}"] = round(b * steps_b / (ms_b / 1e3), 1)
                if not args.no_e2e:
                    n_e2e = min(args.e2e_steps, args.context - args.prompt - e2e_warmup - 2)
                    prompts = [torch.randint(0, V, (e2e_prompt(n_e2e),), generator=gen).tolist() for _ in range(b)]
                    points[f"e2e_b{b}"] = round(e2e_run(prompts, n_e2e)[0], 1)
            if not args.no_e2e:
                # time to the first token of one request, host to host (the reference's tables quote it for a
                # short chat prompt, BENCHMARK.md:186-194): a 32-token and a 2,048-token prompt, best of five
                for n in (32, 2048):
                    if n + 2 > args.context:
                        continue
                    best = float("inf")
                    for _ in range(6):
                        prompt = torch.randint(0, V, (n,), generator=gen).tolist()
                        torch.cuda.synchronize()
                        t0 = time.perf_counter()
                        engine.generate([prompt], tq.GenerationParams.greedy(1, stop_token_ids=()))
                        best = min(best, time.perf_counter() - t0)
                    points[f"ttft_ms_p{n}"] = round(best * 1e3, 3)
            rec["points"] = points

    if not args.no_kernels:
        # device time by class of kernel: one decode step and the prefill, launched kernel by kernel
        graphs = engine.use_graphs
        engine.use_graphs = False
        try:
            slots = fill(ctx_lens)
            sampler = Sampler(tq.GenerationParams.greedy(1), args.batch, V, dev)
            tok = torch.randint(0, V, (args.batch,), generator=gen).tolist()

            def one_decode():
                logits = engine.step([StepRow(s, [t], [0]) for s, t in zip(slots, tok)], check=False)
                kernels.sample(logits, sampler.out)
                kernels.mark("sampler")

            one_decode()
            kern = class_table(timed_by_class(one_decode), "decode", nums, pk, tokens=args.batch,
                               cached_tokens=sum(ctx_lens) + 3 * args.batch, wanted_rows=args.batch, decode=True)
            for s in slots:
                engine.release(s)
            if not args.no_points:
                plens = lengths if unequal else [2048]
                ptoks = [torch.randint(0, V, (n,), generator=gen).tolist() for n in plens]
                held: list = []

                def one_prefill():
                    for s in held:
                        engine.release(s)
                    held[:] = [engine.new_sequence() for _ in plens]
                    engine.step([StepRow(s, t, [len(t) - 1]) for s, t in zip(held, ptoks)], check=False)

                one_prefill()
                attn = nums["attn_flops_per_key"] * sum(n * (n + 1) / 2 for n in plens)
                kern.update(class_table(timed_by_class(one_prefill), "prefill", nums, pk, tokens=sum(plens),
                                        cached_tokens=0, wanted_rows=len(plens), decode=False, attn_flops=attn))
                for s in held:
                    engine.release(s)
            engine.check_status()
            rec["kernels"] = kern
        finally:
            engine.use_graphs = graphs
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
