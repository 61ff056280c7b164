"""Benchmark of the decode step (and of a 2,048-token prefill) of the
Qwen2.5-7B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

Prints ONE JSON line.  `value` is decoded tokens per second at the default
batch, timed on the device with CUDA events around K decode steps that are
launched back to back (tokens are given, nothing waits for the host).  `e2e`
is the same through the Python entry point `Engine.generate()`: token ids go
in from the host and come back to the host every step.  `prefill` is one step
over a 2,048-token prompt; `roofline` relates the decode step's necessary
bytes (every weight it uses once, the cache of the live sequences) to its
time; `points` hold decode at batch 1 and 64.  Peaks come from
MEASURED_PEAKS.json beside this file if it exists, else from an earlier
measurement on the same kind of machine (6.65 TB/s, 1.59 PFLOP/s).

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
    flops of a step."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, I, V = cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    layer_mm = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    layer_small = (nh + 2 * nkv) * hd + 2 * H
    weight_bytes = 2 * (n_layers * (layer_mm + layer_small) + V * H + H)     # the embedding table is not read
    kv_bytes_per_token = 2 * nkv * hd * 2 * n_layers
    return {"layer_mm": layer_mm, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "head_mm": V * H, "attn_flops_per_key": 4 * nh * hd * n_layers}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for profiler captures)")
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
    max_b = args.batch if args.no_points else max(args.batch, 64)
    K, W = args.steps, args.warmup
    # the timed steps sit in the middle of a run from `prompt` to `context` tokens
    span = args.context - args.prompt
    start_ctx = args.prompt + max(0, (span - K - W) // 2)
    if start_ctx + K + W > args.context:
        start_ctx = max(1, args.context - K - W)

    engine = tq.Engine.from_random(cfg, seed=0, dtype="bfloat16", max_slots=max_b, max_context=args.context)
    engine.use_graphs = not args.no_graphs
    gen = torch.Generator().manual_seed(0)
    dev = engine.runtime.device

    def fill(batch: int, ctx: int) -> list[int]:
        slots = [engine.new_sequence() for _ in range(batch)]
        for a in range(0, batch, 4):                       # fill the cache a few rows at a time
            rows = [StepRow(s, torch.randint(0, V, (ctx,), generator=gen).tolist(), []) for s in slots[a:a + 4]]
            engine.step(rows)
        return slots

    def decode_run(batch: int, steps: int, warmup: int):
        """Device time of `steps` decode steps launched back to back."""
        slots = fill(batch, start_ctx)
        sampler = Sampler(tq.GenerationParams.greedy(1), batch, V, dev)
        toks = torch.randint(0, V, (steps + warmup, batch), generator=gen).tolist()

        def one(i):
            logits = engine.step([StepRow(s, [toks[i][r]], [0]) for r, s in enumerate(slots)])
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
        ms = e0.elapsed_time(e1)
        launches = kernels.launches[0] - n0
        for s in slots:
            engine.release(s)
        return ms, launches

    if args.prefill_only:
        T = args.prompt
        for _ in range(2):
            s0 = engine.new_sequence()
            ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepRow(s0, ptoks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            engine.release(s0)
        print(json.dumps({"prefill_ms": round(e0.elapsed_time(e1), 3), "tokens": T, "layers": n_layers}))
        return 0

    with ClockSampler() as clocks:
        ms, launches = decode_run(args.batch, K, W)
    ms_step = ms / K
    value = args.batch * K / (ms / 1e3)
    mean_ctx = start_ctx + W + K / 2
    step_bytes = nums["weight_bytes"] + args.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # end to end through the Python entry point: host token ids in, host token ids out, every step
    prompts = [torch.randint(0, V, (args.prompt,), generator=gen).tolist() for _ in range(args.batch)]
    e2e_steps = min(K, args.context - args.prompt - 1)
    stamps: list[float] = []

    def on_token(i, t):
        if i == args.batch - 1:
            torch.cuda.synchronize()
            stamps.append(time.perf_counter())

    h2d0 = engine.h2d_bytes
    stats: dict = {}
    e2e_value = h2d = d2h = 0.0
    if not args.no_e2e:
        engine.generate(prompts, tq.GenerationParams.greedy(e2e_steps + 1, stop_token_ids=()), on_token=on_token,
                        stats=stats)
        e2e_value = args.batch * (len(stamps) - 1) / (stamps[-1] - stamps[0])
        steps_total = len(stamps)
        h2d = (engine.h2d_bytes - h2d0 + stats.get("h2d_bytes", 0)) / steps_total
        d2h = stats.get("d2h_bytes", 0) / steps_total

    rec = {
        "metric": f"decode tok/s ({args.shape} shape, bf16 random weights)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "gpu_launches": launches,
        "config": {"model": args.shape, "layers": n_layers, "layers_full": full_layers,
                   "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": V, "global_batch": args.batch,
                   "seq_len": args.context, "prompt_len": args.prompt, "decode_ctx_start": start_ctx + W,
                   "parallelism": "single GPU", "weights": "random N(0,0.02) bf16",
                   "l2": f"a step reads {nums['weight_bytes'] / 1e9:.1f} GB of weights, more than the 126 MB L2",
                   "peaks": pk_src},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks.summary(),
    }

    if not args.no_points:
        # prefill: one 2,048-token prompt in one step, logits at its last place
        T = 2048
        s = engine.new_sequence()
        warm = engine.new_sequence()
        engine.step([StepRow(warm, torch.randint(0, V, (T,), generator=gen).tolist(), [T - 1])])
        engine.release(warm)
        ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([StepRow(s, ptoks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        pms = e0.elapsed_time(e1)
        engine.release(s)
        flops = 2 * T * n_layers * nums["layer_mm"] + nums["attn_flops_per_key"] * T * (T + 1) / 2 + 2 * nums["head_mm"]
        peak_tf = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])
        rec["prefill"] = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / 1e12 / peak_tf, 4)}
        points = {}
        for b in (1, 64):
            steps_b = max(16, min(K, 64))
            ms_b, _ = decode_run(b, steps_b, max(3, min(W, 4)))
            points[f"decode_b{b}"] = round(b * steps_b / (ms_b / 1e3), 1)
        rec["points"] = points
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
