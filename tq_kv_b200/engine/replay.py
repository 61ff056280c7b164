"""Trace replay: feeds given token ids through an engine step by step and
writes the logits at the wanted places.  Nothing is sampled.  It drives the
engine's own step function, cache and kernels — the ones generation uses.

Input, one JSON object per line:
  {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` give each request's next tokens and the places among them whose
logits are wanted; `end` lists requests that are finished after the step (what
they hold is given back).  For a step that wants something, the float32
logits [wanted, vocab] are written little-endian to `<out>/<step>.f32`; after
every step a line `done <step>` is printed and flushed.

Reference: src/engine.rs:485-521 (perplexity) feeds a text token by token and
:365-366 feeds a prompt whole; this tool can replay either cut.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Iterable

import numpy as np

from .batch import StepRow
from .engine import Engine


class TraceError(ValueError):
    pass


def replay(engine: Engine, lines: Iterable[str], out_dir: str, done: IO[str] = sys.stdout) -> int:
    """Runs the steps read from `lines`; returns the number of steps run."""
    os.makedirs(out_dir, exist_ok=True)
    slots: dict[str, int] = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        try:
            obj = json.loads(line)
        except json.JSONDecodeError as e:
            raise TraceError(f"trace line {n + 1} is not JSON: {e}") from e
        step = obj["step"]
        rows = []
        new_ids = []
        for e in obj.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_sequence()
                new_ids.append(rid)
            rows.append(StepRow(slots[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if rows:
            try:
                logits = engine.step(rows)
            except Exception:
                for rid in new_ids:            # a refused step leaves nothing behind
                    engine.release(slots.pop(rid))
                raise
            engine.check_status()              # no logits leave here from a kernel that gave up on a wait
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in obj.get("end", []):
            rid = str(rid)
            if rid not in slots:
                raise TraceError(f"step {step} ends request '{rid}', which is not live")
            engine.release(slots.pop(rid))
        n += 1
        print(f"done {step}", file=done, flush=True)
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device, max_tokens=args.max_tokens)
    replay(engine, sys.stdin, args.out)
    return 0
