"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read
back from the files it writes (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")


def run_trace(folder, dtype, steps, out_dir, max_tokens):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
           str(out_dir), "--max-tokens", str(max_tokens)]
    p = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split() == sum((["done", str(s["step"])] for s in steps), [])
    return p


def read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(str(out_dir), f"{step}.f32"), dtype="<f4").reshape(-1, vocab))


def check(got, want, dtype):
    scale = max(1.0, float(want.abs().max()))
    assert got.shape == want.shape and float((got - want).abs().max()) <= TOL[dtype] * scale


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("b", "bfloat16")])
def test_replay_in_three_cuts(tmp_path, name, dtype):
    folder = model_folder(tmp_path, name, dtype)
    V = TINY[name]["vocab_size"]
    reqs = {f"r{i}": random_tokens(n, V, 200 + i) for i, n in enumerate((70, 33, 100))}
    want = {k: plain_logits(folder, t) for k, t in reqs.items()}
    # 1. each request alone and whole; 2. last 32 one by one; 3. an unequal batch whose shorter requests end earlier
    steps, expect = [], {}
    n = 0
    for k, t in reqs.items():
        steps.append({"step": n, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]})
        expect[n] = want[k]
        n += 1
    for k, t in reqs.items():
        cut = len(t) - 32
        steps.append({"step": n, "entries": [{"id": k + "x", "tokens": t[:cut], "want": []}], "end": []})
        n += 1
        for j in range(cut, len(t)):
            steps.append({"step": n, "entries": [{"id": k + "x", "tokens": [t[j]], "want": [0]}],
                          "end": [k + "x"] if j == len(t) - 1 else []})
            expect[n] = want[k][j:j + 1]
            n += 1
    cut = {"r0": 40, "r1": 1, "r2": 64}
    steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][:c], "want": [c - 1]} for k, c in cut.items()],
                  "end": []})
    expect[n] = torch.stack([want[k][c - 1] for k, c in cut.items()])
    n += 1
    live = list(reqs)
    while live:
        ends = [k for k in live if cut[k] + 1 == len(reqs[k])]
        steps.append({"step": n, "entries": [{"id": k, "tokens": [reqs[k][cut[k]]], "want": [0]} for k in live],
                      "end": ends})
        expect[n] = torch.stack([want[k][cut[k]] for k in live])
        n += 1
        for k in live:
            cut[k] += 1
        live = [k for k in live if k not in ends]
    out = tmp_path / f"out_{name}_{dtype}"
    run_trace(folder, dtype, steps, out, max_tokens=64 * (2 + 1 + 2))      # the batch holds 70, 33 and 100 tokens
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(expect)
    for step, w in expect.items():
        check(read(out, step, V), w, dtype)


def test_errors_are_loud(tmp_path):
    folder = model_folder(tmp_path, "a", "float32")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out",
           str(tmp_path / "o"), "--max-tokens", "64"]
    line = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": []}], "end": []})
    p = subprocess.run(cmd, input=line + "\n", capture_output=True, text=True)
    assert p.returncode != 0 and "exceed the context limit 64" in p.stderr
