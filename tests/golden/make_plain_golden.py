"""Writes tests/golden/plain_tiny_logits.json: logits of the plain
implementation (tests/plain_model.py) on both tiny configurations with seeded
random weights.  The reference's model code cannot be compiled or imported in
this environment (no Rust toolchain), so these values rest on the plain
implementation's reading of the reference's formulas; they guard against
accidental changes of that reading.

    python tests/golden/make_plain_golden.py
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import plain_model as pm  # noqa: E402
from helpers import TINY_A, TINY_B, random_tokens  # noqa: E402
from tq_kv_b200.weights import write_model_folder  # noqa: E402

out = {}
with tempfile.TemporaryDirectory() as tmp:
    for name, cfg, seed in (("a", TINY_A, 21), ("b", TINY_B, 22)):
        folder = write_model_folder(cfg, os.path.join(tmp, name), seed=seed)
        c, w = pm.read_model_folder(folder)
        tokens = random_tokens(40, cfg["vocab_size"], seed)
        logits = pm.decoder_logits(c, w, tokens)
        positions, columns = [0, 1, 15, 16, 17, 39], [0, 1, 2, 100, 255]
        out[name] = {"seed": seed, "tokens": tokens, "positions": positions, "columns": columns,
                     "logits": logits[positions][:, columns].tolist(),
                     "argmax": [int(x) for x in logits.argmax(-1)]}
with open(os.path.join(HERE, "plain_tiny_logits.json"), "w") as f:
    json.dump(out, f)
print("written")
