"""The plain implementation checked against itself and against its stored
outputs (CPU).  The reference's own model code cannot be built here, so these
tests pin the formulas: properties that must hold, and golden values that
change only when a formula does."""
import json
import math
import os

import pytest
import torch

import plain_model as pm
from helpers import TINY_A, TINY_B, random_tokens
from tq_kv_b200.weights import write_model_folder

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "plain_tiny_logits.json")


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    got = pm.rms_norm(x, w, 0.0)
    r = math.sqrt((9 + 16) / 2)
    assert torch.allclose(got, torch.tensor([[3 / r * 2, 4 / r * 0.5]]))


def test_rope_is_a_rotation_and_relative():
    cos, sin = pm.rope_tables(8, 10000.0, 32)
    assert torch.allclose(cos[0], torch.ones(4)) and torch.allclose(sin[0], torch.zeros(4))
    assert torch.allclose(cos[3, 1], torch.cos(torch.tensor(3.0 / 10000 ** 0.25)))
    q, k = torch.randn(1, 32, 8), torch.randn(1, 32, 8)
    rq, rk = pm.rope_halved(q, cos, sin), pm.rope_halved(k, cos, sin)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    # scores depend on the distance only: same vectors at (5, 2) and (13, 10)
    q1 = pm.rope_halved(q[:, :1].expand(1, 32, 8), cos, sin)
    k1 = pm.rope_halved(k[:, :1].expand(1, 32, 8), cos, sin)
    assert torch.allclose((q1[0, 5] * k1[0, 2]).sum(), (q1[0, 13] * k1[0, 10]).sum(), atol=1e-4)


def test_mask_and_window():
    m = pm.attention_mask(5, None)
    assert m[0].tolist() == [False, True, True, True, True] and not m[4].any()
    m = pm.attention_mask(5, 2)
    assert m[4].tolist() == [True, True, True, False, False]          # sees keys 3 and 4 only


def test_repeat_kv_mapping():
    x = torch.arange(2).float().reshape(2, 1, 1)
    assert pm.repeat_kv(x, 3).flatten().tolist() == [0, 0, 0, 1, 1, 1]


def test_logits_are_causal_and_window_limits_reach(tmp_path):
    for name, cfg in (("a", TINY_A), ("b", TINY_B)):
        folder = write_model_folder(cfg, str(tmp_path / name), seed=11)
        c, w = pm.read_model_folder(folder)
        toks = random_tokens(40, cfg["vocab_size"], 3)
        full = pm.decoder_logits(c, w, toks)
        assert torch.allclose(pm.decoder_logits(c, w, toks[:17]), full[:17], atol=1e-5)
        changed = list(toks)
        changed[0] = (changed[0] + 1) % cfg["vocab_size"]
        other = pm.decoder_logits(c, w, changed)
        assert not torch.allclose(other[1], full[1], atol=1e-6)
    assert [pm.layer_is_windowed(TINY_B, i) for i in range(3)] == [False, True, True]


def test_sampling_rules():
    l = torch.tensor([1.0, 3.0, 3.0, 2.0, -1.0])
    assert pm.greedy(l) == 1                                            # lowest id among ties
    assert pm.sample(l, 0.0, 0, 1.0, 0.99) == 1
    assert pm.sample(l, 1.0, 1, 1.0, 0.0) == 1 and pm.sample(l, 1.0, 1, 1.0, 0.999) == 2   # ties at the k-th stay
    # top-p 0.5: the two 3.0s carry 2e^0 of ~2+e^-1+e^-2+e^-4 -> they alone are kept
    picks = {pm.sample(l, 1.0, 0, 0.5, u) for u in (0.0, 0.3, 0.6, 0.99)}
    assert picks == {1, 2}
    assert pm.sample(l, 1.0, 0, 1.0, 0.999999) == 4
    pen = pm.apply_repeat_penalty(l, [1, 4, 4], 2.0)
    assert pen.tolist() == [1.0, 1.5, 3.0, 2.0, -4.0]                  # once per occurrence


def test_generate_stops_before_emitting_a_stop_token(tmp_path):
    folder = write_model_folder(TINY_A, str(tmp_path / "a"), seed=11)
    c, w = pm.read_model_folder(folder)
    free = pm.generate(c, w, [5, 6, 7], 6)
    assert len(free) == 6
    stop = free[-1]
    stopped = pm.generate(c, w, [5, 6, 7], 6, stop=(stop,))
    assert stopped == free[:free.index(stop)]


def test_golden_values(tmp_path):
    """Stored logits of the plain implementation on both tiny configurations
    (made by tests/golden/make_plain_golden.py)."""
    with open(GOLDEN) as f:
        gold = json.load(f)
    for name, cfg in (("a", TINY_A), ("b", TINY_B)):
        g = gold[name]
        folder = write_model_folder(cfg, str(tmp_path / name), seed=g["seed"])
        c, w = pm.read_model_folder(folder)
        logits = pm.decoder_logits(c, w, g["tokens"])
        got = logits[g["positions"]][:, g["columns"]]
        assert torch.allclose(got, torch.tensor(g["logits"]), atol=2e-6), name
        assert [int(x) for x in logits.argmax(-1)] == g["argmax"]


def test_the_planted_key_decides_the_logits(tmp_path):
    """A check of the tests that use helpers.planted_model(): in the plain
    implementation, a window one key wider or narrower moves the logits at
    the query's two places by the size of the logits themselves, and so does
    taking the far key away; rounding to bfloat16 moves them a hundred times
    less.  An engine that is off by one key therefore cannot pass there."""
    from helpers import TINY_C, TOL, planted_model, planted_tokens
    folder = planted_model(tmp_path, "float32", windowed=True)
    cfg, w = pm.read_model_folder(folder)
    T, W = 150, TINY_C["sliding_window"]
    toks = planted_tokens(T + 1, T - W, [T - 1, T], 5)
    want = pm.decoder_logits(cfg, w, toks)
    scale = float(want.abs().max())
    wider = pm.decoder_logits({**cfg, "sliding_window": W + 1}, w, toks)
    narrower = pm.decoder_logits({**cfg, "sliding_window": W - 1}, w, toks)
    assert float((wider - want)[T].abs().max()) > 0.5 * scale > 10 * TOL["bfloat16"] * scale
    assert float((narrower - want)[T - 1].abs().max()) > 0.5 * scale
    folder = planted_model(tmp_path, "float32", windowed=False)
    cfg, w = pm.read_model_folder(folder)
    toks = planted_tokens(300, 2, [299], 6)
    want = pm.decoder_logits(cfg, w, toks)
    gone = list(toks)
    gone[2] = 3
    assert float((pm.decoder_logits(cfg, w, gone) - want)[299].abs().max()) > 0.3 * float(want.abs().max())
