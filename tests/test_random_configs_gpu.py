"""Seeded random configurations of the architecture against the plain
implementation (GPU): every size and option is drawn anew — head sizes in
steps of 16, head counts and groups, widths and vocabularies that are no power
of two, depth, eps, theta, tied or untied head, windows that start at any
layer — and every configuration is run in float32 and bfloat16, cut three
ways: whole, prefix + one token at a time, and an unequal batch that continues
token by token."""
import os
import random

import pytest
import torch

import plain_model
from helpers import assert_close

pytestmark = pytest.mark.gpu

N_CONFIGS = 14


def draw_config(seed: int) -> dict:
    r = random.Random(seed)
    head_dim = 16 * (1 + seed % 8)                      # every head size from 16 to 128 comes up
    n_kv = r.choice([1, 2, 3, 4])
    group = r.choice([1, 2, 3, 5, 7])
    n_heads = n_kv * group
    hidden = 8 * r.randint(5, 24)                       # 40 .. 192, mostly no power of two, not heads * head_dim
    layers = r.randint(1, 4)
    window = r.choice([None, 8, 24, 70])
    return {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "float32",
        "num_hidden_layers": layers, "hidden_size": hidden, "num_attention_heads": n_heads,
        "num_key_value_heads": n_kv, "head_dim": head_dim, "intermediate_size": 8 * r.randint(4, 40),
        "vocab_size": r.randint(50, 700), "rope_theta": r.choice([1e4, 5e5, 1e6]),
        "rms_norm_eps": r.choice([1e-6, 1e-5, 3e-4]), "tie_word_embeddings": r.random() < 0.5,
        "use_sliding_window": window is not None, "sliding_window": window,
        "max_window_layers": r.randint(0, layers), "max_position_embeddings": 512,
    }


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("random_models")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(N_CONFIGS))
def test_random_configuration(tmp_root, seed, dtype):
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.weights import write_model_folder
    cfg = draw_config(1000 + seed)
    cfg["torch_dtype"] = dtype
    folder = os.path.join(str(tmp_root), f"cfg{seed}_{dtype}")
    write_model_folder(cfg, folder, seed)
    pcfg, weights = plain_model.read_model_folder(folder)
    g = torch.Generator().manual_seed(seed)
    lengths = [int(torch.randint(3, 150, (1,), generator=g)) for _ in range(3)]
    reqs = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    want = [plain_model.decoder_logits(pcfg, weights, t, torch.float32).float() for t in reqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512)
    what = f"seed {seed}: {cfg}"

    # whole
    for t, w in zip(reqs, want):
        s = eng.new_sequence()
        got = eng.step([StepRow(s, t, list(range(len(t))))])
        eng.release(s)
        assert_close(got, w, dtype, "whole, " + what)

    # a prefix, then one token at a time
    t, w = reqs[0], want[0]
    n = max(1, len(t) - 20)
    s = eng.new_sequence()
    outs = [eng.step([StepRow(s, t[:n], [n - 1])])] + [eng.step([StepRow(s, [x], [0])]) for x in t[n:]]
    eng.release(s)
    assert_close(torch.cat(outs), w[n - 1:], dtype, "token by token, " + what)

    # an unequal batch: prompts cut at different places, then token by token until each request ends
    cut = [max(1, len(t) // (i + 2)) for i, t in enumerate(reqs)]
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([StepRow(slots[i], reqs[i][:cut[i]], [cut[i] - 1]) for i in range(3)])
    assert_close(got, torch.stack([want[i][cut[i] - 1] for i in range(3)]), dtype, "batch prompts, " + what)
    live = [i for i in range(3) if cut[i] < len(reqs[i])]
    for i in range(3):
        if i not in live:
            eng.release(slots[i])
    steps = 0
    while live and steps < 12:                           # a dozen steps are enough to cross pages and windows
        got = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
        assert_close(got, torch.stack([want[i][cut[i]] for i in live]), dtype, f"batch decode {steps}, " + what)
        for i in list(live):
            cut[i] += 1
            if cut[i] == len(reqs[i]):
                eng.release(slots[i])
                live.remove(i)
        steps += 1
    for i in live:
        eng.release(slots[i])
    eng.cache.book.check()
    assert eng.cache.free_slots == eng.cache.max_slots
