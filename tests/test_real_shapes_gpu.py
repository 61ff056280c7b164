"""Layers of the sizes of Qwen2.5-0.5B, 7B and 32B (a few layers, a small
vocabulary, random weights) against the plain implementation: the kernels'
fast paths are picked by head size, group size and widths, and these are the
sizes they will meet (GPU)."""
import os

import pytest
import torch

from helpers import assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

# name of the shape, layers kept, tokens fed
SHAPES = [("qwen2.5-0.5b", 2, 150), ("qwen2.5-7b", 2, 150), ("qwen2.5-32b", 1, 90)]
VOCAB = 3000        # the vocabulary is cut down: the embedding and head matrices of 152k rows only cost time here


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("real")


@pytest.mark.parametrize("shape,layers,n_tokens", SHAPES)
def test_real_layer_sizes_whole_then_decoded_and_batched(tmp_root, shape, layers, n_tokens):
    import tq_kv_b200 as tq
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.weights import write_model_folder
    cfg = dict(tq.named_shape(shape))
    cfg.update(num_hidden_layers=layers, max_window_layers=layers, vocab_size=VOCAB, torch_dtype="bfloat16",
               max_position_embeddings=1024)
    folder = write_model_folder(cfg, os.path.join(str(tmp_root), shape), seed=8, device="cuda")
    reqs = [random_tokens(n_tokens, VOCAB, 300 + i) for i in range(2)]
    reqs[1] = reqs[1][:n_tokens // 2 + 3]
    wants = [plain_logits(folder, r) for r in reqs]
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512)
        # whole
        s = eng.new_sequence()
        got = eng.step([StepRow(s, reqs[0], list(range(n_tokens)))])
        eng.release(s)
        assert_close(got, wants[0], dtype, f"{shape} whole")
        # an unequal batch: prompts, then one token each until the shorter one ends, then the longer one alone
        slots = [eng.new_sequence(), eng.new_sequence()]
        cut = [len(reqs[0]) - 20, len(reqs[1]) - 12]
        got = eng.step([StepRow(slots[i], reqs[i][:cut[i]], [cut[i] - 1]) for i in range(2)])
        assert_close(got, torch.stack([wants[i][cut[i] - 1] for i in range(2)]), dtype, f"{shape} prompts")
        live = [0, 1]
        while live:
            got = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
            assert_close(got, torch.stack([wants[i][cut[i]] for i in live]), dtype, f"{shape} decode")
            for i in list(live):
                cut[i] += 1
                if cut[i] == len(reqs[i]):
                    eng.release(slots[i])
                    live.remove(i)
        del eng
        torch.cuda.empty_cache()


def test_eight_long_prompts_at_the_32b_shape_under_both_prompt_attention_kernels(monkeypatch):
    """Eight prompts of 2,048 tokens through two layers of the 32B shape (40 q heads: 5,120 attention blocks, the
    longest with 32 key tiles; scores with the spread that real projections give them), several times: the
    logits at the prompts' ends must be finite and agree between the tcgen05 attention and the mma.sync
    attention.  A mistake in the tcgen05 kernel's reuse of tensor memory showed only here, and not every time."""
    import importlib
    import tq_kv_b200 as tq
    from tq_kv_b200.engine import Engine, StepRow
    att = importlib.import_module("tq_kv_b200.kernels.attention")
    cfg = dict(tq.named_shape("qwen2.5-32b"))
    cfg.update(num_hidden_layers=2, max_window_layers=2, vocab_size=VOCAB)
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_slots=8, max_context=2048)
    prompts = [random_tokens(2048, VOCAB, 500 + i) for i in range(8)]

    def run(tc):
        monkeypatch.setattr(att, "USE_TC_ATTENTION", tc)
        slots = [eng.new_sequence() for _ in prompts]
        out = eng.step([StepRow(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        for s in slots:
            eng.release(s)
        return out.float().cpu()

    want = run(False)
    assert torch.isfinite(want).all()
    for rep in range(4):
        got = run(True)
        assert torch.isfinite(got).all(), f"run {rep}: non-finite logits in rows {(~torch.isfinite(got)).any(1).nonzero().flatten().tolist()}"
        assert float((got - want).abs().max()) <= 0.03 * max(1.0, float(want.abs().max())), f"run {rep}"


@pytest.mark.parametrize("shape,batch", [("qwen2.5-7b", 8), ("qwen2.5-7b", 40), ("qwen2.5-0.5b", 8)])
def test_many_decode_steps_replayed_and_launched_one_by_one_agree(shape, batch):
    """Sixty decode steps of a batch at real layer sizes, once as replayed graphs (kernels launched as dependents
    of one another, starting before their predecessors end) and once kernel by kernel without graphs: the
    logits must agree step for step.  A kernel that touched its inputs before its predecessor was done, or a
    split whose partial sums met in the wrong place, would show as a drift between the two."""
    import tq_kv_b200 as tq
    from tq_kv_b200.engine import Engine, StepRow
    cfg = dict(tq.named_shape(shape))
    cfg.update(num_hidden_layers=2, max_window_layers=2, vocab_size=VOCAB)
    eng = Engine.from_random(cfg, seed=1, dtype="bfloat16", max_slots=batch, max_context=1024)
    prompts = [random_tokens(200 + 13 * (i % 7), VOCAB, 700 + i) for i in range(batch)]
    forced = [random_tokens(60, VOCAB, 900 + i) for i in range(batch)]
    runs = []
    for graphs in (True, False):
        eng.use_graphs = graphs
        slots = [eng.new_sequence() for _ in prompts]
        eng.step([StepRow(s, p, []) for s, p in zip(slots, prompts)])
        outs = [eng.step([StepRow(s, [f[t]], [0]) for s, f in zip(slots, forced)]).float().cpu() for t in range(60)]
        for s in slots:
            eng.release(s)
        runs.append(torch.stack(outs))
    eng.use_graphs = True
    assert torch.isfinite(runs[0]).all() and torch.isfinite(runs[1]).all()
    scale = max(1.0, float(runs[1].abs().max()))
    err = float((runs[0] - runs[1]).abs().max())
    assert err <= 0.02 * scale, f"{shape}, batch {batch}: replayed and plain launches differ by {err:.3e}"


def test_deterministic_switch_gives_the_same_bits_twice(tmp_path):
    """With TQ_DETERMINISTIC=1 no product's shares of K meet in memory in arrival order: two runs of the same
    prompt and decode steps at the 7B layer shape give identical logits (a child process each, since the switch is
    read once)."""
    import subprocess
    import sys
    script = tmp_path / "run.py"
    script.write_text(
        "import sys, torch\n"
        "sys.path.insert(0, REPO); sys.path.insert(0, TESTS)\n"
        "import tq_kv_b200 as tq\n"
        "from tq_kv_b200.engine import Engine, StepRow\n"
        "from helpers import random_tokens\n"
        "cfg = dict(tq.named_shape('qwen2.5-7b')); cfg.update(num_hidden_layers=2, max_window_layers=2, vocab_size=3000)\n"
        "eng = Engine.from_random(cfg, seed=1, dtype='bfloat16', max_slots=8, max_context=1024)\n"
        "slots = [eng.new_sequence() for _ in range(8)]\n"
        "outs = [eng.step([StepRow(s, random_tokens(300 + 7 * i, 3000, i), [299 + 7 * i]) for i, s in enumerate(slots)])]\n"
        "for t in range(20):\n"
        "    outs.append(eng.step([StepRow(s, [(5 * t + i) % 3000], [0]) for i, s in enumerate(slots)]))\n"
        "torch.save(torch.cat(outs).cpu(), sys.argv[1])\n"
        .replace("REPO", repr(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        .replace("TESTS", repr(os.path.dirname(os.path.abspath(__file__)))))
    results = []
    for i in range(2):
        out = tmp_path / f"out{i}.pt"
        env = dict(os.environ, TQ_DETERMINISTIC="1")
        subprocess.run([sys.executable, str(script), str(out)], check=True, env=env, timeout=300)
        results.append(torch.load(out))
    assert torch.isfinite(results[0]).all()
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("shape", ["qwen2.5-7b", "qwen2.5-0.5b"])
def test_a_long_prompt_whole_and_in_chunks_agree(shape):
    """1,500 tokens in one step (attention over the step's packed keys) and as 700 + 800 (the second chunk reads
    the first from the paged cache through TMA): the logits at the chunk's positions must agree."""
    import tq_kv_b200 as tq
    from tq_kv_b200.engine import Engine, StepRow
    cfg = dict(tq.named_shape(shape))
    cfg.update(num_hidden_layers=2, max_window_layers=2, vocab_size=VOCAB)
    eng = Engine.from_random(cfg, seed=2, dtype="bfloat16", max_slots=2, max_context=2048)
    toks = random_tokens(1500, VOCAB, 41)
    want_rows = [700, 701, 1023, 1024, 1499]
    s = eng.new_sequence()
    whole = eng.step([StepRow(s, toks, want_rows)]).float().cpu()
    eng.release(s)
    s = eng.new_sequence()
    eng.step([StepRow(s, toks[:700], [])])
    chunked = eng.step([StepRow(s, toks[700:], [r - 700 for r in want_rows])]).float().cpu()
    eng.release(s)
    assert torch.isfinite(whole).all() and torch.isfinite(chunked).all()
    assert float((whole - chunked).abs().max()) <= 0.03 * max(1.0, float(whole.abs().max()))
