"""What tiny random models hide: attention that rests on a few keys (so that
a dropped or extra key shows at model level, in bfloat16 too), the full depth
of a real shape, the real vocabulary in the head product, the embedding and
the samplers, and decode batches beyond the skinny products' 64 rows (GPU)."""
import pytest
import torch

import plain_model as pm
from helpers import (TINY_C, assert_close, plain_logits, plain_logits_on, planted_model, planted_tokens,
                     random_tokens, random_weights)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("depth")


# ---- a planted key: the three cuts on models in which one key at a telling place decides the logits ------------
def _three_cuts(eng, reqs, wants, dtype, what):
    from tq_kv_b200.engine import StepRow
    for toks, want in zip(reqs, wants):                       # whole
        s = eng.new_sequence()
        assert_close(eng.step([StepRow(s, toks, list(range(len(toks))))]), want, dtype, f"{what}: whole")
        eng.release(s)
    for toks, want in zip(reqs, wants):                       # the last 32 one by one
        n = len(toks) - 32
        s = eng.new_sequence()
        outs = [eng.step([StepRow(s, toks[:n], [n - 1])])] + [eng.step([StepRow(s, [t], [0])]) for t in toks[n:]]
        eng.release(s)
        assert_close(torch.cat(outs), want[n - 1:], dtype, f"{what}: last 32 one by one")
    for order in (range(len(reqs)), reversed(range(len(reqs)))):     # unequal batches; slots change hands
        order = list(order)
        slots = {i: eng.new_sequence() for i in order}
        cut = {i: len(reqs[i]) - 5 - 9 * k for k, i in enumerate(order)}
        got = eng.step([StepRow(slots[i], reqs[i][:cut[i]], [cut[i] - 1]) for i in order])
        assert_close(got, torch.stack([wants[i][cut[i] - 1] for i in order]), dtype, f"{what}: prompts")
        live = list(order)
        while live:
            got = eng.step([StepRow(slots[i], [reqs[i][cut[i]]], [0]) for i in live])
            assert_close(got, torch.stack([wants[i][cut[i]] for i in live]), dtype, f"{what}: batched decode")
            for i in list(live):
                cut[i] += 1
                if cut[i] == len(reqs[i]):
                    eng.release(slots.pop(i))
                    live.remove(i)
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decisive_key_at_the_windows_edge(tmp_root, dtype):
    """The query token stands at T-1, where the planted key is the oldest key
    its window still holds, and again at T, where the key has just left: a
    window off by one key in either direction moves one of the two rows by
    the size of the logits (test_plain_model.py checks that of the plain
    implementation)."""
    from tq_kv_b200.engine import Engine
    folder = planted_model(tmp_root, dtype, windowed=True)
    W = TINY_C["sliding_window"]
    reqs = [planted_tokens(T + 1, T - W, [T - 1, T], 40 + T) for T in (200, 75, 141, 70)]
    wants = [plain_logits(folder, r) for r in reqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=4)
    _three_cuts(eng, reqs, wants, dtype, "key at the window's edge")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decisive_key_far_back_among_hundreds(tmp_root, dtype):
    """No window: the planted key is the third token, the query comes after
    700 or 330 others (many pages back, in another split of the decode
    attention) and the logits there rest on it."""
    from tq_kv_b200.engine import Engine
    folder = planted_model(tmp_root, dtype, windowed=False)
    reqs = [planted_tokens(n, 2, [n - 1, n - 20], 60 + n) for n in (700, 330, 64)]
    wants = [plain_logits(folder, r) for r in reqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1280, max_slots=3)
    _three_cuts(eng, reqs, wants, dtype, "far key")


# ---- full depth and the real vocabulary -----------------------------------------------------------------------------
def _free():
    import gc
    gc.collect()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_half_billion_shape_at_full_depth_with_its_real_vocabulary(dtype):
    """All 24 layers and the tied 151,936-row head of the Qwen2.5-0.5B shape:
    a 300-token prompt whole, then 16 tokens decoded one by one, against the
    plain implementation run on the GPU in float32 on the same weights (made
    from the same seed, without a file)."""
    import tq_kv_b200 as tq
    from tq_kv_b200.engine import Engine, StepRow
    cfg = dict(tq.named_shape("qwen2.5-0.5b"))
    V = cfg["vocab_size"]
    toks = random_tokens(316, V, 77)
    want = plain_logits_on("cuda", cfg, random_weights(cfg, 9, "cuda"), toks)
    _free()
    eng = Engine.from_random(cfg, seed=9, dtype=dtype, max_slots=1, max_context=512)
    s = eng.new_sequence()
    rows = [0, 1, 63, 64, 150, 298, 299]
    got = eng.step([StepRow(s, toks[:300], rows)])
    assert_close(got, want[rows], dtype, "0.5B shape, 24 layers: prompt")
    outs = [eng.step([StepRow(s, [t], [0])]) for t in toks[300:]]
    assert_close(torch.cat(outs), want[300:], dtype, "0.5B shape, 24 layers: 16 decoded tokens")
    agree = int((torch.cat(outs).argmax(-1).cpu() == want[300:].argmax(-1)).sum())
    assert agree >= (16 if dtype == "float32" else 13), f"arg-max agrees at {agree} of 16 places"
    eng.release(s)
    del eng
    _free()


def test_the_real_head_for_1_8_64_and_65_rows_and_the_sampler_at_that_vocabulary():
    """One layer of the 7B shape with the real untied head of 152,064 rows:
    logits for 1, 8, 64 and 65 wanted rows (the last leaves the decode
    products for the many-row kernel) against the plain implementation, in
    both precisions; then the samplers on those logits against the plain
    sampler, arg-max and with temperature, top-k, top-p and the penalty."""
    import tq_kv_b200 as tq
    from tq_kv_b200 import kernels
    from tq_kv_b200.engine import Engine, StepRow
    cfg = dict(tq.named_shape("qwen2.5-7b"))
    cfg.update(num_hidden_layers=1, max_window_layers=1)
    V = cfg["vocab_size"]
    toks = random_tokens(70, V, 78)
    want = plain_logits_on("cuda", cfg, random_weights(cfg, 10, "cuda"), toks)
    _free()
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(cfg, seed=10, dtype=dtype, max_slots=1, max_context=128)
        for n_rows in (1, 8, 64, 65):
            rows = list(range(70 - n_rows, 70))
            s = eng.new_sequence()
            got = eng.step([StepRow(s, toks, rows)])
            eng.release(s)
            assert_close(got, want[rows], dtype, f"7B head, {n_rows} wanted rows")
        if dtype == "float32":
            logits = got[:8].contiguous()                       # float32 engine: the plain sampler sees the same numbers
            out = torch.zeros(8, dtype=torch.int32, device="cuda")
            kernels.sample(logits, out)
            assert out.tolist() == [pm.greedy(r) for r in logits.cpu()]
            us = [0.03, 0.25, 0.5, 0.61, 0.77, 0.9, 0.999, 0.0]
            u = torch.tensor(us, dtype=torch.float32, device="cuda")
            f32 = lambda x: float(torch.tensor(x, dtype=torch.float32))
            for t, k, p in ((0.8, 0, 1.0), (0.7, 40, 0.9), (1.3, 500, 0.5), (1.0, 0, 0.3)):
                kernels.sample(logits, out, temperature=t, top_k=k, top_p=p, uniforms=u)
                want_ids = [pm.sample(r, f32(t), k, f32(p), f32(x)) for r, x in zip(logits.cpu(), us)]
                assert out.tolist() == want_ids, (t, k, p)
        del eng
        _free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_batch_of_96_rows(tmp_root, dtype):
    """More rows than the decode products take (64): the step runs on the
    many-row kernels; with and without replayed graphs."""
    from helpers import TINY, model_folder
    from tq_kv_b200.engine import Engine, StepRow
    folder = model_folder(tmp_root, "b", dtype)
    V = TINY["b"]["vocab_size"]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=96 * 128, max_slots=96)
    reqs = [random_tokens(8 + (5 * i) % 60 + 4, V, 2000 + i) for i in range(96)]
    wants = [plain_logits(folder, r) for r in reqs]
    for graphs in (True, False):
        eng.use_graphs = graphs
        slots = [eng.new_sequence() for _ in reqs]
        cut = [len(r) - 4 for r in reqs]
        eng.step([StepRow(s, r[:c], []) for s, r, c in zip(slots, reqs, cut)])
        for k in range(4):
            got = eng.step([StepRow(s, [r[c + k]], [0]) for s, r, c in zip(slots, reqs, cut)])
            assert_close(got, torch.stack([w[c + k] for w, c in zip(wants, cut)]), dtype,
                         f"96 rows, decode step {k}, graphs={graphs}")
        for s in slots:
            eng.release(s)
    eng.use_graphs = True
