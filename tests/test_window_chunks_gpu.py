"""Layers with a sliding window whose size is a whole number of cache pages
(64, 128: what real configurations have) take a prompt in portions and take
a new prompt beside decoding rows: the ring keeps `window_chunk - 1` keys
more than the window, so that a portion's keys do not overwrite keys its
first query still needs (GPU)."""
import os

import pytest
import torch

from helpers import TINY_B, assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("windows")


def _folder(tmp_root, window, dtype):
    from tq_kv_b200.weights import write_model_folder
    cfg = {**TINY_B, "sliding_window": window, "torch_dtype": dtype}
    path = os.path.join(str(tmp_root), f"w{window}_{dtype}")
    if not os.path.isdir(path):
        write_model_folder(cfg, path, seed=31 + window)
    return path


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [64, 128])
def test_a_prompt_in_portions_with_a_window_of_whole_pages(tmp_root, window, dtype):
    from tq_kv_b200.cache import ring_pages_for
    from tq_kv_b200.engine import Engine, StepRow
    folder = _folder(tmp_root, window, dtype)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2)
    ring = ring_pages_for(window, 63)
    assert [g.ring_pages for g in eng.cache.groups] == [0, ring] and ring == window // 64 + 1
    toks = random_tokens(420, TINY_B["vocab_size"], 12)
    want = plain_logits(folder, toks)
    # portions of up to 64 tokens; some end exactly where the ring wraps (positions 64 * ring, 2 * 64 * ring)
    edge = 64 * ring
    cuts, at, sizes = [], 0, [40, 64, 64, 1, 63, 17, 64]
    while at < len(toks):
        n = min(sizes[len(cuts) % len(sizes)], len(toks) - at)
        for target in (edge, 2 * edge):
            if at < target:
                n = min(n, target - at)
                break
        cuts.append(n)
        at += n
    ends = [sum(cuts[:i + 1]) for i in range(len(cuts))]
    assert all(0 < c <= 64 for c in cuts) and edge in ends and 2 * edge in ends and 64 in cuts
    s = eng.new_sequence()
    outs, at = [], 0
    for n in cuts:
        outs.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
        at += n
    eng.release(s)
    assert_close(torch.cat(outs), want, dtype, f"window {window}: portions {cuts}")
    # one token more than the ring allows is refused before anything runs
    from tq_kv_b200.kernels import KernelError
    s = eng.new_sequence()
    eng.step([StepRow(s, toks[:10], [])])
    limit = 64 * ring - window + 1
    with pytest.raises(KernelError, match="window_chunk"):
        eng.step([StepRow(s, toks[10:10 + limit + 1], [])])
    got = eng.step([StepRow(s, toks[10:10 + limit], [limit - 1])])        # the limit itself runs
    assert_close(got, want[10 + limit - 1:10 + limit], dtype, "longest portion")
    eng.release(s)
    eng.cache.book.check()


def test_a_larger_window_chunk_takes_longer_portions(tmp_root):
    from tq_kv_b200.engine import Engine, StepRow
    folder = _folder(tmp_root, 64, "float32")
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_slots=2, window_chunk=200)
    assert eng.cache.groups[1].ring_pages == 5                  # 64 + 199 keys in pages of 64
    toks = random_tokens(420, TINY_B["vocab_size"], 13)
    want = plain_logits(folder, toks)
    s = eng.new_sequence()
    outs = [eng.step([StepRow(s, toks[a:b], list(range(b - a)))]) for a, b in ((0, 20), (20, 220), (220, 420))]
    eng.release(s)
    assert_close(torch.cat(outs), want, "float32", "portions of 200")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_new_prompt_beside_decoding_rows(tmp_root, dtype):
    """One step holds a 60-token prompt that starts at position 0 and three
    rows that decode one token each (every row then reads the paged cache,
    windowed layers included); then all four decode together."""
    from tq_kv_b200.engine import Engine, StepRow
    folder = _folder(tmp_root, 64, dtype)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=4)
    V = TINY_B["vocab_size"]
    reqs = [random_tokens(n, V, 50 + n) for n in (150, 90, 30, 75)]
    wants = [plain_logits(folder, r) for r in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    pos = [140, 80, 20, 0]
    eng.step([StepRow(slots[i], reqs[i][:pos[i]], []) for i in range(3)])
    got = eng.step([StepRow(slots[i], [reqs[i][pos[i]]], [0]) for i in range(3)] +
                   [StepRow(slots[3], reqs[3][:60], [0, 59])])
    want = torch.stack([wants[0][140], wants[1][80], wants[2][20], wants[3][0], wants[3][59]])
    assert_close(got, want, dtype, "prompt beside decoding rows")
    pos = [141, 81, 21, 60]
    for _ in range(8):
        got = eng.step([StepRow(slots[i], [reqs[i][pos[i]]], [0]) for i in range(4)])
        assert_close(got, torch.stack([wants[i][pos[i]] for i in range(4)]), dtype, f"decode at {pos}")
        pos = [p + 1 for p in pos]
    for s in slots:
        eng.release(s)
