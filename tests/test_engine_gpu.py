"""The engine against the plain implementation, in float32 and bfloat16, for
both tiny configurations and every way of cutting the work (GPU)."""
import pytest
import torch

from helpers import TINY, assert_close, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = [40, 77, 33, 130, 65]          # 130 crosses pages and laps the 64-token ring of the windowed layers
CASES = [(n, d) for n in "ab" for d in ("float32", "bfloat16")]
_engines = {}


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


def engine_for(tmp_root, name, dtype, max_tokens=1024):
    from tq_kv_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _engines:
        folder = model_folder(tmp_root, name, dtype)
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens), folder)
    return _engines[key]


def requests_for(name):
    return [random_tokens(n, TINY[name]["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS)]


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    for toks in requests_for(name):
        s = eng.new_sequence()
        got = eng.step([StepRow(s, toks, list(range(len(toks))))])
        eng.release(s)
        assert_close(got, plain_logits(folder, toks), dtype, f"whole, {len(toks)} tokens")
    eng.cache.book.check()


def test_library_products_give_the_same_as_the_tcgen05_kernel(tmp_root, monkeypatch):
    """Many-row bfloat16 products run on this package's tcgen05 kernel; the
    library product stays selectable and must agree."""
    from tq_kv_b200 import kernels
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, "b", "bfloat16")
    toks = requests_for("b")[3]
    outs = []
    for own in (True, False):
        monkeypatch.setattr(kernels.gemm, "USE_TCGEN05", own)
        s = eng.new_sequence()
        outs.append(eng.step([StepRow(s, toks, list(range(len(toks))))]))
        eng.release(s)
    assert_close(outs[0], plain_logits(folder, toks), "bfloat16", "tcgen05")
    assert_close(outs[1], plain_logits(folder, toks), "bfloat16", "library")


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    for toks in requests_for(name):
        want = plain_logits(folder, toks)
        n = len(toks) - 32
        s = eng.new_sequence()
        first = eng.step([StepRow(s, toks[:n], [n - 1])])
        assert_close(first, want[n - 1:n], dtype, "end of the prefix")
        outs = [eng.step([StepRow(s, [t], [0])]) for t in toks[n:]]
        eng.release(s)
        assert_close(torch.cat(outs), want[n:], dtype, f"last 32 of {len(toks)}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another_reuse_slots(tmp_root, name, dtype):
    """Batches of unequal prompts; then one token each, teacher-forced; the
    shorter requests end earlier; the cache is so small that the second batch
    gets the slots and pages the first one gave back."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype, max_tokens=384)      # 6 pages: 40+77+130 needs 6
    reqs = requests_for(name)
    used_slots = []
    for batch, cut in (([0, 1, 3], [8, 50, 101]), ([4, 2], [33, 1]), ([1, 2, 0], [77, 2, 17])):
        slots = {i: eng.new_sequence() for i in batch}
        used_slots.append(sorted(slots.values()))
        pos = dict(zip(batch, cut))
        rows = [StepRow(slots[i], reqs[i][:pos[i]], list(range(pos[i]))) for i in batch]
        got = eng.step(rows)
        want = torch.cat([plain_logits(folder, reqs[i])[:pos[i]] for i in batch])
        assert_close(got, want, dtype, f"prompts of batch {batch}")
        live = [i for i in batch if pos[i] < len(reqs[i])]
        for i in batch:
            if i not in live:
                eng.release(slots.pop(i))
        while live:
            rows = [StepRow(slots[i], [reqs[i][pos[i]]], [0]) for i in live]
            got = eng.step(rows)
            want = torch.stack([plain_logits(folder, reqs[i])[pos[i]] for i in live])
            assert_close(got, want, dtype, f"decode at {[pos[i] for i in live]}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(reqs[i])]:
                eng.release(slots.pop(i))
                live.remove(i)
        eng.cache.book.check()
    assert used_slots[0] == used_slots[2] == [0, 1, 2] and used_slots[1] == [0, 1]
    assert eng.cache.free_pages() == 6 and eng.cache.free_slots == eng.cache.max_slots


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    toks = random_tokens(300, TINY[name]["vocab_size"], 55)
    want = plain_logits(folder, toks)
    s = eng.new_sequence()
    eng.step([StepRow(s, toks[:5], [])])
    outs = [eng.step([StepRow(s, [t], [0])]) for t in toks[5:]]
    eng.release(s)
    assert_close(torch.cat(outs), want[5:], dtype, "295 decoded tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_decoding_without_replayed_graphs_gives_the_same(tmp_root, name, dtype):
    """Decode steps normally replay a captured graph; the plain launch path
    must agree with it and with the plain implementation."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    toks = random_tokens(90, TINY[name]["vocab_size"], 56)
    want = plain_logits(folder, toks)
    runs = []
    for graphs in (True, False):
        eng.use_graphs = graphs
        try:
            s = eng.new_sequence()
            eng.step([StepRow(s, toks[:50], [])])
            runs.append(torch.cat([eng.step([StepRow(s, [t], [0])]) for t in toks[50:]]))
            eng.release(s)
        finally:
            eng.use_graphs = True
    assert_close(runs[0], want[50:], dtype, "graph")
    assert_close(runs[1], want[50:], dtype, "no graph")
    # the two differ by rounding only: the graph plans attention's splits for the context limit
    assert_close(runs[0], runs[1].cpu(), dtype, "graph vs no graph")


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    toks = random_tokens(6, TINY[name]["vocab_size"], 77)
    want = plain_logits(folder, toks)
    for first in (1, 2):
        s = eng.new_sequence()
        outs = [eng.step([StepRow(s, toks[:first], list(range(first)))])]
        outs += [eng.step([StepRow(s, [t], [0])]) for t in toks[first:]]
        eng.release(s)
        assert_close(torch.cat(outs), want, dtype, f"prompt of {first}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_in_chunks_reads_the_cache(tmp_root, name, dtype):
    """A sequence continued by several tokens at once attends over the cache."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    toks = requests_for(name)[3]
    want = plain_logits(folder, toks)
    s = eng.new_sequence()
    outs, at = [], 0
    for n in (10, 7, 40, 1, 49, 23):
        outs.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
        at += n
    eng.release(s)
    assert at == len(toks)
    assert_close(torch.cat(outs), want, dtype, "chunks")


def test_refused_steps_change_nothing(tmp_root):
    from tq_kv_b200.engine import StepError, StepRow
    from tq_kv_b200.kernels import KernelError
    eng, folder = engine_for(tmp_root, "b", "float32", max_tokens=384)
    s = eng.new_sequence()
    with pytest.raises(StepError, match="Empty prompt"):
        eng.step([StepRow(s, [], [])])
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([StepRow(s, [1, 1000], [0])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([StepRow(s, [1, 2], [2])])
    with pytest.raises(StepError, match="context limit"):
        eng.step([StepRow(s, [1] * 385, [])])
    other = eng.new_sequence()
    eng.step([StepRow(other, [1] * 200, [])])                        # 4 of the 6 pages
    with pytest.raises(StepError, match="is full"):
        eng.step([StepRow(s, [1] * 150, [])])
    eng.release(other)
    eng.step([StepRow(s, [1, 2, 3], [])])
    with pytest.raises(KernelError, match="window"):                    # 120 tokens onto a 128-key ring, window 16
        eng.step([StepRow(s, [1] * 120, [])])
    assert eng.length(s) == 3
    with pytest.raises(StepError, match="not held"):
        eng.step([StepRow(5, [1], [])])
    eng.release(s)
    eng.cache.book.check()
    assert eng.cache.free_pages() == 6


def test_context_limit_is_enforced(tmp_root):
    from tq_kv_b200.engine import Engine, StepError, StepRow
    folder = model_folder(tmp_root, "a", "float32")
    eng = Engine.from_folder(folder, dtype="float32", max_slots=2, max_context=100)
    s = eng.new_sequence()
    eng.step([StepRow(s, [1] * 100, [])])
    with pytest.raises(StepError, match="context limit"):
        eng.step([StepRow(s, [1], [0])])
    with pytest.raises(ValueError, match="max positions"):
        Engine.from_folder(folder, dtype="float32", max_slots=1, max_context=4096)


def _folder_as(tmp_root, arch_name):
    """Tiny A's folder under another architecture name (same tensors)."""
    import json
    import os
    import shutil
    src = model_folder(tmp_root, "a", "float32")
    dst = os.path.join(str(tmp_root), f"tiny_a_as_{arch_name}")
    if not os.path.isdir(dst):
        os.makedirs(dst)
        shutil.copy(os.path.join(src, "model.safetensors"), dst)
        cfg = json.load(open(os.path.join(src, "config.json")))
        cfg["architectures"] = [arch_name]
        json.dump(cfg, open(os.path.join(dst, "config.json"), "w"))
    return src, dst


def _with_schedule(arch_name, schedule):
    from dataclasses import replace

    from tq_kv_b200.config import Architecture, Qwen2Config, build_qwen2_spec

    def build(cfg):
        return replace(build_qwen2_spec(cfg), architecture=arch_name, schedule=schedule)

    return Architecture(arch_name, arch_name.lower(), Qwen2Config, build)


def test_a_block_named_twice_runs_twice_with_a_cache_each(tmp_root):
    """The order of layers is data: the schedule may name a block twice."""
    import plain_model as pm
    from tq_kv_b200.config import ScheduleEntry, register_architecture, unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    register_architecture(_with_schedule("TwiceForCausalLM", (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1))))
    try:
        src, dst = _folder_as(tmp_root, "TwiceForCausalLM")
        eng = Engine.from_folder(dst, dtype="float32", max_tokens=256)
        assert len(eng.cache.groups[0].entries) == 3            # the repeated block has a cache of its own
        cfg, w = pm.read_model_folder(src)
        w3 = dict(w)
        for k in w:
            if k.startswith("model.layers.1."):
                w3[k.replace("layers.1.", "layers.2.")] = w[k]
        toks = random_tokens(30, 256, 9)
        want = pm.decoder_logits({**cfg, "num_hidden_layers": 3}, w3, toks)
        s = eng.new_sequence()
        got = [eng.step([StepRow(s, toks[:20], list(range(20)))])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in toks[20:]]
        assert_close(torch.cat(got), want, "float32", "block run twice")
    finally:
        unregister_architecture("TwiceForCausalLM")


def test_an_entry_can_read_another_entrys_cache(tmp_root):
    """Third entry: block 1 again, but attending over the keys and values that
    the second entry cached (it writes none of its own)."""
    import math

    import plain_model as pm
    from tq_kv_b200.config import ScheduleEntry, register_architecture, unregister_architecture
    from tq_kv_b200.engine import Engine, StepRow
    register_architecture(_with_schedule("SharedForCausalLM",
                                         (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_of=1))))
    try:
        src, dst = _folder_as(tmp_root, "SharedForCausalLM")
        eng = Engine.from_folder(dst, dtype="float32", max_tokens=256)
        assert len(eng.cache.groups[0].entries) == 2
        cfg, w = pm.read_model_folder(src)
        toks = random_tokens(30, 256, 10)
        T, nh, nkv, hd, eps = len(toks), 4, 2, 16, cfg["rms_norm_eps"]
        cos, sin = pm.rope_tables(hd, cfg["rope_theta"], T)

        def layer(h, i, kv_from=None):
            p = f"model.layers.{i}."
            a = pm.rms_norm(h, w[p + "input_layernorm.weight"], eps)
            src_a = a if kv_from is None else kv_from
            q = (a @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]).reshape(T, nh, hd)
            k = (src_a @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]).reshape(T, nkv, hd)
            v = (src_a @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]).reshape(T, nkv, hd)
            q = pm.rope_halved(q.transpose(0, 1), cos, sin)
            k = pm.repeat_kv(pm.rope_halved(k.transpose(0, 1), cos, sin), nh // nkv)
            v = pm.repeat_kv(v.transpose(0, 1), nh // nkv)
            att = q @ k.transpose(1, 2) / math.sqrt(hd)
            att = torch.where(pm.attention_mask(T, None), torch.full_like(att, float("-inf")), att)
            y = (pm.softmax_last_dim(att) @ v).transpose(0, 1).reshape(T, nh * hd)
            h = h + y @ w[p + "self_attn.o_proj.weight"].T
            m = pm.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
            return h + pm.swiglu_mlp(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                     w[p + "mlp.down_proj.weight"]), a

        h = w["model.embed_tokens.weight"][torch.tensor(toks)]
        h, _ = layer(h, 0)
        h, a1 = layer(h, 1)
        h, _ = layer(h, 1, kv_from=a1)
        want = pm.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T
        s = eng.new_sequence()
        got = [eng.step([StepRow(s, toks[:20], list(range(20)))])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in toks[20:]]
        assert_close(torch.cat(got), want, "float32", "shared cache")
    finally:
        unregister_architecture("SharedForCausalLM")


def test_a_wait_that_ran_out_in_a_replayed_step_surfaces_in_short_runs(tmp_root):
    """Replayed decode steps do not wait for the device.  A bit raised in the status word of the tcgen05
    kernels (here by hand) must still stop a short generation, and `check_status()` must report it to
    whoever replays steps himself; afterwards the word is clear again."""
    import tq_kv_b200 as tq
    from tq_kv_b200 import kernels
    from tq_kv_b200.engine import StepRow
    eng, _ = engine_for(tmp_root, "b", "bfloat16")
    word = kernels._lib.report_buffer(torch.device("cuda:0"))[:1]
    s = eng.new_sequence()
    try:
        eng.step([StepRow(s, [1, 2, 3], [])])
        eng.step([StepRow(s, [4], [0])])                       # a replayed step
        word.fill_(2)
        eng.step([StepRow(s, [5], [0])])                       # replays do not look
        with pytest.raises(kernels.KernelError, match="wait ran out"):
            eng.check_status()
        eng.check_status()                                     # cleared
        eng.release(s)
        s = None
        # a generation of four tokens: the loop reads the word with every step's ids
        real_step, calls = eng.step, []

        def step_then_raise_the_bit(rows, **kw):
            out = real_step(rows, **kw)
            calls.append(1)
            if len(calls) == 2:
                word.fill_(2)
            return out

        eng.step = step_then_raise_the_bit
        with pytest.raises(kernels.KernelError, match="wait ran out"):
            eng.generate([[1, 2, 3]], tq.GenerationParams.greedy(4, stop_token_ids=()))
        assert eng.cache.free_slots == eng.cache.max_slots     # the failed batch gave its slot back
    finally:
        eng.__dict__.pop("step", None)
        word.zero_()
        kernels.check_tc_status()
        if s is not None:
            eng.release(s)


def test_a_step_that_fails_after_reserving_gives_its_pages_back(tmp_root, monkeypatch):
    """An error inside the step (here: the model's forward raises) leaves lengths as they were and returns the
    pages that the step had reserved; the next step runs as if nothing had happened."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, "a", "float32", max_tokens=384)
    toks = random_tokens(150, TINY["a"]["vocab_size"], 91)
    s = eng.new_sequence()
    eng.step([StepRow(s, toks[:10], [])])
    free = eng.cache.free_pages()

    def boom(*a, **k):
        raise RuntimeError("boom")

    monkeypatch.setattr(eng.model, "forward", boom)
    with pytest.raises(RuntimeError, match="boom"):
        eng.step([StepRow(s, toks[10:150], [])])             # would have taken two more pages
    monkeypatch.undo()
    assert eng.length(s) == 10 and eng.cache.free_pages() == free
    eng.cache.book.check()
    got = eng.step([StepRow(s, toks[10:150], [139])])
    assert_close(got, plain_logits(folder, toks)[149:150], "float32", "after a failed step")
    eng.release(s)


@pytest.mark.parametrize("name,dtype", CASES)
def test_single_prompts_replayed_as_padded_graphs(tmp_root, name, dtype):
    """A single prompt from position 0 with one wanted row is padded with rows of token 0 to a multiple of 64
    and replayed as a captured graph (the second prompt of a padded size is a replay).  The padding changes no
    result: the logits equal the plain implementation's, the cache holds the real tokens only (pages, length),
    and tokens decoded afterwards read the right keys."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    assert eng.pad_prompts and eng.use_graphs
    V = TINY[name]["vocab_size"]
    pages0 = eng.cache.free_pages()
    for rnd_seed, n in enumerate([2, 63, 64, 65, 100, 7, 128, 70, 129]):      # 64: 2, 63, 64, 7; 128: 65, 100, 128, 70
        toks = random_tokens(n + 3, V, 500 + rnd_seed)
        want = plain_logits(folder, toks)
        s = eng.new_sequence()
        got = eng.step([StepRow(s, toks[:n], [n - 1])])
        assert_close(got, want[n - 1:n], dtype, f"padded prompt of {n} tokens")
        assert eng.length(s) == n and eng.cache.free_pages() == pages0 - -(-n // 64)
        after = [eng.step([StepRow(s, [t], [0])]) for t in toks[n:]]
        assert_close(torch.cat(after), want[n:], dtype, f"decoding after a padded prompt of {n} tokens")
        eng.release(s)
    assert sorted(eng._prompt_graphs) == [(1, 64), (1, 128), (1, 192)]
    assert all(g.graph is not None for g in eng._prompt_graphs.values())
    eng.check_status()
    eng.cache.book.check()
    assert eng.cache.free_pages() == pages0


@pytest.mark.parametrize("name,dtype", CASES)
def test_several_prompts_replayed_as_one_padded_graph(tmp_root, name, dtype):
    """Prompts of several sequences in one step replay a graph captured per (number of sequences, padded number
    of tokens); how the tokens divide among the sequences is data.  Three steps of three prompts with the same
    padded size and different lengths (the second and third are replays), each against the plain implementation,
    then one decoded token per sequence from what the prompts cached."""
    from tq_kv_b200.engine import StepRow
    eng, folder = engine_for(tmp_root, name, dtype)
    V = TINY[name]["vocab_size"]
    pages0 = eng.cache.free_pages()
    for k, lens in enumerate([(40, 9, 70), (5, 100, 20), (63, 1, 64), (30, 31)]):       # 119, 125, 128 -> 128; 61 -> 64
        reqs = [random_tokens(n + 1, V, 900 + 10 * k + i) for i, n in enumerate(lens)]
        wants = [plain_logits(folder, t) for t in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = eng.step([StepRow(s, t[:-1], [len(t) - 2]) for s, t in zip(slots, reqs)])
        assert_close(got, torch.stack([w[-2] for w in wants]), dtype, f"prompts of {lens} tokens in one padded step")
        assert [eng.length(s) for s in slots] == list(lens)
        assert eng.cache.free_pages() == pages0 - sum(-(-n // 64) for n in lens)
        nxt = eng.step([StepRow(s, [t[-1]], [0]) for s, t in zip(slots, reqs)])
        assert_close(nxt, torch.stack([w[-1] for w in wants]), dtype, f"decoding after prompts of {lens} tokens")
        for s in slots:
            eng.release(s)
    assert (3, 128) in eng._prompt_graphs and (2, 64) in eng._prompt_graphs
    eng.check_status()
    eng.cache.book.check()
    assert eng.cache.free_pages() == pages0
