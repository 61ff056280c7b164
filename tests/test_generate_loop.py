"""Decisions of the generation loop, with a scripted engine and sampler (CPU)."""
import pytest
import torch

from tq_kv_b200.engine.generate import generate, plan_batches
from tq_kv_b200.sampling import GenerationParams, uniform


class FakeCache:
    def __init__(self, slots, pages):
        self.free_slots, self.pages = slots, pages

    def free_pages(self):
        return self.pages


class FakeEngine:
    """Logits are one-hot: the next token of a sequence is (last token + 1) % V."""

    class _Spec:
        stop_token_ids = (7,)

    class _Rt:
        device = "cpu"
        max_context = 64

    def __init__(self, slots=2, vocab=16, max_context=64):
        self.vocab_size, self.spec, self.runtime = vocab, self._Spec(), self._Rt()
        self.runtime.max_context = max_context
        self.cache = FakeCache(slots, 100)
        self.held, self.steps, self.alloc_log = {}, [], []

    def new_sequence(self):
        assert self.cache.free_slots > 0
        s = min(set(range(64)) - set(self.held))
        self.held[s] = 0
        self.cache.free_slots -= 1
        self.alloc_log.append(s)
        return s

    def release(self, slot):
        del self.held[slot]                   # KeyError = freed twice
        self.cache.free_slots += 1

    def step(self, rows):
        self.steps.append([(r.slot, list(r.tokens), list(r.want)) for r in rows])
        out = torch.zeros(sum(len(r.want) for r in rows), self.vocab_size)
        i = 0
        for r in rows:
            assert r.slot in self.held
            self.held[r.slot] += len(r.tokens)
            for w in r.want:
                out[i, (r.tokens[w] + 1) % self.vocab_size] = 1.0
                i += 1
        return out


class ArgmaxSampler:
    def __init__(self, params, n_rows, vocab, device):
        self.n_rows, self.kept = n_rows, []

    def keep(self, rows):
        self.kept.append(list(rows))
        self.n_rows = len(rows)

    def sample(self, logits, requests, index):
        assert logits.shape[0] == self.n_rows == len(requests)
        return logits.argmax(-1).tolist()


def _gen(engine, prompts, **kw):
    params = GenerationParams.greedy(kw.pop("max_tokens", 4))
    for k, v in kw.items():
        setattr(params, k, v)
    return generate(engine, prompts, params, sampler_factory=ArgmaxSampler)


def test_prompts_prefill_together_then_one_token_each():
    e = FakeEngine(slots=3)
    res = _gen(e, [[1], [10, 11], [3, 4, 5]], max_tokens=3, stop_token_ids=())
    assert [r.tokens for r in res] == [[2, 3, 4], [12, 13, 14], [6, 7, 8]]
    assert [r.finish_reason for r in res] == ["length"] * 3
    assert [len(s) for s in e.steps] == [3, 3, 3]                  # 1 prefill + 2 decode steps, no step after the last token
    assert e.steps[0][1] == (1, [10, 11], [1]) and e.steps[1][2][1:] == ([6], [0])
    assert not e.held


def test_stop_token_is_not_emitted_and_frees_the_slot_early():
    e = FakeEngine(slots=2)
    res = _gen(e, [[5], [1]], max_tokens=5)               # default stop id 7: request 0 yields 6 then stops
    assert res[0].tokens == [6] and res[0].finish_reason == "stop"
    assert res[1].tokens == [2, 3, 4, 5, 6] and res[1].finish_reason == "length"
    assert [len(s) for s in e.steps] == [2, 2, 1, 1, 1]
    assert not e.held


def test_first_sampled_token_can_stop():
    e = FakeEngine()
    res = _gen(e, [[6]], max_tokens=5)
    assert res[0].tokens == [] and res[0].finish_reason == "stop" and len(e.steps) == 1


def test_more_requests_than_slots_run_batch_after_batch_reusing_slots():
    e = FakeEngine(slots=2)
    res = _gen(e, [[1], [2], [3], [4], [8]], max_tokens=2, stop_token_ids=())
    assert [r.tokens for r in res] == [[2, 3], [3, 4], [4, 5], [5, 6], [9, 10]]
    assert e.alloc_log == [0, 1, 0, 1, 0] and not e.held
    assert [len(s) for s in e.steps] == [2, 2, 2, 2, 1, 1]


def test_context_limit_ends_a_request():
    e = FakeEngine(max_context=4)
    res = _gen(e, [[1, 2]], max_tokens=10, stop_token_ids=())
    assert res[0].tokens == [3, 4, 5] and res[0].finish_reason == "context"
    assert e.held == {} and sum(len(r[1]) for s in e.steps for r in s) == 4   # the cache is used to its last place


def test_empty_prompt_and_zero_tokens():
    e = FakeEngine()
    with pytest.raises(ValueError, match="Empty prompt"):
        _gen(e, [[1], []])
    res = _gen(e, [[1]], max_tokens=0)
    assert res[0].tokens == [] and e.steps == []


def test_sampler_rows_follow_the_live_rows():
    e = FakeEngine(slots=3)
    kept = []

    class S(ArgmaxSampler):
        def keep(self, rows):
            kept.append(list(rows))
            super().keep(rows)

    generate(e, [[5], [1], [6]], GenerationParams.greedy(3), sampler_factory=S)
    assert kept == [[0, 1], [1]]                       # request 2 stops at once, request 0 after one token


def test_error_in_a_step_gives_slots_back():
    e = FakeEngine(slots=2)
    calls = []
    orig = e.step

    def boom(rows):
        calls.append(1)
        if len(calls) == 2:
            raise RuntimeError("boom")
        return orig(rows)

    e.step = boom
    with pytest.raises(RuntimeError):
        _gen(e, [[1], [2]], stop_token_ids=())
    assert not e.held and e.cache.free_slots == 2


def test_plan_batches_respects_slots_pages_and_order():
    assert plan_batches([10, 10, 10], 5, max_batch=8, free_slots=2, free_pages=100, max_context=64) == [[0, 1], [2]]
    assert plan_batches([60, 60, 60], 10, max_batch=8, free_slots=8, free_pages=3, max_context=128) == [[0], [1], [2]]
    assert plan_batches([1] * 5, 1, max_batch=2, free_slots=8, free_pages=100, max_context=64) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError, match="context limit"):
        plan_batches([100], 1, max_batch=1, free_slots=1, free_pages=10, max_context=64)
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches([100], 100, max_batch=1, free_slots=1, free_pages=2, max_context=1024)


def test_uniform_depends_on_seed_request_and_index_only():
    a = uniform(1, 2, 3)
    assert a == uniform(1, 2, 3) and 0.0 <= a < 1.0
    assert len({uniform(1, r, i) for r in range(10) for i in range(10)}) == 100
    assert uniform(2, 2, 3) != a
    assert float(torch.tensor(a, dtype=torch.float32)) == a
