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


# ---- the loop that runs one step ahead of the tokens it has read ---------------------------------------------
class FakeSampledIds:
    """Stand-in for the device buffer of sampled ids: `fetch` snapshots it, `wait` hands the snapshot over."""

    def __init__(self):
        self.ids = torch.zeros(64, dtype=torch.int32)
        self.rows, self.d2h_bytes = 64, 0

    def fetch(self, n):
        return self.ids[:n].clone()

    def wait(self, ticket):
        return ticket.tolist()


class AheadEngine(FakeEngine):
    """A scripted engine whose rows may take their token from the sampled ids."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.sampled = FakeSampledIds()
        self.sources = []

    def step(self, rows, keep_logits=True):
        from tq_kv_b200.engine import StepRow
        self.sources.append([r.source for r in rows])
        real = [StepRow(r.slot, [int(self.sampled.ids[r.source])] if r.source is not None else r.tokens, r.want)
                for r in rows]
        return super().step(real)


class DeviceArgmaxSampler(ArgmaxSampler):
    def sample_device(self, logits, requests, index, out=None):
        assert logits.shape[0] == self.n_rows == len(requests)
        out[:logits.shape[0]] = logits.argmax(-1).to(torch.int32)
        return out


def _both(prompts, slots, **kw):
    outs = []
    for pipeline in (False, True):
        e = AheadEngine(slots=slots)
        params = GenerationParams.greedy(kw.get("max_tokens", 4))
        if "stop_token_ids" in kw:
            params.stop_token_ids = kw["stop_token_ids"]
        seen = []
        res = generate(e, prompts, params, sampler_factory=DeviceArgmaxSampler, pipeline=pipeline,
                       on_token=lambda i, t: seen.append((i, t)))
        assert not e.held and e.cache.free_slots == slots
        outs.append((e, res, seen))
    return outs


def test_running_ahead_gives_the_same_tokens_reasons_and_callbacks():
    for prompts, kw in (([[5], [1], [3, 4, 5]], dict(max_tokens=6)),             # stop id 7 found late, twice
                        ([[6]], dict(max_tokens=5)),                            # the first sampled token stops
                        ([[1], [2], [3], [4], [8]], dict(max_tokens=2, stop_token_ids=())),
                        ([[5], [5]], dict(max_tokens=5))):                       # all rows stop in the same round
        (e0, r0, s0), (e1, r1, s1) = _both(prompts, slots=3, **kw)
        assert [r.tokens for r in r0] == [r.tokens for r in r1]
        assert [r.finish_reason for r in r0] == [r.finish_reason for r in r1]
        assert s0 == s1
        assert e0.alloc_log == e1.alloc_log


def test_running_ahead_never_steps_past_a_length_or_context_end():
    (e0, _, _), (e1, _, _) = _both([[1], [10, 11], [3, 4, 5]], slots=3, max_tokens=3, stop_token_ids=())
    assert [len(s) for s in e1.steps] == [len(s) for s in e0.steps] == [3, 3, 3]
    assert e1.sources[1:] == [[0, 1, 2], [0, 1, 2]]                  # decode rows are fed on the device
    e = AheadEngine(max_context=4)
    params = GenerationParams.greedy(10)
    params.stop_token_ids = ()
    res = generate(e, [[1, 2]], params, sampler_factory=DeviceArgmaxSampler)
    assert res[0].tokens == [3, 4, 5] and res[0].finish_reason == "context"
    assert sum(len(r[1]) for s in e.steps for r in s) == 4


def test_a_stop_found_late_costs_one_row_of_one_step():
    (e0, r0, _), (e1, r1, _) = _both([[5], [1]], slots=2, max_tokens=5)
    assert r1[0].tokens == [6] and r1[0].finish_reason == "stop"
    assert [len(s) for s in e0.steps] == [2, 2, 1, 1, 1]
    assert [len(s) for s in e1.steps] == [2, 2, 2, 1, 1]             # request 0 rides along once more
    assert e1.sources[3] == [1]                                      # then row 1 of the last ids feeds the only row
