"""The generation loop above the step function.

Requests (token-id prompts of unequal length) are served in batches, one
batch after another until every request is done.  A batch's prompts are
prefilled in ONE step, then each live sequence is decoded one token per step.
A sequence ends on a stop token (which is not emitted), after `max_tokens`
emitted tokens, or when its context is full; it leaves the batch at once and
its slot goes back to the cache, where a later batch uses it again.  No step
is run after a request's last wanted token.

With an engine that can take a row's token from the sampler's ids on the
device, the loop runs one step ahead of what it has read: it launches step
t+1, fed on the device by the ids of step t, and only then waits for those
ids, applies the stop test and calls `on_token`, while the device is already
busy.  What is known without the ids (a request reaching `max_tokens` or the
end of its context) is still decided in time, so such a request never rides a
step too many; a request that samples a stop token is found one step late,
has ridden along in one more step whose token is thrown away, and leaves
then.  Tokens, finish reasons and the order of `on_token` calls are those of
the loop that reads every token before the next step.

Reference: src/engine.rs:333-446 — one prompt; sample from the prompt's
logits, then loop {stop check, emit, forward, penalty, sample}; the stop token
is neither emitted nor counted (:381); that loop runs one forward more than
needed, which is not reproduced here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache import PAGE_TOKENS
from ..sampling import GenerationParams, Sampler
from .batch import StepRow


@dataclass
class GenerationResult:
    tokens: list[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop" | "length" | "context"
    prompt_tokens: int = 0


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, *, max_batch: int, free_slots: int,
                 free_pages: int, max_context: int) -> list[list[int]]:
    """Cuts request indices 0..n-1, in order, into batches that fit: at most
    `max_batch` requests and `free_slots` slots, and pages for every request
    grown to its full length (prompt + max_tokens, capped by the context)."""
    limit = min(max_batch, free_slots)
    if limit <= 0:
        raise ValueError("no slot is free for generation")
    batches: list[list[int]] = []
    cur: list[int] = []
    pages = 0
    for i, n in enumerate(prompt_lens):
        if n > max_context:
            raise ValueError(f"prompt {i} has {n} tokens, more than the context limit {max_context}")
        need = -(-min(n + max_tokens, max_context) // PAGE_TOKENS)
        if need > free_pages:
            raise ValueError(f"request {i} needs {need} cache pages, the cache has {free_pages} free")
        if cur and (len(cur) >= limit or pages + need > free_pages):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], params: Optional[GenerationParams] = None, *,
             max_batch: Optional[int] = None, on_token: Optional[Callable[[int, int], None]] = None,
             sampler_factory=Sampler, stats: Optional[dict] = None,
             pipeline: Optional[bool] = None) -> list[GenerationResult]:
    """Generates a continuation for each prompt (lists of token ids).
    `on_token(request index, token id)` is called for every emitted token.
    `pipeline`: run one step ahead of the tokens read back (default: whenever
    the engine and the sampler can); False reads every token before the next
    step is launched."""
    params = params or GenerationParams()
    params.validate()
    prompts = [list(map(int, p)) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"prompt {i}: Empty prompt")             # src/engine.rs:347-349
    stop = set(params.stop_token_ids if params.stop_token_ids is not None else engine.spec.stop_token_ids)
    results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
    if params.max_tokens == 0:
        for r in results:
            r.finish_reason = "length"
        return results
    cache = engine.cache
    batches = plan_batches(
        [len(p) for p in prompts], params.max_tokens, max_batch=max_batch or len(prompts),
        free_slots=cache.free_slots, free_pages=cache.free_pages(), max_context=engine.runtime.max_context)
    for batch in batches:
        sampler = sampler_factory(params, len(batch), engine.vocab_size, engine.runtime.device)
        ahead = (getattr(engine, "sampled", None) is not None and hasattr(sampler, "sample_device")
                 and len(batch) <= engine.sampled.rows)
        if pipeline is False or not ahead:
            _run_batch(engine, prompts, batch, params, stop, results, on_token, sampler, stats)
        else:
            _run_batch_ahead(engine, prompts, batch, params, stop, results, on_token, sampler, stats)
    return results


def _run_batch(engine, prompts, batch, params, stop, results, on_token, sampler, stats) -> None:
    max_context = engine.runtime.max_context
    live = list(batch)                                   # request indices, in row order
    slots = {i: engine.new_sequence() for i in live}
    try:
        logits = engine.step([StepRow(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live])
        n_sampled = 0
        while True:
            tokens = sampler.sample(logits, live, n_sampled)
            n_sampled += 1
            keep_rows, next_live, next_tokens = [], [], []
            for row, (i, tok) in enumerate(zip(live, tokens)):
                res = results[i]
                if tok in stop:
                    res.finish_reason = "stop"
                else:
                    res.tokens.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if len(res.tokens) >= params.max_tokens:
                        res.finish_reason = "length"
                    elif len(prompts[i]) + len(res.tokens) > max_context:   # the next token has no place in the cache
                        res.finish_reason = "context"
                if res.finish_reason:
                    engine.release(slots.pop(i))          # the slot is free for the next batch at once
                else:
                    keep_rows.append(row)
                    next_live.append(i)
                    next_tokens.append(tok)
            if not next_live:
                break
            if len(next_live) != len(live):
                sampler.keep(keep_rows)
            live = next_live
            logits = engine.step([StepRow(slots[i], [t], [0]) for i, t in zip(live, next_tokens)])
        if stats is not None:
            stats["h2d_bytes"] = stats.get("h2d_bytes", 0) + getattr(sampler, "h2d_bytes", 0)
            stats["d2h_bytes"] = stats.get("d2h_bytes", 0) + getattr(sampler, "d2h_bytes", 0)
    finally:
        for s in slots.values():                          # only reached with live slots on an error
            engine.release(s)


def _run_batch_ahead(engine, prompts, batch, params, stop, results, on_token, sampler, stats) -> None:
    """The same batch, one step ahead of the tokens read back (see the module's text)."""
    max_context = engine.runtime.max_context
    ids = engine.sampled
    live = list(batch)                                   # request indices of the rows of the step in flight
    slots = {i: engine.new_sequence() for i in live}
    d2h0 = ids.d2h_bytes

    def ends_without_stop(i: int) -> str:
        """Why request i ends with the token being sampled now, if that is no stop token."""
        n = len(results[i].tokens) + 1
        if n >= params.max_tokens:
            return "length"
        if len(prompts[i]) + n > max_context:                # the next token has no place in the cache
            return "context"
        return ""

    try:
        logits = engine.step([StepRow(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live])
        n_sampled = 0
        while True:
            sampler.sample_device(logits, live, n_sampled, out=ids.ids)
            ticket = ids.fetch(len(live))
            n_sampled += 1
            # the next step, for every row that does not end for a reason known without its token
            done = [bool(results[i].finish_reason) for i in live]        # found late: rode along, token unused
            ending = ["" if d else ends_without_stop(i) for i, d in zip(live, done)]
            keep_rows = [r for r in range(len(live)) if not done[r] and not ending[r]]
            next_live = [live[r] for r in keep_rows]
            logits = None
            if next_live:
                if len(next_live) != len(live):
                    sampler.keep(keep_rows)
                logits = engine.step([StepRow(slots[i], [0], [0], source=r) for i, r in zip(next_live, keep_rows)],
                                     keep_logits=False)
            # now the tokens of this round, while the device runs the step just launched
            tokens = ids.wait(ticket)
            for r, (i, tok) in enumerate(zip(live, tokens)):
                if done[r]:
                    continue
                res = results[i]
                if tok in stop:
                    res.finish_reason = "stop"
                else:
                    res.tokens.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    res.finish_reason = ending[r]
                if res.finish_reason:
                    engine.release(slots.pop(i))          # ordered behind the step in flight on the stream
            live = next_live
            if not live or all(results[i].finish_reason for i in live):
                break
        if stats is not None:
            stats["h2d_bytes"] = stats.get("h2d_bytes", 0) + getattr(sampler, "h2d_bytes", 0)
            stats["d2h_bytes"] = stats.get("d2h_bytes", 0) + ids.d2h_bytes - d2h0
    finally:
        for s in slots.values():
            engine.release(s)
