"""Decode steps, and single prompts, as replayed CUDA graphs (DecodeGraph, PromptGraph).

A decode step of B sequences launches a few hundred small kernels; launching
them from Python costs more than running them.  For each batch size the step
is therefore captured once into a CUDA graph over static buffers (the packed
step metadata with block tables of full width, the logits) and replayed:
per step, the host fills one pinned staging buffer, copies it to the device
and replays.  Staging buffers form a small ring, each guarded by an event, so
that the host may run a few steps ahead of the device.  A row's token is
either in the staging buffer or, if the row names a `source`, taken on the
device from the ids the sampler wrote last (the captured step begins with
that selection), so that the host can launch a step before it has read the
token that feeds it.

The captured step is the same `DecoderModel.forward` that an uncaptured step
runs; only planning inputs are frozen: attention plans its splits for the
context limit (each token still cuts its own key range evenly).
"""
from __future__ import annotations

import gc

import numpy as np
import torch

from ..cache import SequenceCache
from ..parts import StepBatch
from .batch import _pad4


def forward_step(model, cache: SequenceCache, sampled_ids: torch.Tensor, batch: StepBatch):
    """One step of `model` on a packed batch: tokens that name a source are
    first taken from the sampler's ids on the device."""
    from .. import kernels
    if batch.any_source:
        kernels.select_tokens(batch.tokens, batch.tok_src, sampled_ids)
    return model.forward(batch, cache)


class DecodeGraph:
    RING = 4

    def __init__(self, model, cache: SequenceCache, sampled_ids: torch.Tensor, runtime, B: int):
        self.model, self.cache, self.sampled_ids, self.B = model, cache, sampled_ids, B
        dev = runtime.device
        self.widths = []
        for g in cache.groups:
            full = -(-runtime.max_context // g.book.page_tokens)
            self.widths.append(min(full, g.book.ring_pages) if g.book.ring_pages else full)
        seg = [B, B, B, B + 1, B, B, B, B, B] + [B * w for w in self.widths]
        self.offs, total = [], 0
        for s in seg:
            self.offs.append(total)
            total += _pad4(s)
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        o = self.offs
        arange = np.arange(B + 1, dtype=np.int32)
        for h in self.host:                                   # the parts of the layout that never change
            a = h.numpy()
            a[o[1]:o[1] + B] = arange[:B]                     # tok_seq
            a[o[3]:o[3] + B + 1] = arange                     # cu_seqlens
            a[o[7]:o[7] + B] = arange[:B]                     # logit_rows: every row
        d = self.dev

        def seg_view(i, n):
            return d[o[i]:o[i] + n]

        self.batch = StepBatch(
            n_tokens=B, n_seqs=B, tokens=seg_view(0, B), tok_seq=seg_view(1, B), tok_pos=seg_view(2, B),
            cu_seqlens=seg_view(3, B + 1), slots=seg_view(4, B), start_pos=seg_view(5, B), new_lens=seg_view(6, B),
            logit_rows=seg_view(7, B), n_logit_rows=B,
            block_tables=[(seg_view(9 + gi, B * w), w) for gi, w in enumerate(self.widths)],
            host_slots=[0] * B, host_start=[1] * B, host_lens=[1] * B, packed_bytes=total * 4,
            plan_max_len=runtime.max_context, tok_src=seg_view(8, B), any_source=True)
        self.graph = None
        self.logits = None
        self.kernels_per_replay = 0
        # what the host runtime fills per step (csrc/host_runtime.cpp, tqh_pack_decode), and where
        self._offs = np.asarray(self.offs, dtype=np.int32)
        self._widths = np.asarray(self.widths or [1], dtype=np.int32)
        self._slots = np.zeros(B, dtype=np.int32)
        self._tokens = np.zeros(B, dtype=np.int32)
        self._sources = np.zeros(B, dtype=np.int32)

    def _fill(self, rows) -> torch.Tensor:
        i = self.turn % self.RING
        self.turn += 1
        if self.events[i] is not None:
            self.events[i].synchronize()                      # the copy that last used this buffer is done
        h = self.host[i]
        slots = [r.slot for r in rows]
        self._slots[:] = slots
        self._tokens[:] = [r.tokens[0] for r in rows]
        self._sources[:] = [-1 if r.source is None else r.source for r in rows]
        # tokens, sources, positions, slots, lengths and the block tables, written by the host runtime in one call
        self.cache.book.pack_decode(self._slots, self._tokens, self._sources, self._offs, self._widths, h.data_ptr())
        self.batch.host_slots = slots
        self.dev.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return h

    def run(self, rows, keep: bool = True) -> torch.Tensor:
        """Runs one decode step for `rows` (already reserved in the cache);
        returns float32 logits [B, vocab]: a copy of the graph's static output,
        or with `keep` False that output itself, which the next step overwrites."""
        from .. import kernels
        self._fill(rows)
        if self.graph is None:
            # First use: the step runs once, launched kernel by kernel (which also warms allocators and
            # libraries), and is then captured for the steps to come.  Capturing runs nothing, so a part
            # with state of its own advances it once, like in every other step.
            n0 = kernels.launches[0]
            logits = forward_step(self.model, self.cache, self.sampled_ids, self.batch)
            self.kernels_per_replay = kernels.launches[0] - n0
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            # No garbage collection while the stream captures: collecting an older engine's graphs would
            # destroy them, which CUDA does not permit during a capture and which would invalidate this one.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self.logits = forward_step(self.model, self.cache, self.sampled_ids, self.batch)
            finally:
                if gc_was_on:
                    gc.enable()
            kernels.launches[0] -= self.kernels_per_replay     # capturing launched nothing
            self.graph = g
            return logits
        self.graph.replay()
        kernels.launches[0] += self.kernels_per_replay
        return self.logits.clone() if keep else self.logits


class PromptGraph:
    """Whole prompts of B sequences from position 0, as a replayed CUDA graph.

    A short prompt is a few hundred kernels of a few microseconds each: launched from Python one by one, the
    host sets the pace (a 32-token prompt of a small model takes ten times its device time).  The step is
    therefore padded with rows of token 0 (they continue the last sequence) to a multiple of PAD tokens and
    captured once per (number of sequences, padded size) over static buffers, as decode steps are per batch
    size; how the tokens divide among the sequences is data (cu_seqlens), not part of the capture.  Padded
    rows change nothing that lasts: causal attention lets no real row see them, every other part works row by
    row, and the rotary kernel caches only rows below their sequence's new length (`new_lens`, which holds the
    real one).  Pages are reserved and lengths committed for the real tokens only.  The engine takes this path
    only for models whose parts all say `padded_rows_ok`, with no per-sequence state, and for one wanted row
    per sequence."""
    PAD = 64
    MAX_TOKENS = 2048          # longer steps are bound by the device, not by their launches
    MAX_ROWS = 16
    MAX_GRAPHS = 96            # captured graphs an engine keeps (every size of a single prompt, and some more)
    RING = 2

    def __init__(self, model, cache: SequenceCache, sampled_ids: torch.Tensor, runtime, B: int, T_pad: int,
                 pool=None):
        self.model, self.cache, self.sampled_ids, self.B, self.T = model, cache, sampled_ids, B, T_pad
        dev = runtime.device
        self.widths = []
        for g in cache.groups:
            full = -(-runtime.max_context // g.book.page_tokens)
            self.widths.append(min(full, g.book.ring_pages) if g.book.ring_pages else full)
        T = T_pad
        seg = [T, T, T, B + 1, B, B, B, B, T] + [B * w for w in self.widths]
        self.offs, total = [], 0
        for s in seg:
            self.offs.append(total)
            total += _pad4(s)
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        o = self.offs
        for h in self.host:                                   # what never changes
            a = h.numpy()
            a[o[8]:o[8] + T] = -1                             # no token comes from the sampler's ids
        d = self.dev

        def seg_view(i, n):
            return d[o[i]:o[i] + n]

        self.batch = StepBatch(
            n_tokens=T, n_seqs=B, tokens=seg_view(0, T), tok_seq=seg_view(1, T), tok_pos=seg_view(2, T),
            cu_seqlens=seg_view(3, B + 1), slots=seg_view(4, B), start_pos=seg_view(5, B), new_lens=seg_view(6, B),
            logit_rows=seg_view(7, B), n_logit_rows=B,
            block_tables=[(seg_view(9 + gi, B * w), w) for gi, w in enumerate(self.widths)],
            host_slots=[0] * B, host_start=[0] * B, host_lens=[T] * B, packed_bytes=total * 4,      # (lengths: an upper bound)
            tok_src=seg_view(8, T), any_source=False)
        self.pool = pool
        self.graph = None
        self.logits = None
        self.kernels_per_replay = 0

    def _fill(self, rows) -> None:
        i = self.turn % self.RING
        self.turn += 1
        if self.events[i] is not None:
            self.events[i].synchronize()                      # the copy that last used this buffer is done
        h = self.host[i]
        a, o, B, T = h.numpy(), self.offs, self.B, self.T
        at = 0
        for b, r in enumerate(rows):
            n = len(r.tokens)
            last = b == B - 1
            end = T if last else at + n                       # the padding continues the last sequence
            a[o[0] + at:o[0] + at + n] = r.tokens
            a[o[0] + at + n:o[0] + end] = 0
            a[o[1] + at:o[1] + end] = b
            a[o[2] + at:o[2] + end] = np.arange(end - at, dtype=np.int32)
            a[o[3] + b + 1] = end
            a[o[4] + b] = r.slot
            a[o[6] + b] = n                                   # the real length: rows from n on are not cached
            a[o[7] + b] = at + r.want[0]
            for gi, w in enumerate(self.widths):
                pages = self.cache.book.pages(gi, r.slot)
                a[o[9 + gi] + b * w:o[9 + gi] + b * w + len(pages)] = pages
            at = end
        self.batch.host_slots = [r.slot for r in rows]
        self.dev.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def run(self, rows) -> torch.Tensor:
        """Runs the prompts `rows` (pages reserved, nothing cached yet); returns float32 logits [B, vocab]."""
        from .. import kernels
        self._fill(rows)
        if self.graph is None:
            # first use: once kernel by kernel, then captured for the prompts to come (see DecodeGraph.run)
            n0 = kernels.launches[0]
            logits = forward_step(self.model, self.cache, self.sampled_ids, self.batch)
            self.kernels_per_replay = kernels.launches[0] - n0
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g, pool=self.pool):
                    self.logits = forward_step(self.model, self.cache, self.sampled_ids, self.batch)
            finally:
                if gc_was_on:
                    gc.enable()
            kernels.launches[0] -= self.kernels_per_replay     # capturing launched nothing
            self.graph = g
            return logits
        self.graph.replay()
        kernels.launches[0] += self.kernels_per_replay
        return self.logits.clone()
