"""A decoder assembled from a `ModelSpec`: embedding, the blocks, the order in
which they run (a list that may name a block twice or let an entry read an
earlier entry's cache), final norm and head.

Reference: src/models/turbo_generic.rs:1950-1987 is the forward pass this
generalises; :1983-1986 norms every row and keeps the last — here only the
wanted rows are normed and multiplied with the head.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import KVLayerView, KVRequest, SequenceCache, StateRequest
from ..config import ConfigError, ModelSpec
from ..parts import Runtime, StepBatch, StepContext, WeightSpec, make_block, make_part


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = make_part(spec.embedding)
        self.blocks = [make_block(ls) for ls in spec.layers]
        self.final_norm = make_part(spec.final_norm)
        self.head = make_part(spec.head)
        self.runtime: Optional[Runtime] = None

    # ---- weights ----------------------------------------------------------
    def _all_parts(self):
        yield self.embedding
        for b in self.blocks:
            for p in b.parts():
                yield p
                pos = getattr(p, "position", None)
                if pos is not None:
                    yield pos
        yield self.final_norm
        yield self.head

    @property
    def graph_capturable(self) -> bool:
        return all(getattr(p, "graph_capturable", True) for p in self._all_parts())

    @property
    def padded_rows_ok(self) -> bool:
        """Whether a step may carry padded rows (see Part.padded_rows_ok): every part and block says so."""
        return (all(getattr(p, "padded_rows_ok", False) for p in self._all_parts())
                and all(getattr(b, "padded_rows_ok", False) for b in self.blocks))

    def weight_specs(self) -> dict[str, WeightSpec]:
        """Every tensor the model expects, by name.  Two parts may name the
        same tensor (a tied head) if they agree on its shape."""
        specs: dict[str, WeightSpec] = {}
        for part in self._all_parts():
            for ws in part.weight_specs():
                old = specs.get(ws.name)
                if old is not None and tuple(old.shape) != tuple(ws.shape):
                    raise ConfigError(f"tensor '{ws.name}' is wanted with shapes {old.shape} and {ws.shape}")
                specs.setdefault(ws.name, ws)
        return specs

    def ignored_weights(self) -> list[str]:
        names: list[str] = []
        for part in self._all_parts():
            names += part.ignored_weights()
        expected = self.weight_specs()
        return [n for n in names if n not in expected]

    def bind(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        shared: dict = {}
        self.embedding.bind(tensors, runtime, shared)
        for b in self.blocks:
            for p in b.parts():
                p.bind(tensors, runtime, shared)
        self.final_norm.bind(tensors, runtime, shared)
        self.head.bind(tensors, runtime, shared)

    # ---- cache ------------------------------------------------------------
    def cache_requests(self) -> tuple[dict[int, KVRequest], dict[int, StateRequest]]:
        """What the schedule entries that own a cache ask for, by entry index."""
        kv: dict[int, KVRequest] = {}
        state: dict[int, StateRequest] = {}
        for i, e in enumerate(self.spec.schedule):
            if e.cache_of is not None:
                continue
            mixer = self.blocks[e.layer].mixer
            r = mixer.cache_request()
            if r is not None:
                kv[i] = r
            s = mixer.state_request()
            if s is not None:
                state[i] = s
        return kv, state

    def check_step(self, start_pos: list[int], step_lens: list[int]) -> None:
        for e in self.spec.schedule:
            self.blocks[e.layer].mixer.check_step(start_pos, step_lens, e.cache_of is None)

    # ---- one step -----------------------------------------------------------
    def forward(self, batch: StepBatch, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the scheduled blocks; returns float32
        logits [wanted rows, vocab] (None if no row is wanted)."""
        rt = self.runtime
        h = self.embedding.forward(batch.tokens)
        kernels.mark("embed")
        for i, e in enumerate(self.spec.schedule):
            owner = i if e.cache_of is None else e.cache_of
            ctx = StepContext(batch=batch, runtime=rt, entry=i)
            if owner in cache.group_of_entry:
                gi, k_pages, v_pages = cache.layer_pages(owner)
                table, width = batch.block_tables[gi]
                g = cache.groups[gi]
                ctx.kv = KVLayerView(k_pages, v_pages, table, width, g.ring_pages, g.book.page_tokens,
                                     writes=e.cache_of is None)
            ctx.state = cache.state.get(owner)
            self.blocks[e.layer].forward(h, ctx)
        if batch.n_logit_rows == 0:
            return None
        normed = self.final_norm.forward(h, rt.act_dtype, rows=batch.logit_rows)
        logits = self.head.forward(normed)
        kernels.mark("head")
        return logits
