"""Token selection for the rows of a batch, on the device.

`Sampler.sample(logits, requests, index)` applies the repeat penalty, then
arg-max or temperature / top-k / top-p (csrc/sampling.cu), and returns the
chosen tokens as a host list.  The occurrence counts the penalty needs are
per-row state held here; `keep(rows)` drops the rows of finished requests.

Reference: src/engine.rs:353-362 (choice of sampler), :403-419 (penalty over
generated tokens only; the first sampled token sees none because nothing has
been generated yet).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from .params import GenerationParams
from .rng import uniform


class Sampler:
    def __init__(self, params: GenerationParams, n_rows: int, vocab_size: int, device):
        params.validate()
        self.params = params
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.n_rows = n_rows
        self.counts: Optional[torch.Tensor] = None
        if params.repeat_penalty != 1.0:
            self.counts = torch.zeros((n_rows, vocab_size), dtype=torch.int32, device=self.device)
        self.out = torch.zeros(n_rows, dtype=torch.int32, device=self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def keep(self, rows: Sequence[int]) -> None:
        """Keeps the given rows (indices into the current rows), in order."""
        self.n_rows = len(rows)
        if self.counts is not None and rows:
            idx = torch.tensor(list(rows), dtype=torch.long, device=self.device)
            self.counts = self.counts.index_select(0, idx).contiguous()

    def sample(self, logits: torch.Tensor, requests: Sequence[int], index: int) -> list[int]:
        """One token per row.  `requests[r]` is the request index of row r and
        `index` the number of tokens sampled for these requests so far; the two
        select the row's uniform draw."""
        p = self.params
        R = logits.shape[0]
        if R != self.n_rows or len(requests) != R:
            raise ValueError(f"sampler holds {self.n_rows} rows, got logits for {R}")
        uniforms = None
        if p.temperature > 0:
            u = torch.tensor([uniform(p.seed, r, index) for r in requests], dtype=torch.float32)
            if self.device.type == "cuda":
                u = u.pin_memory()
            uniforms = u.to(self.device, non_blocking=True)
            self.h2d_bytes += 4 * R
        kernels.sample(logits, self.out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                       uniforms=uniforms, counts=self.counts[:R] if self.counts is not None else None,
                       repeat_penalty=p.repeat_penalty)
        self.d2h_bytes += 4 * R
        return self.out[:R].tolist()
