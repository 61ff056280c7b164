"""Token selection for the rows of a batch, on the device.

`Sampler.sample(logits, requests, index)` applies the repeat penalty, then
arg-max or temperature / top-k / top-p (csrc/sampling.cu), and returns the
chosen tokens as a host list; `sample_device` leaves them on the device.  The occurrence counts the penalty needs are
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
        self._requests: Optional[list] = None           # the request index of each row, as the device holds it
        self._requests_dev = torch.zeros(max(n_rows, 1), dtype=torch.int32, device=self.device)

    def keep(self, rows: Sequence[int]) -> None:
        """Keeps the given rows (indices into the current rows), in order."""
        self.n_rows = len(rows)
        if self.counts is not None and rows:
            idx = torch.tensor(list(rows), dtype=torch.long, device=self.device)
            self.counts = self.counts.index_select(0, idx).contiguous()

    def _request_rows(self, requests: Sequence[int]) -> torch.Tensor:
        """The rows' request indices on the device (copied only when the rows change): with the seed and the
        index of the sampled token they select each row's uniform draw, which the kernel generates itself."""
        requests = list(requests)
        if requests != self._requests:
            R = len(requests)
            self._requests_dev[:R].copy_(torch.tensor(requests, dtype=torch.int32), non_blocking=False)
            self._requests = requests
            self.h2d_bytes += 4 * R
        return self._requests_dev

    def sample_device(self, logits: torch.Tensor, requests: Sequence[int], index: int,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row, left on the device in `out` (int32, at least R
        long; the sampler's own buffer if none is given).  `requests[r]` is the
        request index of row r and `index` the number of tokens sampled for
        these requests so far; the two select the row's uniform draw."""
        p = self.params
        R = logits.shape[0]
        if R != self.n_rows or len(requests) != R:
            raise ValueError(f"sampler holds {self.n_rows} rows, got logits for {R}")
        out = self.out if out is None else out
        rows = self._request_rows(requests) if p.temperature > 0 else None
        kernels.sample(logits, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                       requests=rows, seed=p.seed, index=index,
                       counts=self.counts[:R] if self.counts is not None else None, repeat_penalty=p.repeat_penalty)
        return out

    def sample(self, logits: torch.Tensor, requests: Sequence[int], index: int) -> list[int]:
        """As sample_device(), with the chosen tokens brought to the host."""
        R = logits.shape[0]
        out = self.sample_device(logits, requests, index)
        self.d2h_bytes += 4 * R
        return out[:R].tolist()
