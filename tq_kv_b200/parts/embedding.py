"""Token embedding and LM head.

Reference: src/models/turbo_generic.rs:1958 — embedding is a row gather
without scaling; :1983-1986 — final norm, then logits = n · W^T without bias
or scaling, for the wanted rows only; :2079-2084 — the head uses
`lm_head.weight` if the checkpoint has it and the embedding matrix otherwise
(here the configuration decides which).
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, Runtime, WeightSpec


class TokenEmbedding(Part):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.table = None
        self.status = None

    def weight_specs(self):
        return [WeightSpec(self.prefix + "weight", (self.vocab, self.width), "embedding")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.table = tensors[self.prefix + "weight"].contiguous()
        self.status = torch.zeros(1, dtype=torch.int32, device=runtime.device)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """The float32 residual stream [T, width] of the step's tokens."""
        out = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        return kernels.embed(tokens, self.table, out, self.status)


class LMHead(Part):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.tied_to = self.params.get("tied_to")
        self.weight = None

    def weight_specs(self):
        if self.tied_to:
            return [WeightSpec(self.tied_to, (self.vocab, self.width), "embedding")]
        return [WeightSpec(self.prefix + "weight", (self.vocab, self.width), "matrix")]

    def ignored_weights(self):
        return [self.prefix + "weight"] if self.tied_to else []

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.weight = tensors[self.tied_to or self.prefix + "weight"].contiguous()

    def forward(self, normed_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [rows, vocab] of already normed rows."""
        return kernels.linear(normed_rows, self.weight, out_dtype=torch.float32)
