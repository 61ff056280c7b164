"""RMS norm.  Reference: src/models/turbo_generic.rs:41-51 — computed in
float32: x / sqrt(mean(x^2) + eps) * weight; no bias, no `1 + weight`."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Norm, Runtime, WeightSpec, float32_vector


class RMSNorm(Norm):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self.params["width"])
        self.eps = float(self.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.prefix + "weight", (self.width,), "norm_scale")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.weight = float32_vector(tensors[self.prefix + "weight"])

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype, device=x.device)
        return kernels.rmsnorm(x, self.weight, self.eps, out, rows)

    def pending(self, x, out_dtype):
        """The norm of all rows of x as a `kernels.PendingNorm`: a part that
        feeds it to `kernels.linear` lets the product fold the norm in where
        it can (else the norm runs then, as a kernel of its own)."""
        return kernels.PendingNorm(x, self.weight, self.eps, out_dtype)
