"""Dense SwiGLU feed-forward.  Reference: src/models/turbo_generic.rs:105-110
— down(silu(gate x) * (up x)), no biases; :1980 — residual sum.  Gate and up
weights are concatenated at bind time so that one product yields both."""
from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, Runtime, StepContext, WeightSpec


class SwiGLU(FeedForward):
    takes_pending_norm = True           # x goes to kernels.linear only
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.names = dict(self.params.get("names", {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}))
        self.w_gate_up = self.w_down = None

    def _n(self, which):
        return f"{self.prefix}{self.names[which]}.weight"

    def weight_specs(self):
        return [WeightSpec(self._n("gate"), (self.inter, self.hidden), "matrix"),
                WeightSpec(self._n("up"), (self.inter, self.hidden), "matrix"),
                WeightSpec(self._n("down"), (self.hidden, self.inter), "matrix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        g, u = tensors[self._n("gate")], tensors[self._n("up")]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self._n("down")].contiguous()

    def forward(self, x, ctx: StepContext, residual):
        act = kernels.linear(x, self.w_gate_up, swiglu=True, out_dtype=ctx.runtime.act_dtype)
        kernels.mark("gate_up")
        kernels.linear(act, self.w_down, out=residual, accumulate=True)
        kernels.mark("down")
