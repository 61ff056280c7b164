"""Arrangement of a layer's parts.  `prenorm_residual` is the reference's
(src/models/turbo_generic.rs:1959-1981): h += mixer(norm1(h));
h += feed_forward(norm2(h)), with the sums done in float32 on the residual
stream."""
from __future__ import annotations

from .. import kernels
from ..config import LayerSpec
from .base import StepContext
from .registry import make_part


class PrenormResidualBlock:
    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = make_part(spec.mixer_norm)
        self.mixer = make_part(spec.mixer)
        self.feed_forward_norm = make_part(spec.feed_forward_norm)
        self.feed_forward = make_part(spec.feed_forward)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, h, ctx: StepContext) -> None:
        act = ctx.runtime.act_dtype
        x = self.mixer_norm.forward(h, act)
        kernels.mark("norms")
        self.mixer.forward(x, ctx, h)
        x = self.feed_forward_norm.forward(h, act)
        kernels.mark("norms")
        self.feed_forward.forward(x, ctx, h)
