"""Arrangement of a layer's parts.  `prenorm_residual` is the reference's
(src/models/turbo_generic.rs:1959-1981): h += mixer(norm1(h));
h += feed_forward(norm2(h)), with the sums done in float32 on the residual
stream.

A block kind is a class built from a `LayerSpec` with `parts()` (every part
it holds, for weights and binding), `mixer` (the one part that may ask for a
cache or state) and `forward(h, ctx)`.  It takes the parts it arranges from
the layer by name (`spec.part("mixer")`, or any name of `extra_parts`)."""
from __future__ import annotations

from .. import kernels
from ..config import LayerSpec
from .base import StepContext
from .registry import make_part


class PrenormResidualBlock:
    padded_rows_ok = True               # as far as its parts are

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = make_part(spec.part("mixer_norm"))
        self.mixer = make_part(spec.part("mixer"))
        self.feed_forward_norm = make_part(spec.part("feed_forward_norm"))
        self.feed_forward = make_part(spec.part("feed_forward"))

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, h, ctx: StepContext) -> None:
        act = ctx.runtime.act_dtype
        x = self._normed(self.mixer_norm, self.mixer, h, act)
        kernels.mark("norms")
        self.mixer.forward(x, ctx, h)
        x = self._normed(self.feed_forward_norm, self.feed_forward, h, act)
        kernels.mark("norms")
        self.feed_forward.forward(x, ctx, h)

    @staticmethod
    def _normed(norm, consumer, h, act):
        """The norm's result for `consumer` — left pending if the consumer only hands it to `kernels.linear`
        (it says so with `takes_pending_norm`) and the norm can be deferred, so that the product may fold it in."""
        if getattr(consumer, "takes_pending_norm", False) and hasattr(norm, "pending"):
            return norm.pending(h, act)
        return norm.forward(h, act)
