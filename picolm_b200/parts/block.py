"""Arrangements: how one layer's norms, mixer and feed-forward are wired around
the residual stream.  Interface of the family: built from `(layer_spec,
runtime)`; `parts()` lists `(relative prefix, part)` for the weights;
`forward(stream, step, cache)` runs the layer on the stream in place.

`pre_norm` is the reference's Llama layer: `x += mixer(norm(x));
x += feed_forward(norm(x))` (picolm/model_core.c:1797-2210).
"""
from __future__ import annotations

from .base import Part, build_part, register_part


@register_part("arrangement", "pre_norm")
class PreNormBlock(Part):
    def __init__(self, layer_spec, runtime):
        super().__init__({}, runtime)
        self.spec = layer_spec
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.feed_forward_norm = build_part("norm", layer_spec.feed_forward_norm, runtime)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, runtime)

    def parts(self):
        s = self.spec
        return [(s.mixer_norm.prefix, self.mixer_norm), (s.mixer.prefix, self.mixer),
                (s.feed_forward_norm.prefix, self.feed_forward_norm), (s.feed_forward.prefix, self.feed_forward)]

    def forward(self, stream, step, cache):
        h = self._norm(self.mixer_norm, self.mixer, stream)
        stream.pending = self.mixer.forward(h, step, cache)
        h = self._norm(self.feed_forward_norm, self.feed_forward, stream)
        stream.pending = self.feed_forward.forward(h, step)

    @staticmethod
    def _norm(norm, consumer, stream):
        """A norm may leave its scale to the products of the part that takes its result, when both
        say that they can (`can_defer_scale`, `takes_scaled_rows`)."""
        if getattr(norm, "can_defer_scale", False) and getattr(consumer, "takes_scaled_rows", False):
            return norm.forward(stream, defer_scale=True)
        return norm.forward(stream)
