"""Arrangements: how one layer's norms, mixers and feed-forwards are wired around
the residual stream.  Interface of the family: built from `(layer_spec,
runtime)`; the arrangement alone reads `layer_spec.parts` (which parts a layer has
and what they are called is its business, not the model's);
`parts()` lists `(relative prefix, part)` for the weights; `cache_specs()` lists
what the layer wants of the cache, one `CacheSpec` per part that keeps something;
`prepare(max_seq_tokens)` runs once before the first step;
`forward(stream, step, caches)` runs the layer on the stream in place, `caches`
holding one entry per entry of `cache_specs()`, in that order.  An arrangement
with `narrows_rows = True` also takes `keep_rows=`: the rows that anything after the
layer will read (the model says so to the last layer of a step), so that it may
narrow the stream to them as soon as its parts no longer need the others.

`pre_norm` is the reference's Llama layer: `x += mixer(norm(x));
x += feed_forward(norm(x))` (picolm/model_core.c:1797-2210).
"""
from __future__ import annotations

from typing import List

from ..config.spec import LayerSpec, PartSpec
from .base import Part, build_part, register_part


class Arrangement(Part):
    """Base of the arrangements: builds every part the layer's spec names and answers the model's
    questions from them.  A subclass says which names it needs (`wants`) and how they are wired
    (`forward`)."""

    wants: tuple = ()
    narrows_rows = False

    def __init__(self, layer_spec: LayerSpec, runtime):
        super().__init__({}, runtime)
        self.spec = layer_spec
        missing = [n for n in self.wants if n not in layer_spec.parts]
        if missing:
            raise ValueError(f"layer {layer_spec.prefix!r}: the {self.kind} arrangement needs the parts "
                             f"{', '.join(missing)}; the spec has {', '.join(sorted(layer_spec.parts))}")
        self.named = {name: build_part(family, spec, runtime) for name, (family, spec) in layer_spec.parts.items()}
        for name, part in self.named.items():
            setattr(self, name, part)

    def parts(self):
        return [(self.spec.parts[name][1].prefix, part) for name, part in self.named.items()]

    def cache_owners(self) -> List[str]:
        """Names of the parts that keep something in the cache, in the order of `cache_specs()`."""
        return [name for name, part in self.named.items()
                if getattr(part, "cache_spec", None) is not None and part.cache_spec() is not None]

    def cache_specs(self):
        return [self.named[name].cache_spec() for name in self.cache_owners()]

    def prepare(self, max_seq_tokens: int) -> None:
        for part in self.named.values():
            prep = getattr(part, "prepare", None)
            if prep is not None:
                prep(max_seq_tokens)

    @staticmethod
    def _norm(norm, consumer, stream):
        """A norm may leave its scale to the products of the part that takes its result, when both
        say that they can (`can_defer_scale`, `takes_scaled_rows`)."""
        if getattr(norm, "can_defer_scale", False) and getattr(consumer, "takes_scaled_rows", False):
            return norm.forward(stream, defer_scale=True)
        return norm.forward(stream)


@register_part("arrangement", "pre_norm")
class PreNormBlock(Arrangement):
    wants = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    narrows_rows = True

    def forward(self, stream, step, caches, keep_rows=None):
        """`keep_rows` (the model gives it to the last layer of a step when few rows are wanted): once the mixer
        has seen all tokens, the stream is narrowed to those rows and the feed-forward runs on them alone; with
        no row to keep, nothing runs after the mixer."""
        h = self._norm(self.mixer_norm, self.mixer, stream)
        stream.pending = self.mixer.forward(h, step, caches[0] if caches else None)
        if keep_rows is not None:
            if keep_rows.numel() == 0:
                stream.pending = None
                return
            stream.narrow(keep_rows)
        h = self._norm(self.feed_forward_norm, self.feed_forward, stream)
        stream.pending = self.feed_forward.forward(h, step)


def pre_norm_layer(prefix: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                   feed_forward_norm: PartSpec, cache_of=None) -> LayerSpec:
    """The spec of a `pre_norm` layer from its four parts."""
    return LayerSpec(prefix, "pre_norm", {
        "mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer),
        "feed_forward_norm": ("norm", feed_forward_norm), "feed_forward": ("feed_forward", feed_forward),
    }, cache_of=cache_of)
