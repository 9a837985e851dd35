"""Norms.  RMSNorm as the reference computes it: `ss = sum x^2;
r = 1/sqrtf(ss/size + eps); out = (x*r)*w` (picolm/tensor.c:2942-3064), the
weight used as stored (the reference's safetensors loader adds 1.0 to it,
picolm/model_core.c:993-995, which suits another model family, not this one)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Part, WeightSpec, register_part
from .stream import ResidualStream


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: size, eps.  Weight: `weight` [size]."""

    def weight_specs(self):
        return {"weight": WeightSpec((self.params["size"],), init="ones_normal")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    can_defer_scale = True
    graph_safe = True
    graph_safe_prompts = True

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, defer_scale: bool = False):
        """Normalise `x + pending`.  Without `rows` the sum is written back to the
        stream and the delta is consumed; with `rows` only those rows are
        normalised and the stream is left as it is.

        With `defer_scale` (the caller hands the result to products only) a pending product runs
        with the add, this norm's weight and the sums of squares in its epilogue, and the result is
        `ops.ScaledRows`: the product that takes it applies the scale."""
        if (defer_scale and rows is None
                and ops.residual_norm_supported(stream.pending, stream.x, self.weight)):
            h = ops.linear_residual_norm(stream.pending, stream.x, self.weight, self.params["eps"])
            stream.pending = None
            return h
        h = ops.rmsnorm(stream.x, self.weight, self.params["eps"], self.runtime.dtype,
                        delta=stream.pending, rows=rows)
        if rows is None:
            stream.pending = None
        return h
