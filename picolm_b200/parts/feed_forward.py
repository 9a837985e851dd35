"""Feed-forwards.  Interface of the family: `forward(h, step)` takes the normed
activations [T, d] and returns the residual delta [T, d] in fp32.

The gated MLP as the reference computes it: `g = Wg x`, `u = Wu x`,
`h = g / (1 + expf(-g)) * u`, `delta = Wd h`, no bias
(picolm/model_core.c:2182-2204, picolm/tensor.c:3306-3315).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec, register_part
from .mixer import _stack_rows


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """params: hidden_size, intermediate_size, activation ("silu", or "gelu_tanh": the reference's gelu,
    picolm/tensor.c:3317-3323), gate_name/up_name/down_name (relative tensor names).  The product whose
    epilogue applies the activation exists for silu; any other activation runs as a kernel of its own
    after a plain product."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        if self.params["activation"] not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {self.params['activation']!r} has no kernel; known: "
                             + ", ".join(ops.GATE_ACTIVATIONS))

    def weight_specs(self):
        p = self.params
        d, F = p["hidden_size"], p["intermediate_size"]
        return {
            p["gate_name"]: WeightSpec((F, d)),
            p["up_name"]: WeightSpec((F, d)),
            p["down_name"]: WeightSpec((d, F)),
        }

    def load(self, tensors):
        p = self.params
        gate, up = tensors[p["gate_name"]], tensors[p["up_name"]]
        # One projection for both branches.  Where the tensor-core product can apply the activation
        # in its epilogue, the rows are laid out in tiles of 64 gate rows and their 64 up rows;
        # otherwise plainly [gate | up] with the activation as a kernel of its own.
        self.fused = (p["activation"] == "silu" and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.shape[0] % 64 == 0
                      and gate.shape[1] % 8 == 0 and gate.shape[1] >= 64)
        self.w_gate_up = ops.interleave_gate_up(gate, up) if self.fused else _stack_rows([gate, up])
        self.w_down = tensors[p["down_name"]]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    takes_scaled_rows = True          # h goes into a product and nowhere else
    graph_safe = True
    graph_safe_prompts = True

    def forward(self, h, step):
        if self.fused:
            act = ops.linear_swiglu(h, self.w_gate_up, defer=True)      # handed to the next product and nowhere else
        else:
            act = ops.swiglu(ops.linear(h, self.w_gate_up, self.runtime.dtype), activation=self.params["activation"])
        return ops.linear(act, self.w_down, torch.float32, defer=True)
