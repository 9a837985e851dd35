"""Position encodings: parts that a mixer hands its projected queries, keys
and values to, and that rotate (or not) by token position while the keys and
values go into the cache.

Interface of the family: `prepare(n_positions)` once before the first step, and
`apply(qkv, q_out, kv, step, num_heads, num_kv_heads, head_dim)`, which must fill
`q_out` [T, H, hd] and, if `kv.writable`, write this step's keys and values into
`kv.k` / `kv.v` at each token's (sequence, position).

RoPE as the reference builds and applies it: `theta(p, i) = p / base^(2i/rot)`,
`(x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos)`, queries and keys only
(picolm/model_core.c:314-326, picolm/tensor.c:3216-3304).  The reference has both
pairings: adjacent `(x[2i], x[2i+1])` for its permuted GGUF Llama files and
half-split `(x[i], x[i+rot/2])` (picolm/tensor.c:3220-3235), which is how
safetensors checkpoints are laid out.  The llama3 frequency scaling is not in the
reference; it is the rule Llama-3 checkpoints state in `rope_scaling`.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Part, register_part


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> List[float]:
    """base^(-2i/rot) for i < rot/2 in double precision, with the llama3 rule
    applied when `scaling` says so: a frequency whose wavelength is below
    L0/high is kept, above L0/low divided by `factor`, and blended in between."""
    inv = [theta ** (-(2.0 * i) / rotary_dim) for i in range(rotary_dim // 2)]
    if not scaling:
        return inv
    kind = scaling.get("rope_type")
    if kind != "llama3":
        raise ValueError(f"rope scaling of type {kind!r} is not supported")
    factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    L0 = float(scaling["original_max_position_embeddings"])
    out = []
    for f in inv:
        wavelen = 2.0 * math.pi / f
        if wavelen < L0 / high:
            out.append(f)
        elif wavelen > L0 / low:
            out.append(f / factor)
        else:
            smooth = (L0 / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


@register_part("position", "rope")
class RotaryEncoding(Part):
    """params: head_dim, rotary_dim, theta, scaling (dict or None), pairing
    ("half" or "adjacent"), max_positions."""

    graph_safe = True
    graph_safe_prompts = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        if self.params["pairing"] not in ("half", "adjacent"):
            raise ValueError(f"rope pairing {self.params['pairing']!r} is not known (half, adjacent)")
        rot = self.params["rotary_dim"]
        if rot % 2 or rot > self.params["head_dim"] or rot <= 0:
            raise ValueError(f"rotary_dim={rot} must be even, positive and at most head_dim")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, n_positions: int) -> None:
        """Build cos/sin for positions [0, n_positions): angles in double
        precision on the host, rounded once to fp32."""
        if self.cos is not None and self.cos.shape[0] >= n_positions:
            return
        inv = torch.tensor(rope_inverse_frequencies(self.params["rotary_dim"], float(self.params["theta"]),
                                                    self.params.get("scaling")), dtype=torch.float64)
        pos = torch.arange(n_positions, dtype=torch.float64)
        ang = pos[:, None] * inv[None, :]
        self.cos = ang.cos().to(torch.float32).to(self.runtime.device).contiguous()
        self.sin = ang.sin().to(torch.float32).to(self.runtime.device).contiguous()

    def rotation(self):
        """The encoding as data (`ops.Rotation`), for a kernel that applies it itself."""
        return ops.Rotation(self.cos, self.sin, self.params["rotary_dim"], self.params["pairing"])

    def apply(self, qkv, q_out, kv, step, num_heads, num_kv_heads, head_dim) -> None:
        if self.cos is None or step.max_position >= self.cos.shape[0]:
            raise RuntimeError(
                f"position {step.max_position} lies beyond the rotary table; call prepare() with the cache's "
                f"longest sequence first")
        ops.rope_store(qkv, q_out, kv.k, kv.v, self.cos, self.sin, step.tok_pos, step.tok_seq, kv.block_table,
                       num_heads, num_kv_heads, head_dim, self.params["rotary_dim"], self.params["pairing"],
                       store=kv.writable)


@register_part("position", "none")
class NoPositionEncoding(Part):
    """Queries and keys go through unrotated."""

    graph_safe = True
    graph_safe_prompts = True

    def prepare(self, n_positions: int) -> None:
        pass

    def apply(self, qkv, q_out, kv, step, num_heads, num_kv_heads, head_dim) -> None:
        ops.rope_store(qkv, q_out, kv.k, kv.v, None, None, step.tok_pos, step.tok_seq, kv.block_table,
                       num_heads, num_kv_heads, head_dim, 0, "half", store=kv.writable)
