"""Mixers: the part of a layer that lets tokens see other tokens.

Interface of the family: `cache_spec()` says what the layer needs of the cache
(`CacheSpec.kv`, `CacheSpec.state` or None); `prepare(max_seq_tokens)` runs once
before the first step; `forward(h, step, cache)` takes the normed activations
[T, d] of the step's tokens and returns the residual delta [T, d] in fp32.

Attention as the reference computes it: q/k/v projections without bias, RoPE on
q and k, keys and values appended to the cache, causal softmax(q.K * scale) . V
with consecutive query heads sharing a KV head (`g = h / (H/G)`), then the output
projection (picolm/model_core.c:1849-2151, picolm/model_attention.c:43-140).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.spec import CacheSpec
from ..config.spec import PartSpec
from .base import Part, WeightSpec, build_part, register_part


def _stack_rows(tensors):
    """Concatenate weight matrices along the output features.  If their stored
    types differ, all are widened to float32 (exact)."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(list(tensors), dim=0).contiguous()


@register_part("mixer", "attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale (None:
    1/sqrt(head_dim)), window (None: all keys), position (a PartSpec of the
    position family), q_name/k_name/v_name/o_name (relative tensor names)."""

    @property
    def graph_safe(self) -> bool:
        """forward() launches kernels whose dependence on the step goes through device buffers only (apart
        from sizes fixed per batch size); the position encoding has to say the same of itself."""
        return bool(getattr(self.position, "graph_safe", False))

    @property
    def graph_safe_prompts(self) -> bool:
        return bool(getattr(self.position, "graph_safe_prompts", False))

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.H, self.G, self.hd, self.d = p["num_heads"], p["num_kv_heads"], p["head_dim"], p["hidden_size"]
        if self.H % self.G:
            raise ValueError(f"num_heads={self.H} is not a multiple of num_kv_heads={self.G}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.window = p.get("window")
        pos = p.get("position") or PartSpec("none")
        self.position = build_part("position", pos, runtime)

    def weight_specs(self):
        p, H, G, hd, d = self.params, self.H, self.G, self.hd, self.d
        return {
            p["q_name"]: WeightSpec((H * hd, d)),
            p["k_name"]: WeightSpec((G * hd, d)),
            p["v_name"]: WeightSpec((G * hd, d)),
            p["o_name"]: WeightSpec((d, H * hd)),
        }

    def load(self, tensors):
        p = self.params
        # one projection for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = _stack_rows([tensors[p["q_name"]], tensors[p["k_name"]], tensors[p["v_name"]]])
        self.w_o = tensors[p["o_name"]]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def cache_spec(self):
        return CacheSpec.kv(self.G, self.hd, self.window)

    def prepare(self, max_seq_tokens: int) -> None:
        self.position.prepare(max_seq_tokens)

    takes_scaled_rows = True          # h goes into a product and nowhere else

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        qkv = ops.linear(h, self.w_qkv, dt)
        # a position encoding that can describe itself as a rotation (`rotation()`) may be applied, and the
        # cache written, by the decode attention kernel itself
        rotation = self.position.rotation() if step.is_decode and hasattr(self.position, "rotation") else None
        if rotation is not None and ops.attention_decode_rope_supported(qkv, cache, rotation, self.hd):
            ctx = ops.attention_decode_rope(qkv, cache, step, self.H, self.G, self.hd, self.scale, rotation)
        else:
            q = torch.empty((h.shape[0], self.H, self.hd), dtype=dt, device=h.device)
            self.position.apply(qkv, q, cache, step, self.H, self.G, self.hd)
            ctx = ops.attention(q, cache, step, self.G, self.scale)
        return ops.linear(ctx, self.w_o, torch.float32, defer=True)
