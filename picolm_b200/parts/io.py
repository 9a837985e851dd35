"""The two ends of the model: token embedding and LM head.

Embedding: `x = float(embed[token])`, no scale (picolm/model_core.c:1785-1786).
Head: `logits = W x`, fp32, no bias, no soft-cap (picolm/model_core.c:2220); with
tied embeddings W is the embedding matrix itself (picolm/safetensors.c:248-251).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name (absolute tensor name)."""

    def weight_specs(self):
        return {self.params["name"]: WeightSpec((self.params["vocab_size"], self.params["hidden_size"]))}

    def load(self, tensors):
        self.table = tensors[self.params["name"]]

    def forward(self, step):
        return ops.embed(step.tok_ids, self.table)


@register_part("head", "lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, name (absolute tensor name; the
    embedding's own name when the two are tied)."""

    def weight_specs(self):
        return {self.params["name"]: WeightSpec((self.params["vocab_size"], self.params["hidden_size"]))}

    def load(self, tensors):
        self.weight = tensors[self.params["name"]]

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, h_rows):
        return ops.linear(h_rows, self.weight, torch.float32)
