"""Choosing the next token: greedy, or the reference's chain
softmax -> top-k -> top-p -> min-p -> p^(1/T) -> draw (picolm/sampler.c:48-125),
with the reference's defaults: temperature 0.8, top-p 0.9, top-k 40
(picolm/picolm.c:774-776), min-p 0.05 (picolm/picolm.c:1230), seed 42 and seed 0
read as 42 (picolm/sampler.c:43).

The kept set and the weights are the reference's; the draw is not token-identical to it: the kernel walks
the kept tokens in index order where the reference walks them in descending probability
(picolm/sampler.c:112-121), so with the same seed and the same logits the two pick from the same
distribution but not always the same token (tests/test_plain.py shows a case).

Random numbers are the reference's xorshift64 (picolm/sampler.c:10-21).  The
reference has one stream for its one sequence; here every sequence has a stream
of its own, seeded `seed + index of the request`, so that what a request
generates does not depend on which other requests share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops

_MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8          # <= 0: greedy
    top_p: float = 0.9                # >= 1: off
    top_k: int = 40                   # <= 0: off
    min_p: float = 0.05               # <= 0: off
    seed: int = 42

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def stream_seed(seed: int, request_index: int) -> int:
    """The xorshift64 state a request starts from (never 0)."""
    s = (int(seed) + int(request_index)) & _MASK64
    return s if s else 42


def _as_signed(x: int) -> int:
    return x - (1 << 64) if x >= (1 << 63) else x


class Sampler:
    """Samples one token per row of a batch on the device.  `request_indices`
    are the positions of the batch's sequences among all requests of the call."""

    def __init__(self, params: SamplingParams, request_indices: Sequence[int], device):
        self.params = params
        self.device = device
        self.rng: Optional[torch.Tensor] = None
        if not params.greedy:
            states = [_as_signed(stream_seed(params.seed, i)) for i in request_indices]
            self.rng = torch.tensor(states, dtype=torch.int64, device=device)

    def keep(self, rows: Sequence[int]) -> None:
        """Drop the streams of sequences that have ended: keep `rows` (indices
        into the current batch order)."""
        if self.rng is not None:
            self.rng = self.rng[torch.tensor(list(rows), dtype=torch.int64, device=self.device)].contiguous()

    def sample(self, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits fp32 [rows, vocab] -> int32 [rows] (into `out` if given)."""
        p = self.params
        if p.greedy:
            return ops.argmax(logits, out=out)
        return ops.sample(logits, self.rng, p.temperature, p.top_k, p.top_p, p.min_p, out=out)
