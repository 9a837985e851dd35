"""The residual stream of a step: fp32 `x` [T, d] and the delta that the last
part produced and that has not been added yet.  The add is folded into the next
norm (one pass over the stream instead of two)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class ResidualStream:
    x: torch.Tensor                              # fp32 [T, d]
    pending: Optional[torch.Tensor] = None       # fp32 [T, d], to be added to x
    narrowed: bool = False                       # `narrow` has run: the rows are the wanted rows, in their order

    def narrow(self, rows: torch.Tensor) -> None:
        """Keep the rows `rows` (int32, on the device) only, in that order: what is left of a step's last layer
        once its mixer has seen all tokens is needed at the wanted rows alone.  A product that has not run yet
        (`ops.PendingLinear`) is narrowed at its left operand: it then runs on those rows."""
        from .. import ops
        self.x = ops.gather_rows(self.x, rows)
        p = self.pending
        if p is not None:
            if isinstance(p, ops.PendingLinear):
                a = p.a.materialize() if isinstance(p.a, ops.LazyRows) else p.a
                self.pending = ops.PendingLinear(ops.gather_rows(a, rows), p.w)
            else:
                self.pending = ops.gather_rows(p, rows)
        self.narrowed = True
