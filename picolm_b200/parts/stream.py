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
