"""What a layer asks of the cache.

The reference sizes one K block and one V block for the layers that attend
(`kv_layer_map`, `kv_layer_ordinal`, picolm/model.h:416-422,
picolm/model_core.c:590-606) and separate fixed-size state for recurrent layers
(`ssm_conv_state`, `ssm_state`, picolm/model.h:303-304).  Here each mixer hands
back one `CacheSpec`, and layers with equal specs share one storage group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class CacheSpec:
    kind: str                                   # "kv" or "state"
    num_kv_heads: int = 0                       # kv
    head_dim: int = 0                           # kv
    window: Optional[int] = None                # kv: keep only the last `window` positions
    shape: Tuple[int, ...] = ()                 # state: per-sequence shape
    dtype: str = "float32"                      # state: element type

    @staticmethod
    def kv(num_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheSpec":
        if num_kv_heads <= 0 or head_dim <= 0:
            raise ValueError("a kv cache needs positive num_kv_heads and head_dim")
        if window is not None and window <= 0:
            raise ValueError("a window must be positive")
        return CacheSpec("kv", num_kv_heads=num_kv_heads, head_dim=head_dim, window=window)

    @staticmethod
    def state(shape, dtype: str = "float32") -> "CacheSpec":
        return CacheSpec("state", shape=tuple(int(s) for s in shape), dtype=dtype)

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.shape, self.dtype)
