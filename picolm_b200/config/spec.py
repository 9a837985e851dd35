"""The description of a model as data: parts with their sizes and constants,
chosen layer by layer, and the order in which the layers run.

An architecture turns its typed configuration into one `ModelSpec`.  Nothing
below the spec knows which architecture it came from: a part sees only its own
`PartSpec.params`.

The reference keeps the same facts as flags on one flat struct and per-layer
arrays: `layer_type[]` (picolm/model.h:58), `is_attn_layer` (picolm/model.h:186),
`kv_layer_map[]` for layers that share or skip a cache (picolm/model.h:416-422).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` names the implementation inside its family's registry,
    `params` holds every size and constant it needs, `prefix` is the tensor-name
    prefix of its weights relative to its owner (empty: the owner's own)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block kind) and the parts it is made of, by
    the names the arrangement gives them (`pre_norm` wants "mixer_norm", "mixer",
    "feed_forward_norm" and "feed_forward"; another arrangement may want four
    norms, one, or two mixers).  The value of a name is `(family, PartSpec)`.
    `cache_of` names another layer whose caches this layer's parts read instead
    of owning their own (they then write nothing)."""

    prefix: str
    arrangement: str
    parts: Mapping[str, Tuple[str, PartSpec]]
    cache_of: Optional[int] = None

    def part(self, name: str) -> PartSpec:
        """The spec of the part the arrangement calls `name`."""
        try:
            return self.parts[name][1]
        except KeyError:
            raise KeyError(f"layer {self.prefix!r} ({self.arrangement}) has no part {name!r}; it has: "
                           + ", ".join(sorted(self.parts))) from None


@dataclass(frozen=True)
class ModelSpec:
    """A whole model.  `schedule` is the order in which layers run: indices into
    `layers`, and an index may occur more than once."""

    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    max_positions: int
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # Regular expressions of tensor names that a checkpoint may hold and the
    # model does not use (they are not reported as unexpected).
    ignored_tensors: Tuple[str, ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        if not self.schedule:
            raise ValueError("ModelSpec.schedule is empty")
        for i in self.schedule:
            if not 0 <= i < n:
                raise ValueError(f"ModelSpec.schedule names layer {i}, but there are {n} layers")
        for i, layer in enumerate(self.layers):
            if layer.cache_of is not None:
                j = layer.cache_of
                if not 0 <= j < n or j == i:
                    raise ValueError(f"layer {i}: cache_of={j} is not another layer")
                if self.layers[j].cache_of is not None:
                    raise ValueError(f"layer {i}: cache_of={j}, which itself borrows a cache")
                first_i = self.schedule.index(i) if i in self.schedule else None
                first_j = self.schedule.index(j) if j in self.schedule else None
                if first_i is not None and (first_j is None or first_j > first_i):
                    raise ValueError(f"layer {i} reads the cache of layer {j} before that layer has run")
