"""The families of parts a layer is put together from, their interfaces, and
the registries that a `PartSpec.kind` is looked up in.

A part is built from `(params, runtime)`: `params` is its `PartSpec.params`
(every size and constant it needs), `runtime` the device and precision.  It
declares the weights it wants by relative tensor name, receives them in `load`,
and does its work in `forward`.  No part knows which model it is in.

Families and what `forward` takes and returns (T = tokens of the step):
  norm          forward(stream) -> h [T, d] in the run's dtype; folds the stream's
                pending residual delta in first.
  mixer         forward(h, step, cache) -> delta [T, d] fp32.  `cache` is the
                layer's `KVLayerCache`, `StateLayerCache` or None, as its
                `cache_spec()` asked for.
  feed_forward  forward(h, step) -> delta [T, d] fp32.
  position      rotates or shifts queries and keys by token position; used by
                mixers (see `parts/position.py`).
  arrangement   forward(stream, step, cache): one block, i.e. how the layer's
                norms, mixer and feed-forward are wired around the stream.
  embedding     forward(step) -> stream x [T, d] fp32.
  head          forward(h_rows) -> logits [rows, vocab] fp32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..config.spec import PartSpec
from ..runtime import Runtime

FAMILIES = ("norm", "mixer", "feed_forward", "position", "arrangement", "embedding", "head")


@dataclass(frozen=True)
class WeightSpec:
    """A tensor a part wants.  `init` tells the random-weights mode how to fill
    it: "normal" N(0, std), "ones_normal" 1 + N(0, norm_std), "zeros"; `integer`
    tensors are kept as int32."""

    shape: Tuple[int, ...]
    init: str = "normal"
    integer: bool = False


class Part:
    """Base of every part.  Subclasses set `family` through `register_part`."""

    family: str = ""
    kind: str = ""
    # True says: forward() only launches work whose dependence on the step goes through device buffers
    # (no host read of a device value, no shape that depends on the tokens), so that a decode step
    # through this part may be captured in a CUDA graph.  The engine uses graphs only if every part of
    # every block says so.
    graph_safe: bool = False
    # The same promise for steps with prompts (several tokens a sequence): nothing of the step is read on the
    # host, not even `step.slots` or `step.new_lens` (they are None in a captured step), and rows that belong to no
    # sequence (padding) may hold anything.  Steps with prompts replay graphs only if every part says so.
    graph_safe_prompts: bool = False

    def __init__(self, params: Mapping[str, Any], runtime: Optional[Runtime]):
        self.params = dict(params)
        self.runtime = runtime

    # relative tensor name -> WeightSpec
    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    # called once with the tensors named by weight_specs(), already on the device
    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass

    # bytes of weights a decode step has to read (for roofline arithmetic)
    def weight_bytes(self) -> int:
        return 0


_REGISTRY: Dict[str, Dict[str, Callable[..., Part]]] = {f: {} for f in FAMILIES}


def register_part(family: str, kind: str):
    """Class decorator: make `kind` available in `family`."""
    if family not in _REGISTRY:
        raise KeyError(f"unknown part family {family!r}; families: {', '.join(FAMILIES)}")

    def deco(cls):
        cls.family, cls.kind = family, kind
        _REGISTRY[family][kind] = cls
        return cls

    return deco


def part_class(family: str, kind: str):
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        raise KeyError(
            f"no {family} part of kind {kind!r} is registered; registered: "
            + ", ".join(sorted(_REGISTRY.get(family, {})))) from None


def build_part(family: str, spec: PartSpec, runtime: Optional[Runtime]) -> Part:
    return part_class(family, spec.kind)(spec.params, runtime)


def registered_parts(family: str):
    return sorted(_REGISTRY[family])
