"""A model put together from a `ModelSpec`: embedding, blocks, final norm and
head, and the schedule in which the blocks run.  Architecture-agnostic: what the
parts are is decided by the spec, and what runs is decided by the schedule.

One forward of a step follows the reference's order (picolm/model_core.c:1785-2220,
picolm/model_core.c:2757-3225): embed, the layers, then final norm and LM head on
the rows whose logits are wanted only (the reference's prefill does this for the
last row, picolm/model_core.c:3219-3225).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..cache.sequence_cache import KVLayerCache, SequenceCache, StateLayerCache
from ..cache.spec import CacheSpec
from ..config.spec import ModelSpec
from ..parts import ResidualStream, WeightSpec, build_part, part_class
from ..parts.base import Part
from ..runtime import Runtime


def _join(*names: str) -> str:
    return ".".join(n for n in names if n)


class Model:
    def __init__(self, spec: ModelSpec, runtime: Optional[Runtime]):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [part_class("arrangement", layer.arrangement)(layer, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.lm_head, runtime)
        self.loaded = False
        # Called as layer_hook(run, layer, done) before (done False) and after (done True) every scheduled layer
        # of a step: the reference's per-layer benchmark callback (bench_layer_cb_t, picolm/model.h:528-533,
        # fired around each layer in picolm/model_core.c:235-252).  While it is set, steps are not replayed
        # from captured graphs.
        self.layer_hook: Optional[Callable[[int, int, bool], None]] = None

    # ---------------------------------------------------------------- weights
    def named_parts(self) -> List[Tuple[str, Part]]:
        """(absolute tensor-name prefix, part) of every part that owns weights."""
        out: List[Tuple[str, Part]] = [(self.spec.embedding.prefix, self.embedding)]
        for layer, block in zip(self.spec.layers, self.blocks):
            for rel, part in block.parts():
                out.append((_join(layer.prefix, rel), part))
        out.append((self.spec.final_norm.prefix, self.final_norm))
        out.append((self.spec.lm_head.prefix, self.head))
        return out

    def expected_tensors(self) -> Dict[str, WeightSpec]:
        """Every tensor name the model reads, with its shape.  Two parts may name
        the same tensor (tied embeddings); their shapes must agree."""
        out: Dict[str, WeightSpec] = {}
        for prefix, part in self.named_parts():
            for rel, ws in part.weight_specs().items():
                name = _join(prefix, rel)
                if name in out and out[name].shape != ws.shape:
                    raise ValueError(f"tensor {name!r} is wanted with shapes {out[name].shape} and {ws.shape}")
                out.setdefault(name, ws)
        return out

    def load_tensors(self, get: Callable[[str], torch.Tensor]) -> None:
        """Hand every part its tensors; `get(name)` returns the device tensor
        (the same object for the same name, so tied weights stay one buffer)."""
        for prefix, part in self.named_parts():
            part.load({rel: get(_join(prefix, rel)) for rel in part.weight_specs()})
        self.loaded = True

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every matrix of every scheduled
        layer once, the norms, and the LM head (the embedding rows are negligible)."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for i in self.spec.schedule:
            total += sum(part.weight_bytes() for _, part in self.blocks[i].parts())
        return total

    # ------------------------------------------------------------------ cache
    # The cache is kept per *run* of a layer (per entry of the schedule), not per
    # layer: a layer that the schedule names twice shares its weights between
    # the two runs, but each run sees other inputs and so has keys, values or
    # state of its own.  A layer with `cache_of = j` owns nothing: each of its
    # runs reads what the latest earlier run of layer j wrote.  What a layer keeps
    # is its arrangement's business (`cache_specs()`): the model only numbers it.
    def cache_specs(self) -> List[CacheSpec]:
        """What the runs of the schedule own in the cache, as one flat list: for every run that owns
        its caches, what its arrangement asks for (one entry per part that keeps something; none for a
        layer without such parts).  The position in this list is the cache's number in `SequenceCache`."""
        out: List[CacheSpec] = []
        self._run_caches: List[Tuple[List[int], bool]] = []       # per run: (cache numbers, may write them)
        for run, i in enumerate(self.spec.schedule):
            layer = self.spec.layers[i]
            if layer.cache_of is None:
                specs = list(self.blocks[i].cache_specs())
                self._run_caches.append((list(range(len(out), len(out) + len(specs))), True))
                out.extend(specs)
                continue
            src = next((r for r in range(run - 1, -1, -1) if self.spec.schedule[r] == layer.cache_of), None)
            if src is None:
                raise ValueError(f"run {run}: layer {layer.cache_of}, whose cache it reads, has not run before it")
            ids = self._run_caches[src][0]
            if len(ids) != len(self.blocks[i].cache_specs()):
                raise ValueError(f"layer {i} reads the caches of layer {layer.cache_of}, which keeps {len(ids)}; "
                                 f"its own parts want {len(self.blocks[i].cache_specs())}")
            self._run_caches.append((ids, False))
        return out

    def prepare(self, max_seq_tokens: int) -> None:
        for block in self.blocks:
            block.prepare(max_seq_tokens)

    def layer_caches(self, run: int, cache: SequenceCache, step) -> list:
        """What the parts of a run see of the cache: one `KVLayerCache` or `StateLayerCache` per entry of
        the arrangement's `cache_specs()`, in that order."""
        ids, writable = self._run_caches[run]
        out = []
        for c in ids:
            if c in cache.layer_group:
                gi = cache.layer_group[c]
                g = cache.kv_groups[gi]
                o = g.ordinal(c)
                out.append(KVLayerCache(g.k[o], g.v[o], step.block_tables[gi], g.spec.window, writable))
            else:
                out.append(StateLayerCache(cache.state[c], writable))
        return out

    # ---------------------------------------------------------------- forward
    def forward(self, step, cache: SequenceCache) -> Optional[torch.Tensor]:
        """Run the step's tokens through the scheduled layers; returns fp32 logits
        [wanted rows, vocab] (None if no row is wanted)."""
        stream = ResidualStream(self.embedding.forward(step))
        hook = self.layer_hook
        last = len(self.spec.schedule) - 1
        for run, i in enumerate(self.spec.schedule):
            if hook is not None:
                hook(run, i, False)
            block = self.blocks[i]
            # Nothing but the final norm reads what the last layer leaves, and that at the wanted rows only: a layer
            # that can narrows the stream to them once its mixer is through (a prompt's feed-forward then runs on
            # its last row alone).  Worth it where few of the step's rows are wanted.
            if run == last and getattr(block, "narrows_rows", False) and 4 * step.n_want <= step.n_tokens:
                keep = step.want_rows if step.n_want > 0 else torch.empty(0, dtype=torch.int32, device=stream.x.device)
                block.forward(stream, step, self.layer_caches(run, cache, step), keep_rows=keep)
            else:
                block.forward(stream, step, self.layer_caches(run, cache, step))
            if hook is not None:
                hook(run, i, True)
        if step.n_want == 0:
            # the last delta need not be added: nothing reads the stream after it
            return None
        h = self.final_norm.forward(stream, rows=None if stream.narrowed else step.want_rows)
        return self.head.forward(h)
