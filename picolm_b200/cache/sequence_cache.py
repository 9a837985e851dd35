"""The cache of a run: a slot for each live sequence, keys and values for each
layer in pages of `PAGE_TOKENS` positions, each sequence with its own length, and
beside it per-sequence state of fixed size.

Storage.  Layers whose mixers ask for the same `CacheSpec` form a group with
storage of its own: a kv group owns `k`/`v` tensors
`[layers_in_group, pages, kv_heads, PAGE_TOKENS, head_dim]` and one page list per
slot (all layers of the group use the same page numbers); a group with a window
gives pages back as soon as every position on them has left the window.  A state
layer owns a tensor `[slots + 1, *shape]`, a slot's row zeroed when the slot is
handed out.  Page 0 of every kv group is never handed out, and neither is the last
row of a state tensor (`null_slot`): the padding rows of a captured step point at them.

The reference has one sequence per model: one K block and one V block
`[kv_layers][max_seq_len][kv_heads*head_dim]` and a position counter held by the
caller (picolm/model_core.c:590-606, picolm/model_core.c:734-739), with no bound
check on the position (picolm/picolm.c:1496-1500).  Slots, pages and the bound
check are this library's.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .allocator import CacheFull, IndexPool
from .spec import CacheSpec

PAGE_TOKENS = 64

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class KVGroup:
    spec: CacheSpec
    layers: List[int]                           # runs of the schedule that own a layer of this storage, in order
    pool: IndexPool
    pages: Dict[int, List[int]] = field(default_factory=dict)     # slot -> page of each 64-position block (0: none)
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    table: Optional[np.ndarray] = None          # int32 [slots, pages per sequence]: `pages` as rows, 0-padded

    def ordinal(self, layer: int) -> int:
        return self.layers.index(layer)


@dataclass
class KVLayerCache:
    """What a mixer sees of a kv group for one step."""
    k: torch.Tensor                             # [pages, G, PAGE_TOKENS, hd]
    v: torch.Tensor
    block_table: torch.Tensor                   # int32 [seqs of the step, pages per sequence]
    window: Optional[int]
    writable: bool                              # False: the layer reads another layer's cache


@dataclass
class StateLayerCache:
    """What a mixer sees of its fixed-size state: `state[slot]` for each slot."""
    state: torch.Tensor                         # [slots + 1, *shape]; the last row belongs to padding rows
    writable: bool = True


class SequenceCache:
    def __init__(self, layer_specs: Sequence[Optional[CacheSpec]], max_tokens: int, max_seqs: int,
                 kv_dtype: torch.dtype = torch.bfloat16, device="cpu", max_seq_tokens: Optional[int] = None,
                 allocate_storage: bool = True):
        """`layer_specs[i]` is what cache number i holds (None: nothing): the model numbers
        what the runs of its schedule keep, a Llama layer's keys and values being one
        such cache per run.  The indices used throughout this class are those numbers.
        `max_tokens` is the most tokens live sequences hold together, each
        sequence's count rounded up to a page; `max_seqs` the most live
        sequences; `max_seq_tokens` the longest single sequence."""
        if max_tokens <= 0 or max_seqs <= 0:
            raise ValueError("max_tokens and max_seqs must be positive")
        self.max_tokens = pages_for(max_tokens) * PAGE_TOKENS
        self.max_seqs = max_seqs
        self.max_seq_tokens = min(max_seq_tokens or self.max_tokens, self.max_tokens)
        self.pages_per_seq = pages_for(self.max_seq_tokens)
        self.device = torch.device(device)
        self.kv_dtype = kv_dtype
        self.slots = IndexPool(max_seqs, what="slot")
        self.null_slot = max_seqs                      # the state row of a step's padding sequences
        self.lengths: Dict[int, int] = {}
        self.kv_groups: List[KVGroup] = []
        self.layer_group: Dict[int, int] = {}          # layer -> kv group index
        self.state: Dict[int, torch.Tensor] = {}       # layer -> [slots, *shape]
        self.state_specs: Dict[int, CacheSpec] = {}
        n_pages = self.max_tokens // PAGE_TOKENS
        by_key: Dict[tuple, int] = {}
        for layer, spec in enumerate(layer_specs):
            if spec is None:
                continue
            if spec.kind == "kv":
                gi = by_key.get(spec.group_key())
                if gi is None:
                    gi = len(self.kv_groups)
                    by_key[spec.group_key()] = gi
                    self.kv_groups.append(KVGroup(spec, [], IndexPool(n_pages, first=1, what="page")))
                self.kv_groups[gi].layers.append(layer)
                self.layer_group[layer] = gi
            elif spec.kind == "state":
                self.state_specs[layer] = spec
            else:
                raise ValueError(f"layer {layer}: unknown cache kind {spec.kind!r}")
        for g in self.kv_groups:
            g.table = np.zeros((max_seqs, self.pages_per_seq), dtype=np.int32)
        if allocate_storage:
            for g in self.kv_groups:
                shape = (len(g.layers), n_pages + 1, g.spec.num_kv_heads, PAGE_TOKENS, g.spec.head_dim)
                g.k = torch.zeros(shape, dtype=kv_dtype, device=self.device)
                g.v = torch.zeros(shape, dtype=kv_dtype, device=self.device)
            for layer, spec in self.state_specs.items():
                self.state[layer] = torch.zeros((max_seqs + 1,) + spec.shape, dtype=_STATE_DTYPES[spec.dtype],
                                                device=self.device)

    # ------------------------------------------------------------------ slots
    def allocate(self) -> int:
        """A free slot for a new sequence, its length 0 and its state zeroed."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.kv_groups:
            g.pages[slot] = []
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """Give back a slot and every page it holds."""
        if not self.slots.holds(slot):
            self.slots.give_back(slot)              # raises with the reason
        for g in self.kv_groups:
            for p in g.pages.pop(slot):
                if p:
                    g.pool.give_back(p)
            g.table[slot, :] = 0
        del self.lengths[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ------------------------------------------------------------------ pages
    def _new_pages_needed(self, g: KVGroup, slot: int, n_new: int) -> int:
        return max(0, pages_for(self.lengths[slot] + n_new) - len(g.pages[slot]))

    def reserve(self, requests: Sequence[tuple]) -> None:
        """Make room for `(slot, n_new)` of every sequence of a step, or raise
        `CacheFull` and change nothing."""
        seen = set()
        for slot, n_new in requests:
            if not self.slots.holds(slot):
                raise RuntimeError(f"slot {slot} is not in use")
            if slot in seen:
                raise RuntimeError(f"slot {slot} occurs twice in one step")
            seen.add(slot)
            if n_new <= 0:
                raise ValueError("a sequence must bring at least one token")
            if self.lengths[slot] + n_new > self.max_seq_tokens:
                raise CacheFull(
                    f"slot {slot}: {self.lengths[slot]} + {n_new} tokens exceed the longest sequence the cache "
                    f"was sized for ({self.max_seq_tokens})")
        for g in self.kv_groups:
            need = sum(self._new_pages_needed(g, s, n) for s, n in requests)
            if need > g.pool.free:
                raise CacheFull(
                    f"the cache needs {need} more pages of {PAGE_TOKENS} tokens and has {g.pool.free} free "
                    f"(sized for {self.max_tokens} tokens)")
        for g in self.kv_groups:
            for s, n in requests:
                for _ in range(self._new_pages_needed(g, s, n)):
                    page = g.pool.take()
                    g.table[s, len(g.pages[s])] = page
                    g.pages[s].append(page)

    def advance(self, slot: int, n_new: int) -> None:
        """The step wrote `n_new` positions of `slot`.  Pages of windowed groups
        whose every position has left the window go back to the pool."""
        self.lengths[slot] += n_new
        new_len = self.lengths[slot]
        for g in self.kv_groups:
            w = g.spec.window
            if w is None:
                continue
            first_needed = max(0, new_len - w + 1)      # the next query (position new_len) reads from here
            pages = g.pages[slot]
            for b in range(min(first_needed // PAGE_TOKENS, len(pages))):
                if pages[b]:
                    g.pool.give_back(pages[b])
                    pages[b] = 0
                    g.table[slot, b] = 0

    def block_table_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        """int32 [len(slots), pages per sequence]: the page of every 64-position block of each slot (0: none)."""
        return self.kv_groups[group].table[np.asarray(slots, dtype=np.int64)]

    # ------------------------------------------------------------- accounting
    def check(self) -> None:
        """No slot or page lost, held twice, or held by a slot that is free."""
        self.slots.check()
        if set(self.lengths) != self.slots._used:
            raise AssertionError("lengths are kept for slots that are not in use")
        for g in self.kv_groups:
            g.pool.check()
            held = [p for pages in g.pages.values() for p in pages if p]
            if len(held) != len(set(held)):
                raise AssertionError("a page is held by two sequences")
            if set(held) != g.pool._used:
                raise AssertionError("pages in use and pages held by sequences differ")
            if set(g.pages) != self.slots._used:
                raise AssertionError("page lists are kept for slots that are not in use")
            for s in range(self.max_seqs):
                want = g.pages.get(s, [])
                row = g.table[s]
                if list(row[:len(want)]) != list(want) or row[len(want):].any():
                    raise AssertionError(f"the page table row of slot {s} differs from its page list")

    def kv_bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.kv_dtype).element_size()
        return sum(2 * len(g.layers) * g.spec.num_kv_heads * g.spec.head_dim * item for g in self.kv_groups)
