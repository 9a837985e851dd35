"""The description of one step for the device: which tokens run, to which
sequence and position each belongs, where each sequence's pages are, and which
rows' logits are wanted.  Built on the host, sent to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepBatch:
    n_seqs: int
    n_tokens: int
    n_want: int
    # The three host lists are None in a step that is replayed from a captured graph: the graph
    # serves every batch of its size, so only what lives in device buffers may be read there
    # (`seq_slot`, `tok_pos`, `seq_kv_len`, ...).
    slots: Optional[List[int]]            # host: cache slot of each sequence
    new_lens: Optional[List[int]]         # host: tokens each sequence brings
    start_pos: Optional[List[int]]        # host: position of each sequence's first new token
    max_position: int                     # host: largest position written by this step
    max_new: int                          # host: the most tokens a sequence brings (an upper bound in a captured step)
    is_decode: bool                       # every sequence brings exactly one token
    tok_ids: torch.Tensor                 # int32 [T]
    tok_seq: torch.Tensor                 # int32 [T]  index of the token's sequence within the step
    tok_pos: torch.Tensor                 # int32 [T]  absolute position
    seq_slot: torch.Tensor                # int32 [B]
    seq_start: torch.Tensor               # int32 [B+1] offsets of each sequence's tokens
    seq_kv_len: torch.Tensor              # int32 [B]  length after this step
    want_rows: torch.Tensor               # int32 [n_want] flat token indices
    block_tables: List[torch.Tensor]      # per kv group: int32 [B, pages per sequence]
    h2d_bytes: int = 0                    # size of the one host-to-device copy that brought all of the above
    _seq_slot_long: Optional[torch.Tensor] = None

    @property
    def seq_slot_long(self) -> torch.Tensor:
        """`seq_slot` as int64 [B], for indexing state tensors with torch.  Made from the device buffer when
        first asked for, on the current stream: inside a graph capture the conversion is part of the graph and
        follows the buffer on every replay."""
        if self._seq_slot_long is None:
            self._seq_slot_long = self.seq_slot.to(torch.int64)
        return self._seq_slot_long


def build_step_batch(entries: Sequence[tuple], wants: Sequence[Sequence[int]], cache, device) -> StepBatch:
    """`entries`: (slot, token list) per sequence, positions continuing from the
    cache's lengths; `wants`: per sequence the indices among its new tokens whose
    logits are wanted.  Pages must already be reserved."""
    B = len(entries)
    new_lens = [len(toks) for _, toks in entries]
    slots = [s for s, _ in entries]
    start = [cache.length(s) for s in slots]
    T = sum(new_lens)
    P = cache.pages_per_seq
    n_groups = len(cache.kv_groups)
    want_flat: List[int] = []
    offs = [0]
    for n in new_lens:
        offs.append(offs[-1] + n)
    for b, w in enumerate(wants):
        for i in w:
            if not 0 <= i < new_lens[b]:
                raise IndexError(f"sequence {b}: wanted place {i} is not among its {new_lens[b]} tokens")
            want_flat.append(offs[b] + i)
    W = len(want_flat)
    sizes = [T, T, T, B, B + 1, B, W] + [B * P] * n_groups
    total = sum(sizes)
    host = np.zeros(total, dtype=np.int32)
    o = 0
    views = []
    for n in sizes:
        views.append(host[o:o + n])
        o += n
    tok_ids, tok_seq, tok_pos, seq_slot, seq_start, seq_kv_len, want_rows = views[:7]
    for b, (slot, toks) in enumerate(entries):
        a, e = offs[b], offs[b + 1]
        tok_ids[a:e] = toks
        tok_seq[a:e] = b
        tok_pos[a:e] = np.arange(start[b], start[b] + new_lens[b], dtype=np.int32)
        seq_kv_len[b] = start[b] + new_lens[b]
    seq_slot[:] = slots
    seq_start[:] = offs
    want_rows[:] = want_flat
    for gi in range(n_groups):
        views[7 + gi].reshape(B, P)[:] = cache.block_table_rows(gi, slots)
    pinned = torch.from_numpy(host)
    if torch.device(device).type == "cuda":
        pinned = pinned.pin_memory()
    dev = pinned.to(device, non_blocking=True)
    o = 0
    dviews = []
    for n in sizes:
        dviews.append(dev[o:o + n])
        o += n
    return StepBatch(
        n_seqs=B, n_tokens=T, n_want=W, slots=slots, new_lens=new_lens, start_pos=start,
        max_position=max(s + n for s, n in zip(start, new_lens)) - 1, max_new=max(new_lens),
        is_decode=all(n == 1 for n in new_lens),
        tok_ids=dviews[0], tok_seq=dviews[1], tok_pos=dviews[2], seq_slot=dviews[3], seq_start=dviews[4],
        seq_kv_len=dviews[5], want_rows=dviews[6],
        block_tables=[dviews[7 + gi].view(B, P) for gi in range(n_groups)],
        h2d_bytes=int(host.nbytes),
    )
