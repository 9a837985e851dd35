"""A step with prompts as a CUDA graph: for a padded number of tokens and of sequences the kernels of one
step are captured once and replayed, as `decode_graph` does for steps of one token each.  A prompt of a few
hundred tokens is launched as about 130 kernels; from Python that takes longer than the kernels run, from a
graph it is one launch.

The graph runs the same `Model.forward` on the same parts and kernels as a step launched kernel by kernel.
Tokens are padded to the next size class: padding tokens belong to a sequence of their own whose page table
points at the cache's null page and whose state row is the null slot, so that what is written for them lands
where nothing reads it; no sequence of the step covers them (`seq_start` ends before them), so attention
skips them, and every other kernel works row by row, so whatever their rows hold stays in their rows.
Sequences are padded with sequences of no tokens.  Logits are computed for the last token of every sequence.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .step_batch import StepBatch

# padded token counts: steps of 64 up to 512, of 128 up to 1,024, of 256 up to 2,048
TOKEN_CLASSES = tuple(range(64, 513, 64)) + tuple(range(640, 1025, 128)) + tuple(range(1280, 2049, 256))
SEQ_CLASSES = (1, 2, 4, 8, 16, 32, 64)      # real sequences a graph serves (one more row is the padding sequence)


def token_class(n: int) -> Optional[int]:
    for t in TOKEN_CLASSES:
        if n <= t:
            return t
    return None


def seq_class(n: int) -> Optional[int]:
    for b in SEQ_CLASSES:
        if n <= b:
            return b
    return None


class PromptGraph:
    def __init__(self, engine, tokens: int, seqs: int):
        self.engine = engine
        self.T, self.n_real = tokens, seqs
        self.B = B = seqs + 1                               # the last sequence takes the padding tokens' writes
        cache = engine.cache
        dev = engine.runtime.device
        T, P, n_groups = tokens, cache.pages_per_seq, len(cache.kv_groups)
        # layout: tok_ids, tok_seq, tok_pos, seq_slot, seq_start, seq_kv_len, want_rows, block tables
        self.sizes = [T, T, T, B, B + 1, B, B] + [B * P] * n_groups
        total = sum(self.sizes)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.h, self.d = [], []
        o = 0
        for n in self.sizes:
            self.h.append(self.host_np[o:o + n])
            self.d.append(self.dev[o:o + n])
            o += n
        self.tables_h = [self.h[7 + g].reshape(B, P) for g in range(n_groups)]
        self.step = StepBatch(
            n_seqs=B, n_tokens=T, n_want=B, slots=None, new_lens=None, start_pos=None,
            max_position=cache.max_seq_tokens - 1, max_new=T, is_decode=False,
            tok_ids=self.d[0], tok_seq=self.d[1], tok_pos=self.d[2], seq_slot=self.d[3], seq_start=self.d[4],
            seq_kv_len=self.d[5], want_rows=self.d[6],
            block_tables=[self.d[7 + g].view(B, P) for g in range(n_groups)], h2d_bytes=int(self.host_np.nbytes))
        self.copied = torch.cuda.Event()
        self.replayed: Optional[torch.cuda.Event] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0

    def _fill(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> None:
        cache = self.engine.cache
        h, T, B = self.h, self.T, self.B
        n = len(entries)
        self.copied.synchronize()                           # do not overwrite what a pending copy still reads
        o = 0
        for b, (slot, toks) in enumerate(entries):
            m, start = len(toks), cache.length(slot)
            h[0][o:o + m] = toks
            h[1][o:o + m] = b
            h[2][o:o + m] = np.arange(start, start + m, dtype=np.int32)
            h[3][b] = slot
            h[4][b] = o
            h[5][b] = start + m
            h[6][b] = o + m - 1                              # the last token's logits
            o += m
        pad = B - 1                                         # the padding sequence: no tokens of its own in seq_start
        h[0][o:] = 0
        h[1][o:] = pad
        h[2][o:] = np.arange(T - o, dtype=np.int32) % 64    # (all on the null page, whatever the position)
        h[3][n:] = cache.null_slot
        h[4][n:] = o
        h[5][n:] = 0
        h[6][n:] = 0
        slots = [s for s, _ in entries]
        for g, table in enumerate(self.tables_h):
            table[:n] = cache.block_table_rows(g, slots)
            table[n:] = 0
        cur = torch.cuda.current_stream(self.dev.device)
        side = self.engine.side_stream("h2d")
        if self.replayed is not None:
            side.wait_event(self.replayed)
        with torch.cuda.stream(side):
            self.dev.copy_(self.host, non_blocking=True)
            self.copied.record(side)
        cur.wait_event(self.copied)

    def _mark_replayed(self) -> None:
        if self.replayed is None:
            self.replayed = torch.cuda.Event()
        self.replayed.record(torch.cuda.current_stream(self.dev.device))

    def capture(self) -> None:
        import gc
        from .. import ops
        eng = self.engine
        self._fill([])                                      # every token a padding token: touches the null page only
        with ops.stream_scope():
            eng.model.forward(self.step, eng.cache)         # first-call set-up of every kernel, allocator warm-up
        self._mark_replayed()
        torch.cuda.synchronize()
        self.step._seq_slot_long = None
        n0 = ops.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()                                        # nothing may be freed while the stream is capturing
        try:
            with torch.cuda.graph(self.graph), ops.stream_scope():
                self.logits = eng.model.forward(self.step, eng.cache)
        finally:
            if was_enabled:
                gc.enable()
        self.launches = ops.launch_count() - n0
        ops.count_launches(-self.launches)

    def run(self, entries: Sequence[Tuple[int, Sequence[int]]]) -> torch.Tensor:
        """Replay for `entries` (slot, tokens); returns the logits of every sequence's last token
        [len(entries), vocab], valid until the next replay of this graph."""
        from .. import ops
        self._fill(entries)
        self.graph.replay()
        self._mark_replayed()
        ops.count_launches(self.launches)
        return self.logits[:len(entries)]
