"""A decode step as a CUDA graph: for a fixed (padded) batch size the kernels
of one step are captured once and replayed, so that a step costs one metadata
copy and one graph launch instead of a launch per kernel from Python.

The graph runs the same `Model.forward` on the same parts and kernels as an
ordinary step; only the step's metadata lives in fixed device buffers that are
refilled before every replay.  Batches are padded to the next size that has a
graph; padding rows are single tokens of an empty sequence whose block table
points at the cache's null page, so they read and write nothing that a real
sequence sees, and their logits are dropped.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .step_batch import StepBatch

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def bucket_for(n: int) -> Optional[int]:
    for b in BUCKETS:
        if n <= b:
            return b
    return None


LENGTH_QUANTUM = 512          # sequence lengths are rounded up for the sizes a graph bakes in: to this ...


def length_class(max_len: int, longest: int) -> int:
    """The length a graph is captured for: kernels that size their grids by the longest sequence
    (how many ranges the decode attention cuts the keys into) get this instead of the true length,
    so that a graph serves all steps until the batch's longest sequence grows past it.  Steps of 512
    up to 2,048, then of a quarter of the next power of two (1,024 up to 4,096, 2,048 up to 8,192, ...):
    less than half the true length above it (beyond the first steps of 512), and a few dozen classes for any context."""
    q = LENGTH_QUANTUM
    while q * 4 < max_len:
        q *= 2
    return min(longest, (max_len + q - 1) // q * q)


class DecodeGraph:
    def __init__(self, engine, batch: int, max_len: int):
        self.engine = engine
        self.batch = B = batch
        cache = engine.cache
        dev = engine.runtime.device
        P = cache.pages_per_seq
        n_groups = len(cache.kv_groups)
        # layout: tok_ids, tok_seq, tok_pos, seq_slot, seq_start, seq_kv_len, want_rows, block tables.
        # On the device the token ids live in the engine's one token buffer instead (all graphs read
        # it, and a sampler may write the next step's ids straight into it).
        self.sizes = [B, B, B, B, B + 1, B, B] + [B * P] * n_groups
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
        self.d[0] = engine.token_buffer(B)
        self.h[1][:] = np.arange(B)                       # tok_seq: one token per sequence
        self.h[4][:] = np.arange(B + 1)                   # seq_start
        self.h[6][:] = np.arange(B)                       # want_rows: every row
        self.tables_h = [self.h[7 + g].reshape(B, P) for g in range(n_groups)]
        self.step = StepBatch(
            n_seqs=B, n_tokens=B, n_want=B, slots=None, new_lens=None, start_pos=None,
            max_position=max_len - 1,                     # the graph's length class (see length_class)
            max_new=1,
            is_decode=True, tok_ids=self.d[0], tok_seq=self.d[1], tok_pos=self.d[2], seq_slot=self.d[3],
            seq_start=self.d[4], seq_kv_len=self.d[5], want_rows=self.d[6],
            block_tables=[self.d[7 + g].view(B, P) for g in range(n_groups)],
            h2d_bytes=int(self.host_np.nbytes))
        self.copied = torch.cuda.Event()                  # the last metadata copy has left the pinned buffer
        self.replayed: Optional[torch.cuda.Event] = None  # the last run of the step has read the metadata
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0

    def _fill(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int],
              device_tokens: Optional[torch.Tensor] = None) -> None:
        n, B = len(slots), self.batch
        cache = self.engine.cache
        h = self.h
        self.copied.synchronize()                         # do not overwrite what a pending copy still reads
        h[0][:n] = tokens
        h[0][n:] = 0
        h[2][:n] = positions
        h[2][n:] = 0
        h[3][:n] = slots
        h[3][n:] = cache.null_slot                        # state of their own for the padding rows
        h[5][:n] = h[2][:n] + 1
        h[5][n:] = 1
        for g, table in enumerate(self.tables_h):
            table[:n] = cache.block_table_rows(g, slots)
            table[n:] = 0                                 # the null page
        # The copy runs on a stream of its own, as soon as the last replay has read the buffers it overwrites:
        # beside the sampling and the copy of the ids that follow that replay, not behind them.
        cur = torch.cuda.current_stream(self.dev.device)
        side = self.engine.side_stream("h2d")
        if self.replayed is not None:
            side.wait_event(self.replayed)
        with torch.cuda.stream(side):
            self.dev.copy_(self.host, non_blocking=True)
            self.copied.record(side)
        cur.wait_event(self.copied)
        if device_tokens is None:
            self.engine.before_token_write()              # a copy of the last ids to the host may still read it
            self.d[0].copy_(self.dev[:B])
        elif device_tokens.data_ptr() != self.d[0].data_ptr():
            # the token ids are on the device already; rows of padding keep whatever valid id they held
            self.engine.before_token_write()
            self.d[0][:n].copy_(device_tokens)

    def _mark_replayed(self) -> None:
        if self.replayed is None:
            self.replayed = torch.cuda.Event()
        self.replayed.record(torch.cuda.current_stream(self.dev.device))

    def capture(self) -> None:
        from .. import ops
        eng = self.engine
        # (the token buffer is shared with the steps around this capture and may hold the ids that the next
        # replay is to read: it is left as it is; whatever valid ids it holds serve the warm-up run)
        self._fill([], [], [], device_tokens=self.d[0])
        # once outside the capture: first-call set-up of every kernel, allocator warm-up
        with ops.stream_scope():
            eng.model.forward(self.step, eng.cache)
        self._mark_replayed()
        torch.cuda.synchronize()
        self.step._seq_slot_long = None                   # made again inside the capture, so that replays refresh it
        n0 = ops.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        # Nothing may be freed while the stream is capturing: collect what is dead now and keep the
        # collector off until the capture has ended (a dead engine's graphs and buffers would
        # otherwise be destroyed in the middle of it, which CUDA refuses).
        import gc
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph), ops.stream_scope():     # the capture has a stream of its own
                self.logits = eng.model.forward(self.step, eng.cache)
        finally:
            if was_enabled:
                gc.enable()
        self.launches = ops.launch_count() - n0
        ops.count_launches(-self.launches)                # the capture itself ran nothing

    def run(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int],
            device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Replay for `len(slots)` real sequences; returns logits [len(slots), vocab],
        valid until the next replay of this graph.  With `device_tokens` (int32 [len(slots)] on the
        device) the token ids come from there instead of `tokens`."""
        from .. import ops
        self._fill(slots, tokens, positions, device_tokens)
        self.graph.replay()
        self._mark_replayed()
        ops.count_launches(self.launches)
        return self.logits[:len(slots)]
