"""The engine: a model, its cache, and the one step function that both
generation and trace replay drive.

`step` runs exactly the tokens it is given, as one batch, against what earlier
steps left in the cache, and returns the logits at the wanted places.  A batch's
sequences start together with their whole prompts (unequal lengths) in one step
and then go on by one token each; sequences that have ended are simply no longer
in the entries.  The reference's two entry points are the single-sequence cases
of it: `model_forward(token, pos)` (picolm/model_core.c:1682) and
`model_forward_prefill(tokens, n, start_pos)` (picolm/model_core.c:2671).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .. import architectures  # noqa: F401  (registers the known architectures)
from ..cache import SequenceCache
from ..config.registry import read_config, spec_of
from ..runtime import Runtime
from ..weights.loader import load_weights
from .model import Model
from .step_batch import build_step_batch


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 max_seq_tokens: Optional[int] = None, use_graphs: Optional[bool] = None):
        """`max_tokens`: the most tokens that live sequences hold at any time, each
        sequence's count rounded up to a multiple of the page size.  `max_seqs`:
        the most sequences alive at once (default: one per page).
        `max_seq_tokens`: the longest single sequence (default: the model's
        position limit, or the whole cache if that is smaller)."""
        if not model.loaded:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.runtime = model.runtime
        spec = model.spec
        longest = min(max_seq_tokens or spec.max_positions, spec.max_positions)
        self.cache = SequenceCache(model.cache_specs(), max_tokens=max_tokens,
                                   max_seqs=max_seqs or max(1, (max_tokens + 63) // 64),
                                   kv_dtype=self.runtime.dtype, device=self.runtime.device,
                                   max_seq_tokens=longest)
        model.prepare(self.cache.max_seq_tokens)
        self.vocab_size = spec.vocab_size
        # Decode steps replay a CUDA graph when every part of every block says that its forward only
        # launches work that depends on the step through device buffers (`graph_safe`).
        safe = all(getattr(part, "graph_safe", False) for b in model.blocks for _, part in b.parts())
        self.use_graphs = safe if use_graphs is None else (use_graphs and safe)
        from ..ops import _lib
        if _lib.CHECKED or _lib.TRACED:
            # the checked build hands its kernels their bounds by a copy before every launch; the per-kernel
            # table needs every launch between two events
            self.use_graphs = False
        self._graphs: Dict[Tuple[int, int], "DecodeGraph"] = {}
        self._prompt_graphs: Dict[Tuple[int, int], "PromptGraph"] = {}
        # steps with prompts replay a graph too where every sequence wants its last token's logits (generation);
        # float32 runs launch them kernel by kernel (their kernels take longer than the launches)
        import os
        self.prompt_graphs = (os.environ.get("PICOLM_B200_PROMPT_GRAPHS", "1") != "0" and self.runtime.dtype == torch.bfloat16 and
                              all(getattr(part, "graph_safe_prompts", False) for b in model.blocks for _, part in b.parts()))
        # one id per live sequence, and never fewer than the largest captured batch size (its padding rows read it)
        from .decode_graph import BUCKETS
        self._tokens = torch.zeros(max(BUCKETS[-1], self.cache.max_seqs), dtype=torch.int32,
                                   device=self.runtime.device)
        self._side_streams: Dict[str, torch.cuda.Stream] = {}
        self._fetched: Optional[torch.cuda.Event] = None      # the last copy of sampled ids to the host
        self.reset_counters()

    def token_buffer(self, n: int) -> torch.Tensor:
        """The first `n` entries of the buffer from which captured decode steps read their token ids.  A
        sampler that writes its result here (`out=`) saves `step_device_tokens` a copy.  The buffer holds one
        id per sequence the cache can hold; more are refused."""
        if not 0 < n <= self._tokens.numel():
            raise ValueError(f"{n} token ids asked for; the engine holds at most {self._tokens.numel()} sequences")
        return self._tokens[:n]

    def before_token_write(self) -> None:
        """Called by whatever is about to write the token buffer on the current stream: that write has to
        wait until the last copy of sampled ids to the host (`fetch_later`) has read the buffer."""
        if self._fetched is not None:
            torch.cuda.current_stream(self.runtime.device).wait_event(self._fetched)
            self._fetched = None

    def reset_counters(self) -> None:
        """Bytes copied between host and device by the steps since the last reset."""
        self.counters = {"steps": 0, "h2d_bytes": 0, "d2h_bytes": 0}

    def to_host(self, tokens: torch.Tensor):
        """Sampled token ids as a host list (one device-to-host copy)."""
        self.counters["d2h_bytes"] += tokens.numel() * tokens.element_size()
        return tokens.tolist()

    def pinned_tokens(self, rows: int, cols: int) -> torch.Tensor:
        """A [rows, cols] int32 view of pinned host memory for `fetch_later` (allocated once and kept:
        pinning memory is slow)."""
        need = rows * cols
        buf = getattr(self, "_pinned", None)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 64 * 64), dtype=torch.int32)
            if self.runtime.device.type == "cuda":
                buf = buf.pin_memory()
            self._pinned = buf
        return buf[:need].view(rows, cols)

    def mark(self) -> torch.cuda.Event:
        """An event after everything launched so far on the current stream."""
        e = torch.cuda.Event()
        e.record()
        return e

    def side_stream(self, name: str) -> torch.cuda.Stream:
        """One of the engine's streams beside the one that runs the steps: "h2d" carries a captured step's
        metadata to the device, "d2h" carries sampled ids to the host, so that neither copy stands between two
        steps on the stream that computes."""
        if name not in self._side_streams:
            self._side_streams[name] = torch.cuda.Stream(self.runtime.device)
        return self._side_streams[name]

    def fetch_later(self, tokens: torch.Tensor, pinned_row: torch.Tensor) -> torch.cuda.Event:
        """Start copying sampled token ids into a row of pinned host memory without waiting for them.  The copy
        runs on a stream of its own once the ids are there; the event that is returned says when they have
        reached the host.  Whatever is launched after the engine's next step waits for the copy (a sampler may
        then write the same buffer again); the step itself does not."""
        cur = torch.cuda.current_stream(self.runtime.device)
        side = self.side_stream("d2h")
        ready = torch.cuda.Event()
        ready.record(cur)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            pinned_row.copy_(tokens, non_blocking=True)
            done = torch.cuda.Event()
            done.record(side)
        tokens.record_stream(side)
        self._fetched = done
        self.counters["d2h_bytes"] += tokens.numel() * tokens.element_size()
        return done

    # ----------------------------------------------------------- construction
    @staticmethod
    def from_folder(model_dir: str, dtype="bfloat16", max_tokens: int = 4096, max_seqs: Optional[int] = None,
                    max_seq_tokens: Optional[int] = None, device="cuda:0",
                    use_graphs: Optional[bool] = None) -> "Engine":
        """Load `model_dir` (config.json + safetensors); the model class is chosen
        by config.json's `architectures` through the registry."""
        runtime = Runtime.create(dtype, device)
        config = read_config(model_dir)
        model = Model(spec_of(config), runtime)
        load_weights(model, model_dir)
        eng = Engine(model, max_tokens, max_seqs, max_seq_tokens, use_graphs=use_graphs)
        eng.config = config
        return eng

    # -------------------------------------------------------------- sequences
    def new_sequence(self) -> int:
        """A cache slot for a sequence that starts now."""
        return self.cache.allocate()

    def end_sequence(self, slot: int) -> None:
        """Give back the slot and everything it holds."""
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.runtime.device)

    # ------------------------------------------------------------------- step
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             wants: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step.  `entries`: for each sequence its slot and its next
        tokens.  `wants`: for each sequence the places among these tokens whose
        logits are wanted (default: the last one).  Returns fp32 logits
        [wanted places, vocab] on the device, in the order of the entries and of
        `wants`, or None if nothing is wanted."""
        if not entries:
            return None
        if wants is None:
            wants = [[len(toks) - 1] for _, toks in entries]
        if len(wants) != len(entries):
            raise ValueError("wants must have one list per entry")
        for slot, toks in entries:
            if len(toks) == 0:
                raise ValueError(f"slot {slot}: a sequence must bring at least one token")
            lo, hi = min(toks), max(toks)
            if lo < 0 or hi >= self.vocab_size:
                raise ValueError(f"slot {slot}: token id {lo if lo < 0 else hi} is outside the vocabulary "
                                 f"[0, {self.vocab_size})")
        return self._run(entries, wants, None)

    def step_device_tokens(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One more token for each of the sequences in `slots`, the tokens taken from an int32 tensor
        on the device (what the sampler wrote for the step before): the same step as
        `step([(slot, [token]), ...])`, but the host need not know the tokens to launch it, so it can
        prepare and launch steps while earlier ones still run.  The token ids must lie inside the
        vocabulary (the sampling kernels' results do).  Returns the logits of every sequence."""
        if not slots:
            raise ValueError("no sequences")
        if tokens.dtype != torch.int32 or not tokens.is_cuda or tokens.numel() != len(slots):
            raise ValueError("tokens must be an int32 tensor on the device, one per sequence")
        return self._run([(slot, [0]) for slot in slots], [[0]] * len(slots), tokens)

    def _run(self, entries, wants, device_tokens: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        self.cache.reserve([(slot, len(toks)) for slot, toks in entries])
        logits = None
        graphed = False
        if self.use_graphs and self.model.layer_hook is None and all(len(toks) == 1 for _, toks in entries):
            logits, graphed = self._decode_with_graph(entries, wants, device_tokens)
        elif self.use_graphs and self.prompt_graphs and self.model.layer_hook is None and device_tokens is None:
            logits, graphed = self._prompts_with_graph(entries, wants)
        if not graphed:
            batch = build_step_batch(entries, wants, self.cache, self.runtime.device)
            self.counters["h2d_bytes"] += batch.h2d_bytes
            if device_tokens is not None:
                batch.tok_ids.copy_(device_tokens)
            from .. import ops
            with ops.stream_scope():
                logits = self.model.forward(batch, self.cache)
        self.before_token_write()                            # what follows this step may write the ids' buffer
        self.counters["steps"] += 1
        for slot, toks in entries:
            self.cache.advance(slot, len(toks))
        return logits

    def _prompts_with_graph(self, entries, wants) -> Tuple[Optional[torch.Tensor], bool]:
        """A step with prompts through the captured graph of its size class.  Returns the logits (None if none are
        wanted) and whether a graph ran: it does not if the step is too large or logits are wanted at other
        places than every sequence's last token."""
        from .prompt_graph import PromptGraph, seq_class, token_class
        n = len(entries)
        n_tokens = sum(len(toks) for _, toks in entries)
        key = (token_class(n_tokens), seq_class(n))
        if key[0] is None or key[1] is None:
            return None, False
        n_want = sum(len(w) for w in wants)
        if n_want not in (0, n) or (n_want and any(list(w) != [len(toks) - 1] for w, (_, toks) in zip(wants, entries))):
            return None, False
        g = self._prompt_graphs.get(key)
        if g is None:
            g = PromptGraph(self, key[0], key[1])
            g.capture()
            self._prompt_graphs[key] = g
        logits = g.run(entries)
        self.counters["h2d_bytes"] += g.step.h2d_bytes
        return (logits if n_want else None), True

    def _decode_with_graph(self, entries, wants, device_tokens=None) -> Tuple[Optional[torch.Tensor], bool]:
        """One token for each sequence through the captured graph of the batch's size class.  Returns the
        logits (None if none are wanted) and whether a graph ran: it does not if the batch is too large
        or places are wanted that are not exactly [0]."""
        from .decode_graph import DecodeGraph, bucket_for, length_class
        n = len(entries)
        bucket = bucket_for(n)
        if bucket is None:
            return None, False
        n_want = sum(len(w) for w in wants)
        if n_want not in (0, n) or any(list(w) not in ([], [0]) for w in wants):
            return None, False
        slots = [s for s, _ in entries]
        positions = [self.cache.length(s) for s in slots]
        key = (bucket, length_class(max(positions) + 1, self.cache.max_seq_tokens))
        g = self._graphs.get(key)
        if g is None:
            g = DecodeGraph(self, key[0], key[1])
            g.capture()
            self._graphs[key] = g
        logits = g.run(slots, [t[0] for _, t in entries], positions, device_tokens)
        self.counters["h2d_bytes"] += g.step.h2d_bytes
        return (logits if n_want else None), True
