"""The generation loop above the step function: as many batches one after
another as there are requests; in a batch, prompts of unequal lengths in one
step, then one token for each sequence that is still alive.

The reference's loop is `prefill; loop { sample; stop on EOS; forward(next) }`
for one sequence (picolm/picolm.c:1502-1610).  Kept from it: the stop token is
part of the output and is not fed; generation stops at `max_tokens` new tokens or
when the context is full.  Not kept: it samples up to `max_tokens + 1` tokens and
may run one position past its cache (picolm/picolm.c:1496-1500, :1539).

The decisions (which requests form the next batch, when a sequence ends) are
plain functions of host values, so they can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache.sequence_cache import PAGE_TOKENS, pages_for
from ..sampling import Sampler, SamplingParams


@dataclass
class Request:
    index: int                       # position among the call's prompts
    prompt: List[int]
    max_new: int
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None       # "stop", "length", "context"


@dataclass
class GenerationStats:
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    generated_tokens: int = 0
    generation_seconds: float = 0.0
    batches: int = 0
    steps: int = 0


def tokens_reserved(prompt_len: int, max_new: int, max_seq_tokens: int) -> int:
    """Cache tokens a request may come to hold: its prompt and all but the last
    of its new tokens (the last is never fed), capped by the longest sequence,
    rounded up to whole pages."""
    return pages_for(min(prompt_len + max(max_new - 1, 0), max_seq_tokens)) * PAGE_TOKENS


def plan_batch(pending: Sequence[Request], free_tokens: int, free_slots: int, max_batch: int,
               max_seq_tokens: int) -> List[Request]:
    """The next batch: requests in their order, as many as fit the free slots,
    `max_batch` and the free cache (each counted with all it may come to hold).
    Raises if the first pending request can never fit."""
    batch: List[Request] = []
    used = 0
    for r in pending:
        if len(batch) >= min(max_batch, free_slots):
            break
        need = tokens_reserved(len(r.prompt), r.max_new, max_seq_tokens)
        if used + need > free_tokens:
            break
        batch.append(r)
        used += need
    if not batch and pending:
        r = pending[0]
        raise RuntimeError(
            f"request {r.index} (prompt of {len(r.prompt)} tokens, up to {r.max_new} new) does not fit the cache: "
            f"{free_tokens} tokens and {free_slots} slots are free")
    return batch


def finish_reason(token: int, n_generated: int, max_new: int, stop_ids, length_after_feed: int,
                  max_seq_tokens: int) -> Optional[str]:
    """Why a sequence ends after producing `token` as its `n_generated`-th new
    token, or None if it goes on.  `length_after_feed` is the length the
    sequence would have once this token were fed."""
    if token in stop_ids:
        return "stop"
    if n_generated >= max_new:
        return "length"
    if length_after_feed > max_seq_tokens:
        return "context"
    return None


def _to_host(engine, tokens):
    fetch = getattr(engine, "to_host", None)
    return fetch(tokens) if fetch is not None else tokens.tolist()


def _decode_ahead(engine, sampler, batch, slots, live, first_tokens, stop, on_token, stats, depth) -> None:
    """The decode loop of one batch with up to `depth` steps in flight: a step's sampled ids feed the next
    step on the device, the host looks at them `depth - 1` steps late (see `generate`).  `live`: indices
    into `batch` of the sequences that run; `first_tokens`: what the prompts' step sampled, on the host."""
    import collections
    import torch
    cache = engine.cache
    device = engine.runtime.device
    buffer = getattr(engine, "token_buffer", None)       # where the engine's captured steps read their ids
    mark = getattr(engine, "mark", None)                 # an event after what was launched so far
    n0 = len(live)
    pinned = engine.pinned_tokens(depth + 1, n0) if hasattr(engine, "pinned_tokens") else \
        torch.empty((depth + 1, n0), dtype=torch.int32)

    def judge(members, tokens, lengths_after_feed):
        """Append a step's tokens to the sequences that no earlier token has ended, and decide whether they end."""
        for i, tok, length in zip(members, tokens, lengths_after_feed):
            r = batch[i]
            if r.finish_reason is not None:              # ended by an earlier token: this one is surplus
                continue
            r.output.append(tok)
            stats.generated_tokens += 1
            if on_token is not None:
                on_token(r.index, tok)
            r.finish_reason = finish_reason(tok, len(r.output), r.max_new, stop, length, cache.max_seq_tokens)

    judge(live, [int(t) for t in first_tokens], [engine.length(slots[i]) + 1 for i in live])
    # what the host knows to be launched: per sequence the number of tokens sampled or being sampled
    launched = {i: len(batch[i].output) for i in live}
    cur = [i for i in live if batch[i].finish_reason is None]       # the sequences of the next step
    rows_of = list(live)                                             # whose ids the rows of tok_dev hold
    tok_dev = torch.tensor([int(t) for t in first_tokens], dtype=torch.int32, device=device)
    inflight = collections.deque()
    step_no = 0
    while True:
        while len(inflight) < depth:
            # a sequence runs another step unless a token ended it or its limits are reached by what is
            # already launched (those are known without looking at any token)
            cur = [i for i in cur if batch[i].finish_reason is None and launched[i] < batch[i].max_new
                   and engine.length(slots[i]) < cache.max_seq_tokens]
            if not cur:
                break
            if cur != rows_of:                           # some left: keep the others' rows, on the device
                keep = [rows_of.index(i) for i in cur]
                sampler.keep(keep)
                tok_dev = tok_dev[torch.tensor(keep, dtype=torch.int64, device=device)].contiguous()
                rows_of = list(cur)
            cur_slots = [slots[i] for i in cur]
            logits = engine.step_device_tokens(cur_slots, tok_dev)
            tok_dev = sampler.sample(logits, out=buffer(len(cur))) if buffer else sampler.sample(logits)
            row = pinned[step_no % (depth + 1), :len(cur)]
            fetched = engine.fetch_later(tok_dev, row)          # an event, if the engine has one for the copy
            if fetched is None and mark:
                fetched = mark()
            inflight.append((list(cur), row, [engine.length(s) + 1 for s in cur_slots], fetched))
            for i in cur:
                launched[i] += 1
            stats.steps += 1
            step_no += 1
        if not inflight:
            return
        members, row, lengths, event = inflight.popleft()
        if event is not None:
            event.synchronize()
        judge(members, row.tolist(), lengths)


def greedy_steps_in_flight(engine, slots: Sequence[int], tok_dev, steps: int, pinned):
    """`steps` greedy decode steps of the sequences in `slots`, none of which the host waits for: each
    step's ids (int32 on the device, `tok_dev` for the first) feed the next step on the device and go to
    row j of `pinned` (host memory, [steps, sequences]) by a copy of their own.  Returns the last ids on the
    device; the rows of `pinned` are complete once the device has been synchronised.  This is the decode
    loop of `generate` without its decisions: what a benchmark of the step itself times."""
    from .. import ops
    n = len(slots)
    for j in range(steps):
        tok_dev = ops.argmax(engine.step_device_tokens(slots, tok_dev), out=engine.token_buffer(n))
        engine.fetch_later(tok_dev, pinned[j])
    return tok_dev


def generate(engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_ids: Optional[Sequence[int]] = None,
             max_batch: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None,
             sampler_factory=None, steps_per_sync: int = 3) -> Tuple[List[List[int]], GenerationStats]:
    """Generate up to `max_tokens` new tokens for every prompt (lists of token
    ids).  Returns the new tokens of each prompt, in the prompts' order, and
    timing counters.  `stop_ids` defaults to the model's own end-of-sequence ids;
    `on_token(request index, token)` is called for every new token.
    `sampler_factory(params, request indices, device)` replaces the device
    sampler (tests of the loop's decisions use it).

    With `steps_per_sync` > 1 (and an engine that can take a step's tokens from the device) that many
    decode steps may be in flight: the sampled ids feed the next step on the device and reach the host
    by copies that nobody waits for, and the host looks at a step's ids only when later steps are
    already launched, so the device never waits for it.  A sequence that meets a stop token runs on for
    the steps already launched; its surplus tokens are dropped, so the output is the same.  Ends by
    `max_tokens` or by the context are known in advance and cost nothing."""
    sampling = sampling or SamplingParams()
    stop = frozenset(engine.model.spec.stop_token_ids if stop_ids is None else stop_ids)
    cache = engine.cache
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) > cache.max_seq_tokens:
            raise ValueError(f"prompt {i} has {len(p)} tokens; the cache holds sequences of up to "
                             f"{cache.max_seq_tokens}")
    requests = [Request(i, list(map(int, p)), int(max_tokens)) for i, p in enumerate(prompts)]
    pending = [r for r in requests if r.max_new > 0]
    for r in requests:
        if r.max_new <= 0:
            r.finish_reason = "length"
    stats = GenerationStats()
    max_batch = max_batch or cache.max_seqs

    while pending:
        free_tokens = min(g.pool.free for g in cache.kv_groups) * PAGE_TOKENS if cache.kv_groups else cache.max_tokens
        batch = plan_batch(pending, free_tokens, cache.slots.free, max_batch, cache.max_seq_tokens)
        pending = pending[len(batch):]
        stats.batches += 1
        slots = [engine.new_sequence() for _ in batch]
        try:
            sampler = (sampler_factory or Sampler)(sampling, [r.index for r in batch], engine.runtime.device)
            live = list(range(len(batch)))
            # the prompts, whole, in one step
            engine.synchronize()
            t0 = time.perf_counter()
            logits = engine.step([(slots[i], batch[i].prompt) for i in live])
            tokens = _to_host(engine, sampler.sample(logits))
            stats.prefill_seconds += time.perf_counter() - t0
            stats.prefill_tokens += sum(len(r.prompt) for r in batch)
            stats.steps += 1
            t0 = time.perf_counter()
            if steps_per_sync > 1 and hasattr(engine, "step_device_tokens"):
                _decode_ahead(engine, sampler, batch, slots, live, tokens, stop, on_token, stats, steps_per_sync)
                stats.generation_seconds += time.perf_counter() - t0
                continue
            while True:
                still = []
                for row, i in enumerate(live):
                    r, tok = batch[i], int(tokens[row])
                    r.output.append(tok)
                    stats.generated_tokens += 1
                    if on_token is not None:
                        on_token(r.index, tok)
                    r.finish_reason = finish_reason(tok, len(r.output), r.max_new, stop,
                                                    engine.length(slots[i]) + 1, cache.max_seq_tokens)
                    if r.finish_reason is None:
                        still.append(row)
                if not still:
                    break
                if len(still) != len(live):
                    sampler.keep(still)
                feed = [(slots[live[row]], [int(tokens[row])]) for row in still]
                live = [live[row] for row in still]
                logits = engine.step(feed)
                tokens = _to_host(engine, sampler.sample(logits))
                stats.steps += 1
            stats.generation_seconds += time.perf_counter() - t0
        finally:
            for s in slots:
                engine.end_sequence(s)
    return [r.output for r in requests], stats
