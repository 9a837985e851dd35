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
from typing import Callable, Dict, List, Optional, Sequence, Tuple

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


def steps_ahead(most: int, generated: Sequence[int], max_new: Sequence[int], lengths: Sequence[int],
                max_seq_tokens: int) -> int:
    """How many steps a batch may run before the host has to look at it for another reason than a stop
    token: until the first of its sequences produces its last allowed token or fills the context.
    `generated[i]` new tokens exist of sequence i (the last one not fed yet), `lengths[i]` tokens of it
    are in the cache; every sequence is one that goes on (`finish_reason` said None)."""
    k = most
    for n, limit, length in zip(generated, max_new, lengths):
        k = min(k, limit - n, max_seq_tokens - length)
    return max(k, 1)


def _to_host(engine, tokens):
    fetch = getattr(engine, "to_host", None)
    return fetch(tokens) if fetch is not None else tokens.tolist()


def _decode_in_stretches(engine, sampler, batch, slots, live, first_tokens, stop, on_token, stats, most) -> None:
    """The decode loop of one batch with the host looking in every `most` steps at the latest (see
    `generate`).  `first_tokens`: what the prompts' step sampled, on the host."""
    import torch
    cache = engine.cache
    device = engine.runtime.device
    pinned = torch.empty((most, len(live)), dtype=torch.int32)
    if torch.device(device).type == "cuda":
        pinned = pinned.pin_memory()
    buffer = getattr(engine, "token_buffer", None)       # where the engine's captured steps read their ids
    rows = [[int(t) for t in first_tokens]]              # stretches of token rows still to be judged
    base = [engine.length(slots[i]) for i in live]       # cache length when rows[0] was sampled
    tok_dev = None
    while True:
        still = list(range(len(live)))
        for j, row_tokens in enumerate(rows):
            nxt = []
            for row in still:
                r, tok = batch[live[row]], row_tokens[row]
                r.output.append(tok)
                stats.generated_tokens += 1
                if on_token is not None:
                    on_token(r.index, tok)
                r.finish_reason = finish_reason(tok, len(r.output), r.max_new, stop, base[row] + j + 1,
                                                cache.max_seq_tokens)
                if r.finish_reason is None:
                    nxt.append(row)
            still = nxt
        if not still:
            return
        last = rows[-1]
        if len(still) != len(live) or tok_dev is None:
            sampler.keep(still)
            tok_dev = torch.tensor([last[row] for row in still], dtype=torch.int32, device=device)
            live = [live[row] for row in still]
        cur = [slots[i] for i in live]
        base = [engine.length(s) for s in cur]
        k = steps_ahead(most, [len(batch[i].output) for i in live], [batch[i].max_new for i in live], base,
                        cache.max_seq_tokens)
        for j in range(k):
            logits = engine.step_device_tokens(cur, tok_dev)
            tok_dev = sampler.sample(logits, out=buffer(len(cur))) if buffer else sampler.sample(logits)
            engine.fetch_later(tok_dev, pinned[j, :len(live)])
            stats.steps += 1
        engine.synchronize()
        rows = pinned[:k, :len(live)].tolist()
        base = [b + 1 for b in base]                     # rows[j] was sampled with base + j + 1 tokens cached


def generate(engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_ids: Optional[Sequence[int]] = None,
             max_batch: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None,
             sampler_factory=None, steps_per_sync: int = 8) -> Tuple[List[List[int]], GenerationStats]:
    """Generate up to `max_tokens` new tokens for every prompt (lists of token
    ids).  Returns the new tokens of each prompt, in the prompts' order, and
    timing counters.  `stop_ids` defaults to the model's own end-of-sequence ids;
    `on_token(request index, token)` is called for every new token.
    `sampler_factory(params, request indices, device)` replaces the device
    sampler (tests of the loop's decisions use it).

    With `steps_per_sync` > 1 (and an engine that can take a step's tokens from the device) the host
    looks at the new tokens only every so many steps: the sampled ids feed the next step on the device
    and reach the host by copies that nobody waits for, so the host prepares and launches steps while
    earlier ones run.  A sequence that meets a stop token in between runs on to the end of that
    stretch; its surplus tokens are dropped, so the output is the same."""
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
                _decode_in_stretches(engine, sampler, batch, slots, live, tokens, stop, on_token, stats,
                                     steps_per_sync)
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
