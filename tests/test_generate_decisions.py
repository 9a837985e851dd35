"""The generation loop's decisions, with a fake engine and sampler (no device):
which requests form a batch, when a sequence ends, what is fed, that slots come
back."""
from types import SimpleNamespace

import pytest

from picolm_b200.cache import CacheSpec, SequenceCache
from picolm_b200.engine.generate import Request, finish_reason, generate, plan_batch, tokens_reserved
from picolm_b200.sampling import SamplingParams, stream_seed


def test_tokens_reserved_counts_what_is_fed():
    assert tokens_reserved(5, 8, 1000) == 64            # 5 + 7 fed
    assert tokens_reserved(60, 5, 1000) == 64           # 60 + 4 = 64
    assert tokens_reserved(60, 6, 1000) == 128
    assert tokens_reserved(60, 500, 100) == 128         # capped by the longest sequence


def test_plan_batch_takes_requests_in_order_while_they_fit():
    reqs = [Request(i, [1] * n, 8) for i, n in enumerate([5, 70, 5, 5])]
    assert [r.index for r in plan_batch(reqs, 64 * 4, 8, 8, 4096)] == [0, 1, 2]
    assert [r.index for r in plan_batch(reqs, 64 * 4, 2, 8, 4096)] == [0, 1]
    assert [r.index for r in plan_batch(reqs, 64 * 4, 8, 1, 4096)] == [0]
    assert [r.index for r in plan_batch(reqs, 64, 8, 8, 4096)] == [0]
    with pytest.raises(RuntimeError, match="does not fit"):
        plan_batch(reqs[1:], 64, 8, 8, 4096)


def test_finish_reason():
    assert finish_reason(7, 1, 5, {7}, 10, 100) == "stop"
    assert finish_reason(3, 5, 5, {7}, 10, 100) == "length"
    assert finish_reason(3, 2, 5, {7}, 101, 100) == "context"
    assert finish_reason(3, 2, 5, {7}, 100, 100) is None


def test_stream_seed_follows_the_reference():
    assert stream_seed(42, 0) == 42 and stream_seed(42, 3) == 45
    assert stream_seed(0, 0) == 42                       # picolm/sampler.c:43: seed 0 reads as 42


class FakeEngine:
    """Counts what the loop feeds; the 'model' continues every sequence with
    last token + 1 (the fake sampler reads that from the fake logits)."""

    def __init__(self, max_tokens=64 * 6, max_seqs=3, max_seq_tokens=100):
        self.cache = SequenceCache([CacheSpec.kv(1, 16)], max_tokens, max_seqs, device="cpu",
                                   max_seq_tokens=max_seq_tokens, allocate_storage=False)
        self.model = SimpleNamespace(spec=SimpleNamespace(stop_token_ids=(50,)))
        self.runtime = SimpleNamespace(device="cpu")
        self.steps = []

    def new_sequence(self):
        return self.cache.allocate()

    def end_sequence(self, slot):
        self.cache.release(slot)

    def length(self, slot):
        return self.cache.length(slot)

    def synchronize(self):
        pass

    def step(self, entries, wants=None):
        self.cache.reserve([(s, len(t)) for s, t in entries])
        for s, t in entries:
            self.cache.advance(s, len(t))
        self.steps.append([(s, list(t)) for s, t in entries])
        return [t[-1] + 1 for _, t in entries]           # "logits": the next token itself


class FakeSampler:
    made = []

    def __init__(self, params, request_indices, device):
        self.rows = list(request_indices)
        FakeSampler.made.append(list(request_indices))

    def keep(self, rows):
        self.rows = [self.rows[r] for r in rows]

    def sample(self, logits):
        assert len(logits) == len(self.rows)
        return SimpleNamespace(tolist=lambda: list(logits))


def test_loop_batches_stops_and_gives_slots_back():
    FakeSampler.made.clear()
    eng = FakeEngine()
    prompts = [[10, 11, 12], [47], [20] * 40, [30, 31], [48, 49]]
    outs, stats = generate(eng, prompts, max_tokens=4, sampling=SamplingParams(temperature=0.0),
                           sampler_factory=FakeSampler)
    # the fake model counts up from the last prompt token; 50 is the stop token
    assert outs == [[13, 14, 15, 16], [48, 49, 50], [21, 22, 23, 24], [32, 33, 34, 35], [50]]
    assert FakeSampler.made == [[0, 1, 2], [3, 4]]       # 3 slots: two batches, requests in order
    first = eng.steps[0]
    assert [len(t) for _, t in first] == [3, 1, 40]      # unequal prompts in one step
    # decode steps feed one token each; the stop token and the last token are never fed
    fed = [t for step in eng.steps[1:] for _, toks in step for t in toks]
    assert 50 not in fed and 16 not in fed and 24 not in fed
    # request 1 ends after 3 tokens: the batch goes on without it
    assert [len(step) for step in eng.steps[:4]] == [3, 3, 3, 2]
    assert stats.batches == 2 and stats.generated_tokens == 4 + 3 + 4 + 4 + 1
    assert stats.prefill_tokens == 3 + 1 + 40 + 2 + 2
    eng.cache.check()
    assert eng.cache.slots.used == 0 and eng.cache.kv_groups[0].pool.used == 0


def test_loop_stops_at_the_context_limit():
    eng = FakeEngine(max_seq_tokens=8)
    outs, _ = generate(eng, [[1, 2, 3, 4, 5, 6]], max_tokens=10, sampling=SamplingParams(temperature=0.0),
                       sampler_factory=FakeSampler)
    # 6 prompt tokens + 2 fed = 8 positions; the third new token cannot be fed any more
    assert outs == [[7, 8, 9]]
    assert max(eng.cache.lengths.values(), default=0) == 0
    with pytest.raises(ValueError, match="holds sequences"):
        generate(eng, [[1] * 9], max_tokens=1, sampler_factory=FakeSampler)


def test_zero_new_tokens_and_empty_prompt():
    eng = FakeEngine()
    outs, stats = generate(eng, [[1, 2]], max_tokens=0, sampler_factory=FakeSampler)
    assert outs == [[]] and stats.steps == 0
    with pytest.raises(ValueError, match="empty"):
        generate(eng, [[]], max_tokens=1, sampler_factory=FakeSampler)


class StretchEngine(FakeEngine):
    """A fake engine that can take a step's tokens from 'the device' (a tensor)."""

    def step_device_tokens(self, slots, tokens):
        import torch
        return torch.tensor(self.step([(s, [int(t)]) for s, t in zip(slots, tokens.tolist())]), dtype=torch.int32)

    def fetch_later(self, tokens, row):
        row.copy_(tokens)


class TensorSampler(FakeSampler):
    def sample(self, logits):
        import torch
        assert len(logits) == len(self.rows)
        return torch.as_tensor(logits, dtype=torch.int32)


@pytest.mark.parametrize("most", [2, 3, 8])
def test_steps_in_flight_give_the_same_output(most):
    """The host looking at a step's tokens only when later steps are launched changes nothing but the
    work done: a stop token cuts the output where it stands, limits are met exactly (no step is
    launched past them), slots come back."""
    prompts = [[10, 11, 12], [45], [20] * 40, [30, 31], [48, 49], [44], [90] * 95]
    want, _ = generate(FakeEngine(), prompts, max_tokens=7, sampling=SamplingParams(temperature=0.0),
                       sampler_factory=FakeSampler, steps_per_sync=1)
    eng = StretchEngine()
    outs, stats = generate(eng, prompts, max_tokens=7, sampling=SamplingParams(temperature=0.0),
                           sampler_factory=TensorSampler, steps_per_sync=most)
    assert outs == want
    assert outs[1] == [46, 47, 48, 49, 50] and outs[4] == [50] and outs[6] == [91, 92, 93, 94, 95, 96]
    assert stats.generated_tokens == sum(len(o) for o in outs)
    # surplus work is bounded: a sequence runs at most `most - 1` steps past its stop token, none past
    # its limits (the cache would have refused a token beyond the context)
    fed = sum(len(toks) for step in eng.steps for _, toks in step)
    assert fed <= sum(len(p) for p in prompts) + sum(len(o) + most - 1 for o in outs)
    eng.cache.check()
    assert eng.cache.slots.used == 0 and eng.cache.kv_groups[0].pool.used == 0


def test_graph_size_and_length_classes():
    """A captured decode step serves every batch up to its size class and every length up to its
    length class: the classes must cover what they are asked for, never shrink, and stay few."""
    from picolm_b200.engine.decode_graph import BUCKETS, bucket_for, length_class
    assert [bucket_for(n) for n in (1, 2, 3, 8, 9, 64, 65, 256)] == [1, 2, 4, 8, 16, 64, 96, 256]
    assert bucket_for(BUCKETS[-1] + 1) is None                     # beyond the largest class: no graph
    longest = 1 << 17
    classes, last = set(), 0
    for n in range(1, longest + 1, 37):
        c = length_class(n, longest)
        assert n <= c <= longest and c >= last                      # covers the length, never shrinks
        assert c - n < max(512, n // 2 + 1)                         # less than a step of 512, or than half the length, above it
        classes.add(c)
        last = c
    assert len(classes) <= 40
    assert length_class(100, 64) == 64                              # never beyond the longest sequence of the cache


class LateCopyEngine(StretchEngine):
    """A fake engine with a token buffer of its own whose copies to the host run as late as they may:
    when their event is waited for.  If the buffer has been written in between, the copy would carry
    other ids than were sampled: the stand-in raises.  `guard` says whether a write of the buffer first
    waits for the pending copy, as `Engine.before_token_write` does."""

    class Copy:
        def __init__(self, src, row):
            self.src, self.row, self.seen, self.done = src, row, src.clone(), False

        def synchronize(self):
            if not self.done:
                import torch
                assert torch.equal(self.src, self.seen), "the token buffer was overwritten before its copy to the host ran"
                self.row.copy_(self.src)
                self.done = True

    def __init__(self, guard=True, **kw):
        import torch
        super().__init__(**kw)
        self.buf = torch.zeros(self.cache.max_seqs, dtype=torch.int32)
        self.pending, self.guard = None, guard

    def token_buffer(self, n):
        return self.buf[:n]

    def before_token_write(self):
        if self.pending is not None:
            self.pending.synchronize()
            self.pending = None

    def step_device_tokens(self, slots, tokens):
        n = len(slots)
        if tokens.data_ptr() != self.buf.data_ptr():          # the batch shrank: other rows than the buffer holds
            if self.guard:
                self.before_token_write()
            self.buf[:n] = tokens
        out = super().step_device_tokens(slots, self.buf[:n])
        self.before_token_write()                             # the sampler that follows writes the buffer
        return out

    def fetch_later(self, tokens, row):
        self.pending = self.Copy(tokens, row)
        return self.pending


class BufferSampler(TensorSampler):
    def sample(self, logits, out=None):
        import torch
        t = torch.as_tensor(logits, dtype=torch.int32)
        if out is None:
            return t
        out.copy_(t)
        return out


def test_the_token_buffer_is_not_written_under_a_pending_copy():
    """A sequence that leaves the batch from its first row (here: its context is full) makes the loop
    regroup the ids on the device and write them into the engine's token buffer; that write has to wait
    for the last copy of the buffer to the host."""
    prompts = [[90] * 97, [10, 11, 12], [45], [20] * 40]
    want, _ = generate(FakeEngine(max_seqs=4, max_tokens=64 * 6), prompts, max_tokens=7,
                       sampling=SamplingParams(temperature=0.0), sampler_factory=FakeSampler, steps_per_sync=1)
    assert [len(o) for o in want] == [4, 7, 5, 7]
    eng = LateCopyEngine(max_seqs=4, max_tokens=64 * 6)
    outs, _ = generate(eng, prompts, max_tokens=7, sampling=SamplingParams(temperature=0.0),
                       sampler_factory=BufferSampler, steps_per_sync=3)
    assert outs == want
    with pytest.raises(AssertionError, match="overwritten before its copy"):
        generate(LateCopyEngine(guard=False, max_seqs=4, max_tokens=64 * 6), prompts, max_tokens=7,
                 sampling=SamplingParams(temperature=0.0), sampler_factory=BufferSampler, steps_per_sync=3)


def test_more_sequences_than_token_ids_are_refused():
    """The engine's token buffer holds one id per sequence of the cache; a sampler's `out` that is not
    exactly the batch's size is refused before any kernel writes it."""
    import torch
    from picolm_b200.engine.engine import Engine
    from picolm_b200.ops import KernelError
    from picolm_b200.ops.sampling import _token_out
    eng = Engine.__new__(Engine)
    eng._tokens = torch.zeros(300, dtype=torch.int32)
    assert eng.token_buffer(257).numel() == 257
    with pytest.raises(ValueError, match="at most 300"):
        eng.token_buffer(301)
    logits = torch.zeros((257, 8))
    assert _token_out(None, 257, logits, "argmax").shape == (257,)
    with pytest.raises(KernelError, match=r"int32 \[257\]"):
        _token_out(torch.zeros(256, dtype=torch.int32), 257, logits, "argmax")
    with pytest.raises(KernelError, match="int32"):
        _token_out(torch.zeros(257, dtype=torch.int64), 257, logits, "sample")
    # the loop with 257 sequences alive at once and a buffer sized by the cache
    big = LateCopyEngine(max_seqs=257, max_tokens=64 * 257)
    prompts = [[1 + i % 40] for i in range(257)]
    outs, _ = generate(big, prompts, max_tokens=3, sampling=SamplingParams(temperature=0.0),
                       sampler_factory=BufferSampler, steps_per_sync=2)
    assert outs == [[p[0] + 1, p[0] + 2, p[0] + 3] for p in prompts]
