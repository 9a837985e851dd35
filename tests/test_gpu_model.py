"""The engine against the plain implementation, in float32 and in bfloat16,
for every way of cutting requests into steps."""
import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import llama_plain as P
from util import TINY, assert_close, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
MODELS = ["A", "B", "A_sharp", "B_sharp"]


@pytest.fixture(scope="module")
def engines(model_dirs):
    from picolm_b200.engine import Engine
    cache = {}

    def get(name, dtype):
        key = (name, dtype)
        if key not in cache:
            cache[key] = Engine.from_folder(model_dirs[name], dtype=dtype, max_tokens=64 * 24, max_seqs=8)
        return cache[key]

    return get


@pytest.fixture(scope="module")
def plain(model_dirs):
    models, memo = {}, {}

    def logits(name, tokens, dtype):
        if name not in models:
            models[name] = P.load_model(model_dirs[name])
        key = (name, tuple(tokens), dtype)
        if key not in memo:
            cfg, w = models[name]
            memo[key] = P.forward(cfg, w, list(tokens), act_dtype=torch.bfloat16 if dtype == "bfloat16" else None)
        return memo[key]

    return logits


def _vocab(name):
    return TINY[name[0]]["config"]["vocab_size"]


def _ctx(name):
    return TINY[name[0]]["config"]["max_position_embeddings"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_each_request_alone_and_whole(engines, plain, name, dtype):
    eng = engines(name, dtype)
    for n, seed in ((1, 11), (5, 12), (17, 13), (64, 14), (65, 15), (_ctx(name), 16)):
        toks = random_tokens(n, _vocab(name), seed)
        assert_close(run_whole(eng, toks), plain(name, toks, dtype), dtype, f"{name} {dtype} whole n={n}")
    eng.cache.check()
    assert eng.cache.slots.used == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_last_32_tokens_one_by_one(engines, plain, name, dtype):
    eng = engines(name, dtype)
    for n, seed in ((33, 21), (80, 22), (_ctx(name), 23), (20, 24)):
        toks = random_tokens(n, _vocab(name), seed)
        got = run_tail(eng, toks, tail=32)
        assert_close(got, plain(name, toks, dtype), dtype, f"{name} {dtype} tail n={n}")
    assert eng.cache.slots.used == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_batches_of_unequal_lengths_one_after_another(engines, plain, name, dtype):
    """Prompts of unequal lengths start together, decode from their own
    continuations, the shorter ones end earlier; then the next batch takes the
    slots over.  The configuration's own batch comes first (A: 5/11/17 + 8,
    B: 1/40 + 12)."""
    eng = engines(name, dtype)
    base = TINY[name[0]]
    plans = [(base["prompts"], [base["decode"]] * len(base["prompts"])),
             ([3, 64, 1, 30], [5, 1, 20, 0]),
             ([70, 2], [3, 40]),
             ([9, 9, 9, 9, 9, 9, 9, 9], [2, 4, 6, 8, 1, 3, 5, 7])]
    seed = 100
    for prompt_lens, decodes in plans:
        reqs = []
        for n, dcd in zip(prompt_lens, decodes):
            seed += 1
            reqs.append(random_tokens(n + dcd, _vocab(name), seed))
        outs = run_batch(eng, reqs, prompt_lens)
        for r, got in zip(reqs, outs):
            assert_close(got, plain(name, r, dtype), dtype, f"{name} {dtype} batch {prompt_lens}+{decodes} len={len(r)}")
        eng.cache.check()
        assert eng.cache.slots.used == 0 and all(g.pool.used == 0 for g in eng.cache.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_long_decoding_and_first_tokens(engines, plain, name, dtype):
    """A one-token prompt, then every further token decoded one by one up to the
    context limit: the first tokens of a sequence and a long decode in one."""
    eng = engines(name, dtype)
    toks = random_tokens(_ctx(name), _vocab(name), 31)
    got = run_tail(eng, toks, tail=len(toks) - 1)
    ref = plain(name, toks, dtype)
    assert_close(got[:4], ref[:4], dtype, f"{name} {dtype} first tokens")
    assert_close(got, ref, dtype, f"{name} {dtype} long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_prompt_in_pieces(engines, plain, name, dtype):
    """A prompt fed in pieces of several tokens: every piece after the first attends to a cached prefix
    and to itself (pieces that end inside a page, a piece of one token in between)."""
    eng = engines(name, dtype)
    n = min(_ctx(name), 128)
    toks = random_tokens(n, _vocab(name), 77)
    sizes = [40, 30, 1, 17, n - 88]
    assert_close(run_chunks(eng, toks, sizes), plain(name, toks, dtype), dtype, f"{name} {dtype} pieces")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_and_a_prompt_in_one_step(engines, plain, dtype):
    """The step function takes any mixture: a sequence that goes on by one token beside one that brings a
    whole prompt, then both go on with pieces of unequal lengths."""
    name = "A_sharp"
    eng = engines(name, dtype)
    a, b = random_tokens(60, _vocab(name), 81), random_tokens(45, _vocab(name), 82)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    try:
        got_a = [eng.step([(sa, a[:20])], [list(range(20))]).float().cpu()]
        out = eng.step([(sa, a[20:21]), (sb, b[:30])], [[0], list(range(30))]).float().cpu()
        got_a.append(out[:1])
        got_b = [out[1:]]
        out = eng.step([(sb, b[30:45]), (sa, a[21:60])], [list(range(15)), list(range(39))]).float().cpu()
        got_b.append(out[:15])
        got_a.append(out[15:])
    finally:
        eng.end_sequence(sa)
        eng.end_sequence(sb)
    assert_close(torch.cat(got_a), plain(name, a, dtype), dtype, f"{dtype} mixed step, first sequence")
    assert_close(torch.cat(got_b), plain(name, b, dtype), dtype, f"{dtype} mixed step, second sequence")
    eng.cache.check()


def test_float32_results_do_not_depend_on_the_cut(engines):
    """In float32 every kernel accumulates in an order fixed by the row itself,
    so the three ways of cutting agree to the last bit."""
    eng = engines("B_sharp", "float32")
    toks = random_tokens(90, _vocab("B"), 41)
    other = random_tokens(50, _vocab("B"), 42)
    whole = run_whole(eng, toks)
    tail = run_tail(eng, toks, tail=32)
    batch = run_batch(eng, [other, toks], [7, 33])[1]
    assert torch.equal(whole, tail) and torch.equal(whole, batch)


def test_step_refuses_bad_input_before_any_launch(engines):
    from picolm_b200.cache import CacheFull
    eng = engines("A", "float32")
    s = eng.new_sequence()
    try:
        with pytest.raises(ValueError, match="vocabulary"):
            eng.step([(s, [1, 256])])
        with pytest.raises(ValueError, match="at least one token"):
            eng.step([(s, [])])
        with pytest.raises(CacheFull):
            eng.step([(s, [1] * 129)])                      # beyond max_position_embeddings
        with pytest.raises(IndexError):
            eng.step([(s, [1, 2])], [[2]])
        assert eng.length(s) == 0
        eng.cache.check()
    finally:
        eng.end_sequence(s)
