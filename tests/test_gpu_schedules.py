"""Schedules that the other model tests do not reach: decode steps of 65 to 200 live sequences (the
captured step's larger size classes, the prompt-shaped product inside a decode step), a window through
the engine with pages given back while steps are in flight, the benchmark's timed loop, and sampling
with steps in flight in bfloat16."""
import dataclasses

import pytest
import torch

from harness import run_batch, run_chunks
from plain import llama_plain as P
from util import TINY, assert_close, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu

# Llama-3.2-1B's layer widths, two layers; a small vocabulary keeps the plain implementation's 200
# sequences cheap (the products of a layer, which are what changes with the number of rows, keep their sizes).
WIDE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 4096, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 1, "eos_token_id": 2,
}


def _crowd(vocab, seed):
    """200 requests that start together: prompts of 1 to 6 tokens, then 2, 3, 5, 6, 7 or 9 tokens one by
    one, so that 200, 130, 100, 65, 60 and 40 sequences are alive in turn: the batch passes through the size
    classes 256, 192, 128, 96, 64 and 48 of the captured step."""
    g = torch.Generator().manual_seed(seed)
    prompt_lens = torch.randint(1, 7, (200,), generator=g).tolist()
    more = [2] * 70 + [3] * 30 + [5] * 35 + [6] * 5 + [7] * 20 + [9] * 40
    order = torch.randperm(200, generator=g).tolist()
    more = [more[i] for i in order]
    reqs = [random_tokens(p + m, vocab, seed * 1000 + i) for i, (p, m) in enumerate(zip(prompt_lens, more))]
    return reqs, prompt_lens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["tiny", "wide"])
def test_two_hundred_live_sequences(tmp_path, model_dirs, which, dtype):
    from picolm_b200 import ops
    from picolm_b200.engine import Engine
    if which == "tiny":
        d, vocab = model_dirs["A_sharp"], TINY["A"]["config"]["vocab_size"]
    else:
        d, vocab = make_model_dir(str(tmp_path / "wide"), WIDE, 21, sharpen=4.0), WIDE["vocab_size"]
    cfg, w = P.load_model(d)
    reqs, prompt_lens = _crowd(vocab, 5)
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 200, max_seqs=200)
    outs = run_batch(eng, reqs, prompt_lens)
    from picolm_b200.ops import _lib
    if not (_lib.CHECKED or _lib.TRACED):                     # (those builds launch every kernel by itself)
        assert {k[0] for k in eng._graphs} >= {256, 192, 128, 96, 64, 48}
    act = torch.bfloat16 if dtype == "bfloat16" else None
    for i in list(range(0, 200, 7)) + [199]:
        assert_close(outs[i], P.forward(cfg, w, reqs[i], act_dtype=act), dtype, f"{which} {dtype} request {i} of 200")
    eng.cache.check()
    assert eng.cache.slots.used == 0
    # a second crowd through the same slots and pages
    reqs2, lens2 = _crowd(vocab, 6)
    outs2 = run_batch(eng, reqs2[:100], lens2[:100])
    for i in (0, 31, 99):
        assert_close(outs2[i], P.forward(cfg, w, reqs2[i], act_dtype=act), dtype, f"{which} {dtype} second crowd {i}")
    eng.cache.check()
    if dtype == "bfloat16":
        ops.check_status()


def test_more_sequences_than_the_largest_graph(model_dirs):
    """Beyond the largest size class a decode step is launched kernel by kernel, and the buffer that the
    sampled ids pass through holds them all."""
    from picolm_b200.api import generate
    from picolm_b200.engine import Engine
    eng = Engine.from_folder(model_dirs["A_sharp"], dtype="float32", max_tokens=64 * 300, max_seqs=300)
    prompts = [random_tokens(1 + i % 5, 256, 900 + i) for i in range(300)]
    got = generate(eng, prompts, max_tokens=4, temperature=0.0, stop_ids=[])
    cfg, w = P.load_model(model_dirs["A_sharp"])
    for i in (0, 150, 256, 257, 299):
        assert got[i] == P.greedy(cfg, w, prompts[i], 4)
    eng.cache.check()


# ------------------------------------------------------------------ a window through the engine
WINDOW = 90


def _register_windowed():
    """Llama's layout with a sliding window on every attention, registered from here: the library's own
    architecture has none (the reference's Llama path has none)."""
    from picolm_b200 import register_architecture
    from picolm_b200.architectures.llama import llama_spec
    from picolm_b200.config import LlamaConfig
    from picolm_b200.config.spec import PartSpec

    def spec(cfg):
        s = llama_spec(cfg)
        layers = []
        for layer in s.layers:
            parts = dict(layer.parts)
            fam, mixer = parts["mixer"]
            parts["mixer"] = (fam, PartSpec(mixer.kind, dict(mixer.params, window=WINDOW), mixer.prefix))
            layers.append(dataclasses.replace(layer, parts=parts))
        return dataclasses.replace(s, layers=tuple(layers))

    register_architecture("WindowedLlamaForCausalLM", LlamaConfig.from_dict, spec)


def _windowed_greedy(cfg, w, prompt, n_new):
    toks, out = list(prompt), []
    for _ in range(n_new):
        out.append(P.argmax(P.forward(cfg, w, toks, window=WINDOW)[-1]))
        toks.append(out[-1])
    return out


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_through_the_engine(tmp_path, dtype, graphs):
    """Prompts in pieces that start after pages were given back, decoding across the pages on which the
    window's first key moves on, pages that one sequence gave back taken by another, with steps in flight.
    The null page, which the freed entries of a page table point at, holds large keys and values, so that a
    key read from it without the mask would show."""
    import json
    import os
    from picolm_b200.api import generate
    from picolm_b200.engine import Engine
    _register_windowed()
    cfg_dict = dict(TINY["A"]["config"], max_position_embeddings=512)
    d = make_model_dir(str(tmp_path / "win"), cfg_dict, 31, sharpen=3.0)
    with open(os.path.join(d, "config.json")) as f:
        on_disk = json.load(f)
    on_disk["architectures"] = ["WindowedLlamaForCausalLM"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(on_disk, f)
    cfg, w = P.load_model(d)
    # 9 pages: a sequence of 330 tokens would need 6 without the window; two of them run side by side below
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 9, max_seqs=3, use_graphs=graphs)
    assert eng.cache.kv_groups[0].spec.window == WINDOW
    for g in eng.cache.kv_groups:
        g.k[:, 0] = 30.0
        g.v[:, 0] = 30.0
    act = torch.bfloat16 if dtype == "bfloat16" else None
    a = random_tokens(330, 256, 71)
    ref = P.forward(cfg, w, a, window=WINDOW, act_dtype=act)
    assert not torch.allclose(ref[200:], P.forward(cfg, w, a, act_dtype=act)[200:], atol=1e-2)   # the window matters
    assert_close(run_chunks(eng, a, [100, 70, 30, 130]), ref, dtype, f"window {dtype} pieces")
    eng.cache.check()
    # two sequences of unequal lengths, then one token each for 200 steps: every page of the first 128
    # positions goes back to the pool meanwhile and is taken again by the other sequence
    b = random_tokens(290, 256, 72)
    outs = run_batch(eng, [a, b], [130, 60])
    assert_close(outs[0], ref, dtype, f"window {dtype} batch a")
    assert_close(outs[1], P.forward(cfg, w, b, window=WINDOW, act_dtype=act), dtype, f"window {dtype} batch b")
    eng.cache.check()
    assert eng.cache.kv_groups[0].pool.used == 0
    # generation with steps in flight: the pages are given back on the host while later steps are launched
    prompts = [a[:70], b[:9]]
    stretches = generate(eng, prompts, max_tokens=150, temperature=0.0, stop_ids=[], steps_per_sync=3)
    every = generate(eng, prompts, max_tokens=150, temperature=0.0, stop_ids=[], steps_per_sync=1)
    assert stretches == every
    if dtype == "float32":
        assert stretches[1][:40] == _windowed_greedy(cfg, w, prompts[1], 40)
    eng.cache.check()


# ------------------------------------------------------------- the benchmark's loop, and sampling in flight
def test_the_timed_loop_of_the_benchmark_gives_the_tokens_of_generate(tmp_path):
    """`greedy_steps_in_flight` (what bench.py times: every step's ids fed to the next step on the device
    and copied to the host by copies that nobody waits for) produces the tokens that `generate` produces
    when the host looks at every step, at the layer widths of the benchmark."""
    from picolm_b200 import ops
    from picolm_b200.api import generate
    from picolm_b200.engine import Engine
    from picolm_b200.engine.generate import greedy_steps_in_flight
    d = make_model_dir(str(tmp_path / "wide"), WIDE, 22, sharpen=4.0)
    eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8 * 4, max_seqs=8)
    prompts = [random_tokens(n, WIDE["vocab_size"], 40 + n) for n in (150, 9, 64, 65, 1, 33, 100, 128)]
    steps = 48
    want = generate(eng, prompts, max_tokens=steps + 1, temperature=0.0, stop_ids=[], steps_per_sync=1)
    slots = [eng.new_sequence() for _ in prompts]
    try:
        first = ops.argmax(eng.step(list(zip(slots, prompts))))
        pinned = torch.empty((steps, len(prompts)), dtype=torch.int32).pin_memory()
        greedy_steps_in_flight(eng, slots, first, steps, pinned)
        eng.synchronize()
        got = [[int(first[i])] + pinned[:, i].tolist() for i in range(len(prompts))]
    finally:
        for s in slots:
            eng.end_sequence(s)
    assert got == want
    ops.check_status()


def test_sampling_with_steps_in_flight_in_bfloat16(model_dirs):
    """Temperature sampling in bfloat16 gives the same tokens whether the host looks at every step or
    three steps are in flight, with sequences that end at different steps."""
    from picolm_b200.api import generate, model_load
    eng = model_load(model_dirs["B_sharp"], dtype="bfloat16", max_batch=5)
    prompts = [random_tokens(n, 384, 60 + i) for i, n in enumerate([4, 30, 2, 11, 7])]
    kw = dict(max_tokens=40, temperature=0.8, top_k=30, top_p=0.9, seed=11)
    free = generate(eng, prompts, stop_ids=[], steps_per_sync=1, **kw)
    stop = [free[0][5], free[3][17]]                           # tokens that end two sequences early
    every = generate(eng, prompts, stop_ids=stop, steps_per_sync=1, **kw)
    flight = generate(eng, prompts, stop_ids=stop, steps_per_sync=3, **kw)
    assert every == flight
    assert len(every[0]) <= 6 and len(every[3]) <= 18 and any(len(o) == 40 for o in every)
    eng.cache.check()


def test_prompt_steps_from_graphs_give_the_logits_of_single_launches(tmp_path):
    """Steps with prompts whose sequences want their last token's logits replay a captured graph of their size
    class (tokens padded to the class, sequences padded with empty ones): the same logits as the step launched
    kernel by kernel, for single prompts, unequal batches, a prompt fed in pieces, and size classes met twice
    (the second time the padding differs), at the 1B widths and a tiny size."""
    from picolm_b200.engine import Engine
    d = make_model_dir(str(tmp_path / "wide"), WIDE, 24, sharpen=4.0)
    cfg, w = P.load_model(d)
    eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 40, max_seqs=8)
    plain = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 40, max_seqs=8)
    plain.prompt_graphs = False
    from picolm_b200.ops import _lib
    if _lib.CHECKED or _lib.TRACED:
        pytest.skip("the checked and the traced build launch every kernel by itself")
    assert eng.prompt_graphs
    V = WIDE["vocab_size"]

    def last_logits(e, prompts, pieces=None):
        slots = [e.new_sequence() for _ in prompts]
        try:
            if pieces:                                     # the first prompt in pieces, nothing wanted but at the end
                o = 0
                for n in pieces[:-1]:
                    assert e.step([(slots[0], prompts[0][o:o + n])], [[]]) is None
                    o += n
                return e.step([(slots[0], prompts[0][o:])]).float().cpu()
            return e.step(list(zip(slots, prompts))).float().cpu()
        finally:
            for s in slots:
                e.end_sequence(s)

    cases = [[random_tokens(300, V, 1)], [random_tokens(n, V, 10 + n) for n in (150, 9, 64, 65)],
             [random_tokens(257, V, 2)], [random_tokens(n, V, 20 + n) for n in (1, 40)], [random_tokens(64, V, 3)]]
    for prompts in cases:
        got, want = last_logits(eng, prompts), last_logits(plain, prompts)
        assert_close(got, want, "bfloat16", f"prompts of {[len(p) for p in prompts]} from a graph")
        ref = torch.stack([P.forward(cfg, w, p, act_dtype=torch.bfloat16)[-1] for p in prompts])
        assert_close(got, ref, "bfloat16", "against the plain implementation")
    long = random_tokens(500, V, 4)
    got = last_logits(eng, [long], pieces=[200, 130, 170])
    assert_close(got, P.forward(cfg, w, long, act_dtype=torch.bfloat16)[-1:], "bfloat16", "a prompt in pieces from graphs")
    assert len(eng._prompt_graphs) >= 5 and not plain._prompt_graphs
    eng.cache.check()
    from picolm_b200 import ops
    ops.check_status()
