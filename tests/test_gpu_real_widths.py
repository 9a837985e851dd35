"""The engine at the widths of a real model (Llama-3.2-1B's layer sizes, two layers): the tcgen05
products, the tcgen05 prefill attention, the cluster kernel of decode and the CUDA graphs all run at
the shapes that serving uses, against the plain implementation on the CPU."""
import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import llama_plain as P
from util import assert_close, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 128000, "eos_token_id": 128001,
}


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    d = make_model_dir(str(tmp_path_factory.mktemp("real") / "m"), CONFIG, 2, sharpen=4.0)
    cfg, w = P.load_model(d)
    toks = {n: random_tokens(n, CONFIG["vocab_size"], 300 + n) for n in (200, 70, 33)}
    ref = {}

    def plain(n, dtype):
        key = (n, dtype)
        if key not in ref:
            ref[key] = P.forward(cfg, w, toks[n], act_dtype=torch.bfloat16 if dtype == "bfloat16" else None)
        return ref[key]

    return d, toks, plain


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_real_widths_in_every_cut(real, dtype):
    from picolm_b200.engine import Engine
    d, toks, plain = real
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 16, max_seqs=4)
    for n in (200, 33):
        assert_close(run_whole(eng, toks[n]), plain(n, dtype), dtype, f"real widths {dtype} whole {n}")
    assert_close(run_tail(eng, toks[70], tail=32), plain(70, dtype), dtype, f"real widths {dtype} tail")
    assert_close(run_chunks(eng, toks[200], [90, 70, 40]), plain(200, dtype), dtype, f"real widths {dtype} pieces")
    outs = run_batch(eng, [toks[200], toks[33], toks[70]], [150, 20, 64])
    for n, got in zip((200, 33, 70), outs):
        assert_close(got, plain(n, dtype), dtype, f"real widths {dtype} batch {n}")
    eng.cache.check()
    if dtype == "bfloat16":
        from picolm_b200 import ops
        ops.check_status()


def test_graph_and_plain_launches_agree(real):
    """A decode step replayed from a CUDA graph gives the logits of the same step launched kernel by
    kernel, up to rounding: the graph sizes the decode attention's key ranges for its length class,
    the plain launch for the true length, so the partial sums are cut differently."""
    from picolm_b200.engine import Engine
    from picolm_b200.ops import _lib
    d, toks, _ = real
    outs = []
    for graphs in (True, False):
        eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8, max_seqs=4, use_graphs=graphs)
        outs.append(torch.cat(run_batch(eng, [toks[70], toks[33]], [40, 9])))
        if not (_lib.CHECKED or _lib.TRACED):                     # (those builds launch every kernel by itself)
            assert bool(eng._graphs) == graphs
        del eng
    assert_close(outs[0], outs[1], "bfloat16", "graph against plain launches")


# A narrow model with the head size of the larger Llamas: 128-wide heads go through the other
# instantiation of every attention kernel (tcgen05 prefill, mma.sync decode in and outside a cluster).
CONFIG_HD128 = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 640,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 1792,
    "vocab_size": 2000, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 4096, "tie_word_embeddings": False, "hidden_act": "silu",
    "bos_token_id": 1, "eos_token_id": 2,
}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_head_size_128_in_every_cut(tmp_path_factory, dtype):
    from picolm_b200.engine import Engine
    d = make_model_dir(str(tmp_path_factory.mktemp("hd128") / "m"), CONFIG_HD128, 5, sharpen=4.0)
    cfg, w = P.load_model(d)
    toks = {n: random_tokens(n, CONFIG_HD128["vocab_size"], 500 + n) for n in (300, 130, 40)}
    act = torch.bfloat16 if dtype == "bfloat16" else None
    ref = {n: P.forward(cfg, w, t, act_dtype=act) for n, t in toks.items()}
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 24, max_seqs=4)
    assert_close(run_whole(eng, toks[300]), ref[300], dtype, f"hd128 {dtype} whole")
    assert_close(run_tail(eng, toks[130], tail=32), ref[130], dtype, f"hd128 {dtype} tail")
    assert_close(run_chunks(eng, toks[300], [130, 100, 70]), ref[300], dtype, f"hd128 {dtype} pieces")
    outs = run_batch(eng, [toks[300], toks[40], toks[130]], [200, 25, 100])
    for n, got in zip((300, 40, 130), outs):
        assert_close(got, ref[n], dtype, f"hd128 {dtype} batch {n}")
    eng.cache.check()
    if dtype == "bfloat16":
        from picolm_b200 import ops
        ops.check_status()


# A long sequence: dozens of pages, so that the prompt kernel walks many of them per query tile and the
# decode kernel cuts the keys into more ranges than a cluster holds (scratch memory and a merge kernel).
CONFIG_LONG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 512,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 1024,
    "vocab_size": 1500, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 1024},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 1, "eos_token_id": 2,
}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_long_sequence(tmp_path_factory, dtype):
    from picolm_b200 import ops
    from picolm_b200.engine import Engine
    d = make_model_dir(str(tmp_path_factory.mktemp("long") / "m"), CONFIG_LONG, 9, sharpen=4.0)
    cfg, w = P.load_model(d)
    n = 4700
    toks = random_tokens(n, CONFIG_LONG["vocab_size"], 77)
    ref = P.forward(cfg, w, toks, act_dtype=torch.bfloat16 if dtype == "bfloat16" else None)
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 76, max_seqs=2)
    if dtype == "bfloat16":
        assert ops.decode_splits(1, 8, 2, n, 64) > 8            # the decode steps below go through scratch memory
    s = eng.new_sequence()
    try:
        head = n - 12
        rows = [0, 63, 64, 1000, 2047, 2048, 4000, head - 1]
        got = [eng.step([(s, toks[:head])], [rows]).float().cpu()]
        want = [ref[rows]]
        for t in range(head, n):
            got.append(eng.step([(s, [toks[t]])], [[0]]).float().cpu())
            want.append(ref[t:t + 1])
    finally:
        eng.end_sequence(s)
    assert_close(torch.cat(got), torch.cat(want), dtype, f"long sequence {dtype}")
    eng.cache.check()
    if dtype == "bfloat16":
        ops.check_status()


# Prompts long enough for the forms of the prompt-shaped product that short prompts never reach: pairs of CTAs
# with two tiles of K per copy (QKV, gate/up with SwiGLU), pairs that walk few tiles' stages as one stream (the down
# projection of 1,024 tokens), the add to the stream and the stores by the copy engine, and a prompt step replayed
# from a CUDA graph of its length class.  Layer sizes of Llama-3.2-1B, a small vocabulary.
CONFIG_PROMPT = dict(CONFIG, vocab_size=2000, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)


def test_long_prompts_at_real_widths(tmp_path_factory):
    from picolm_b200 import ops
    from picolm_b200.engine import Engine
    from picolm_b200.ops.gemm import _pair_streamed, pair_pays
    assert pair_pays(1024, 3072, 2048, 0) and pair_pays(1024, 16384, 2048, 1)       # the forms named above are
    assert pair_pays(1024, 2048, 8192, 2) and _pair_streamed(1024, 2048, 8192) > 0  # what these prompts run
    d = make_model_dir(str(tmp_path_factory.mktemp("prompt") / "m"), CONFIG_PROMPT, 11, sharpen=4.0)
    cfg, w = P.load_model(d)
    toks = {n: random_tokens(n, CONFIG_PROMPT["vocab_size"], 900 + n) for n in (1024, 700)}
    ref = {n: P.forward(cfg, w, t, act_dtype=torch.bfloat16) for n, t in toks.items()}
    rows = {1024: [0, 1, 127, 128, 255, 256, 511, 777, 1023], 700: [0, 63, 64, 300, 699]}
    for graphs in (True, False):
        eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 40, max_seqs=2)
        eng.prompt_graphs = graphs and eng.prompt_graphs
        for n in (1024, 700, 1024):                           # the second 1,024 replays the graph of the first
            s = eng.new_sequence()
            try:
                got = eng.step([(s, toks[n])], [rows[n]]).float().cpu()
            finally:
                eng.end_sequence(s)
            assert_close(got, ref[n][rows[n]], "bfloat16", f"{n} tokens, graphs {graphs}")
        both = [eng.new_sequence(), eng.new_sequence()]       # the two prompts in one step: 1,724 rows
        try:
            got = eng.step([(both[0], toks[1024]), (both[1], toks[700])], [rows[1024], rows[700]]).float().cpu()
        finally:
            for s in both:
                eng.end_sequence(s)
        assert_close(got, torch.cat([ref[1024][rows[1024]], ref[700][rows[700]]]), "bfloat16", f"both, graphs {graphs}")
        eng.cache.check()
        ops.check_status()
        del eng


def test_the_last_layer_runs_on_the_wanted_rows_alone(real):
    """A prompt whose last logits alone are wanted runs its last layer's feed-forward on that row only (the
    stream is narrowed once the attention has seen all tokens): the same logits, up to rounding, as when every
    row is wanted and nothing is narrowed; and a prompt of which nothing is wanted leaves the cache as the other
    steps do (the next token's logits agree with the plain implementation)."""
    from picolm_b200.engine import Engine
    d, toks, plain = real
    eng = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8, max_seqs=2)
    n = 200
    ref = plain(n, "bfloat16")
    s = eng.new_sequence()
    try:
        few = eng.step([(s, toks[n])], [[n - 1]]).float().cpu()
    finally:
        eng.end_sequence(s)
    s = eng.new_sequence()
    try:
        every = eng.step([(s, toks[n])], [list(range(n))]).float().cpu()
    finally:
        eng.end_sequence(s)
    assert_close(few, ref[n - 1:], "bfloat16", "the last row alone")
    assert_close(every, ref, "bfloat16", "every row")
    s = eng.new_sequence()
    try:
        assert eng.step([(s, toks[n][:n - 1])], [[]]) is None       # nothing wanted: the last layer stops after its mixer
        nxt = eng.step([(s, toks[n][n - 1:])], [[0]]).float().cpu()
    finally:
        eng.end_sequence(s)
    assert_close(nxt, ref[n - 1:], "bfloat16", "after a prompt of which nothing was wanted")
    eng.cache.check()
