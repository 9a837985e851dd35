"""Greedy and sampled generation through the Python entry point and the command line."""
import os
import re
import subprocess
import sys

import pytest
import torch

from plain import llama_plain as P
from util import TINY, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_greedy_generation_matches_the_plain_implementation(model_dirs, name):
    """float32: token for token.  Unequal prompts, more requests than fit one
    batch (so slots are used again), a stop token that ends one request early."""
    from picolm_b200.api import generate, model_load
    cfg, w = P.load_model(model_dirs[name])
    vocab = TINY[name[0]]["config"]["vocab_size"]
    prompts = [random_tokens(n, vocab, 50 + i) for i, n in enumerate([5, 11, 17, 1, 40, 3, 64])]
    free_run = [P.greedy(cfg, w, p, 10) for p in prompts]
    stop = free_run[2][4]                                       # request 2 meets this token at its 5th step
    want = [P.greedy(cfg, w, p, 10, stop=(stop,)) for p in prompts]
    assert len(want[2]) <= 5
    eng = model_load(model_dirs[name], dtype="float32", max_batch=3)
    got, stats = generate(eng, prompts, max_tokens=10, temperature=0.0, stop_ids=[stop], return_stats=True)
    assert got == want
    assert stats.batches == 3 and eng.cache.slots.used == 0
    eng.cache.check()
    # alone or in a batch: the same tokens
    assert generate(eng, [prompts[1]], max_tokens=10, temperature=0.0, stop_ids=[stop]) == [want[1]]
    # the host looking at the tokens after every step, or only every few steps: the same tokens
    for every in (1, 3):
        assert generate(eng, prompts, max_tokens=10, temperature=0.0, stop_ids=[stop], steps_per_sync=every) == want
    eng.cache.check()


def test_bfloat16_greedy_follows_the_plain_bfloat16_twin(model_dirs):
    from picolm_b200.api import generate, model_load
    name = "A_sharp"
    cfg, w = P.load_model(model_dirs[name])
    prompts = [random_tokens(n, 256, 70 + i) for i, n in enumerate([9, 30])]
    eng = model_load(model_dirs[name], dtype="bfloat16", max_batch=2)
    got = generate(eng, prompts, max_tokens=12, temperature=0.0, stop_ids=[])
    # every generated token is the argmax of the twin's logits for the sequence so far,
    # or so close to it that 16-bit rounding decides
    for p, out in zip(prompts, got):
        assert len(out) == 12
        seq = list(p)
        for tok in out:
            logits = P.forward(cfg, w, seq, act_dtype=torch.bfloat16)[-1]
            assert logits[tok] >= logits.max() - 0.05 * logits.std()
            seq.append(tok)


def test_generation_across_a_new_graph(tmp_path):
    """Greedy generation that crosses the length at which decode steps get another CUDA graph (every
    512 positions), while the sampled ids stay on the device: the capture in the middle must not touch
    them.  Against the plain implementation, token for token, in float32; bfloat16 must agree with itself
    whether the host looks at every token or not."""
    from picolm_b200.api import generate, model_load
    from util import make_model_dir
    cfg_dict = dict(TINY["A"]["config"], max_position_embeddings=1024)
    d = make_model_dir(str(tmp_path / "long"), cfg_dict, 7, sharpen=3.0)
    cfg, w = P.load_model(d)
    prompts = [random_tokens(500, 256, 91), random_tokens(470, 256, 92)]
    want = [P.greedy(cfg, w, p, 40) for p in prompts]
    eng = model_load(d, dtype="float32", max_batch=2)
    assert generate(eng, prompts, max_tokens=40, temperature=0.0, stop_ids=[]) == want
    from picolm_b200.ops import _lib
    if not (_lib.CHECKED or _lib.TRACED):                     # (those builds launch every kernel by itself)
        assert len(eng._graphs) >= 2                          # the two length classes each have a graph
    eng16 = model_load(d, dtype="bfloat16", max_batch=2)
    a = generate(eng16, prompts, max_tokens=40, temperature=0.0, stop_ids=[])
    b = generate(eng16, prompts, max_tokens=40, temperature=0.0, stop_ids=[], steps_per_sync=1)
    assert a == b


def test_sampling_is_seeded_per_request(model_dirs):
    """The same seed gives the same tokens; a request's tokens do not depend on
    its batch (its stream is seeded by its index among the prompts)."""
    from picolm_b200.api import generate, model_load
    eng = model_load(model_dirs["B_sharp"], dtype="float32", max_batch=4)
    prompts = [random_tokens(n, 384, 80 + i) for i, n in enumerate([4, 9, 2, 20])]
    a = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=7, stop_ids=[])
    b = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=7, stop_ids=[])
    c = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=8, stop_ids=[])
    assert a == b and a != c
    one_by_one = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=7, stop_ids=[],
                          max_batch=1)
    assert one_by_one == a
    every_step = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=7, stop_ids=[a[1][3]],
                          steps_per_sync=1)
    stretches = generate(eng, prompts, max_tokens=16, temperature=0.9, top_k=20, top_p=0.95, seed=7, stop_ids=[a[1][3]])
    assert every_step == stretches and len(stretches[1]) <= 4


def test_command_line(model_dirs):
    cfg, w = P.load_model(model_dirs["A_sharp"])
    want = [P.greedy(cfg, w, p, 5) for p in ([5, 6, 7], [9])]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "picolm_b200"), model_dirs["A_sharp"],
                        "-p", "5,6,7; 9", "-n", "5", "-t", "0", "--dtype", "float32", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = [[int(t) for t in ln.split()] for ln in r.stdout.strip().splitlines()]
    assert lines == want
    assert "Prefill: 4 tokens" in r.stderr and "Generation: 10 tokens" in r.stderr
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "picolm_b200"), model_dirs["A_sharp"],
                        "--list-tensors"], capture_output=True, text=True, timeout=60)
    assert "model.layers.1.mlp.down_proj.weight\t[64, 172]\tBF16" in r.stdout
    # the reference's --benchmark-ctx: one CSV line per round, the cached length growing by prompt + -n
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "picolm_b200"), model_dirs["A_sharp"],
                        "-p", "5,6,7,8,9,10", "-n", "10", "-c", "70", "--benchmark-ctx"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [ln.split(",") for ln in r.stderr.splitlines() if re.fullmatch(r"\d+,[0-9.]+,[0-9.]+", ln)]
    assert "ctx_size,prefill_tok/s,gen_tok/s" in r.stderr
    assert [int(x[0]) for x in rows] == [0, 16, 32, 48] and all(float(x[1]) > 0 and float(x[2]) > 0 for x in rows)
    # the reference's --benchmark: per iteration a row for every run of the schedule with the time of the layer
    # in the prompt's step and in a decode step (events around every layer, on the device)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "picolm_b200"), model_dirs["A_sharp"],
                        "-p", "5,6,7,8,9,10", "-n", "6", "--benchmark"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert r.stderr.count("=== iteration") == 3 and r.stderr.count("layer,prefill_ms,gen_ms") == 3
    rows = [ln.split(",") for ln in r.stderr.splitlines() if re.fullmatch(r"\d+,[0-9.]+,[0-9.]+,[0-9.]+,\d+", ln)]
    assert [int(x[0]) for x in rows] == [0, 1] * 3                     # two layers, three iterations
    assert all(float(x[1]) > 0 and float(x[2]) > 0 and float(x[3]) > 0 for x in rows)
    assert r.stderr.count("Prefill: 6 tokens") == 3 and r.stderr.count("Generation: 6 tokens") == 3
    # the per-kernel table: every launch between two events, a row per kind of launch with its time and rates
    env = dict(os.environ, PICOLM_B200_TRACE="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "picolm_b200"), model_dirs["A_sharp"],
                        "-p", "5,6,7,8,9,10", "-n", "4", "-t", "0", "--dtype", "bfloat16"], capture_output=True, text=True,
                       timeout=300, env=env)
    assert r.returncode == 0, r.stderr
    table = [ln for ln in r.stderr.splitlines() if re.match(r"^(gemm|attention|rmsnorm|embed|argmax)", ln)]
    assert any(ln.startswith("gemm_tc_skinny") for ln in table) and any(ln.startswith("attention") for ln in table)
    assert all(float(ln.split()[-6]) > 0 for ln in table)              # every row has a device time
