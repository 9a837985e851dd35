"""The C API (picolm_b200/capi/plm.h) from a C program: tests/capi/plm_demo.c is compiled against
libplm.so and run as a process of its own.  Without a GPU: the configuration through the registry and an
error with its text.  On the GPU: BASELINE's Tiny-A workload through plm_step (three unequal prompts in
one step, then eight tokens each) against the plain implementation in float32, and plm_generate against
the plain implementation's greedy tokens."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from util import TINY, assert_close

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def demo(tmp_path_factory):
    from picolm_b200.capi import build_library, include_dir, python_link_flags
    lib = build_library()
    exe = str(tmp_path_factory.mktemp("capi") / "plm_demo")
    cmd = ["gcc", "-O1", "-std=c11", os.path.join(ROOT, "tests", "capi", "plm_demo.c"), f"-I{include_dir()}",
           f"-L{os.path.dirname(lib)}", "-lplm", f"-Wl,-rpath,{os.path.dirname(lib)}", "-o", exe] + python_link_flags()
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_config_and_errors_from_c(demo, model_dirs):
    r = subprocess.run([demo, "config", model_dirs["B"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    cfg = json.loads(r.stdout)
    want = TINY["B"]["config"]
    assert cfg["num_key_value_heads"] == want["num_key_value_heads"] and cfg["head_dim"] == want["head_dim"]
    assert cfg["rope_scaling"]["factor"] == 4.0 and cfg["eos_token_id"] == [3, 4]
    r = subprocess.run([demo, "missing", os.path.join(model_dirs["B"], "nothing-here")], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    code, _, text = r.stdout.strip().partition(" ")
    assert int(code) != 0 and "nothing-here" in text


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_step_and_generate_from_c(demo, model_dirs, tmp_path, dtype):
    from plain import llama_plain as P
    d = model_dirs["A_sharp"]
    out = str(tmp_path / "logits.f32")
    r = subprocess.run([demo, "run", d, dtype, out], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    cfg, w = P.load_model(d)
    vocab = cfg["vocab_size"]
    got = torch.from_numpy(np.fromfile(out, dtype=np.float32).reshape(33 + 24, vocab))
    lens = [5, 11, 17]
    seqs = [[(7 * s + 3 * t + 1) % vocab for t in range(n + 8)] for s, n in enumerate(lens)]
    act = torch.bfloat16 if dtype == "bfloat16" else None
    refs = [P.forward(cfg, w, seq, act_dtype=act) for seq in seqs]
    assert_close(got[:33], torch.cat([ref[:n] for ref, n in zip(refs, lens)]), dtype, "prompts through plm_step")
    decoded = torch.stack([refs[s][lens[s] + step] for step in range(8) for s in range(3)])
    assert_close(got[33:], decoded, dtype, "one token each through plm_step")
    tokens = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    if dtype == "float32":
        assert tokens == [P.greedy(cfg, w, seq[:n], 6) for seq, n in zip(seqs, lens)]
    else:
        assert [len(t) for t in tokens] == [6, 6, 6]
