"""bin/trace_run as a user runs it: a child process fed one JSON line per step,
answering `done <step>`, writing <step>.f32 files.  The same requests are
replayed whole, with the last 32 tokens one by one, and in batches of unequal
lengths (one batch after another, so that slots and pages are used again), in
float32 and in bfloat16, against the plain implementation."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from plain import llama_plain as P
from util import TINY, assert_close, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out_dir = out_dir
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step = 0

    def send(self, entries, end=()):
        rec = {"step": self.step, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step}", f"expected 'done {self.step}', got {line!r}"
        path = os.path.join(self.out_dir, f"{self.step}.f32")
        n_want = sum(len(e["want"]) for e in entries)
        self.step += 1
        if n_want == 0:
            assert not os.path.exists(path)
            return None
        arr = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(arr.reshape(n_want, -1).copy())

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A_sharp", "B_sharp"])
def test_trace_replay_in_every_cut(model_dirs, tmp_path, name, dtype):
    cfg, w = P.load_model(model_dirs[name])
    vocab = TINY[name[0]]["config"]["vocab_size"]
    act = torch.bfloat16 if dtype == "bfloat16" else None
    reqs = {f"r{i}": random_tokens(n, vocab, 200 + i) for i, n in enumerate([40, 75, 33, 100, 36])}
    ref = {k: P.forward(cfg, w, t, act_dtype=act) for k, t in reqs.items()}
    # 4 pages: each batch below fits, but only because what earlier batches held came back
    rp = Replay(model_dirs[name], dtype, str(tmp_path / "out"), max_tokens=256)
    try:
        # 1. each request alone and whole (wanting only some places, in a shuffled order, is allowed)
        for k, t in reqs.items():
            got = rp.send([{"id": k, "tokens": t, "want": list(range(len(t)))}], end=[k])
            assert got.shape == (len(t), vocab)
            assert_close(got, ref[k], dtype, f"{name} {dtype} whole {k}")
        got = rp.send([{"id": "x", "tokens": reqs["r0"], "want": [39, 0, 7]}], end=["x"])
        assert_close(got, ref["r0"][[39, 0, 7]], dtype, "picked places")
        # 2. the last 32 tokens one by one; the prompt step wants nothing
        for k in ("r1", "r2"):
            t = reqs[k]
            head = len(t) - 32
            assert rp.send([{"id": k, "tokens": t[:head], "want": []}]) is None
            rows = []
            for i in range(head, len(t)):
                rows.append(rp.send([{"id": k, "tokens": [t[i]], "want": [0]}], end=[k] if i == len(t) - 1 else []))
            assert_close(torch.cat(rows), ref[k][head:], dtype, f"{name} {dtype} tail {k}")
        # 3. batches of unequal lengths, shorter requests end earlier, batch after batch
        for batch, prompt_lens in ((["r0", "r2", "r4"], [5, 33, 20]), (["r1", "r3"], [70, 64]), (["r4", "r0", "r2"], [1, 2, 3])):
            pos = dict(zip(batch, prompt_lens))
            got = rp.send([{"id": k, "tokens": reqs[k][:pos[k]], "want": list(range(pos[k]))} for k in batch],
                          end=[k for k in batch if pos[k] == len(reqs[k])])
            o = 0
            for k in batch:
                assert_close(got[o:o + pos[k]], ref[k][:pos[k]], dtype, f"{name} {dtype} batch prompt {k}")
                o += pos[k]
            live = [k for k in batch if pos[k] < len(reqs[k])]
            while live:
                ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
                got = rp.send([{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live], end=ending)
                for row, k in enumerate(live):
                    assert_close(got[row:row + 1], ref[k][pos[k]:pos[k] + 1], dtype,
                                 f"{name} {dtype} batch decode {k} at {pos[k]}")
                    pos[k] += 1
                live = [k for k in live if pos[k] < len(reqs[k])]
    finally:
        rp.close()
