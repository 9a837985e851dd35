"""The kernels' safety nets, made to act: a bounded wait that runs out (the kernel returns, the status word
says where, the next kernel runs as if nothing had happened), and the checked build of the kernels that walk
page tables (a page number, position or row outside its bounds is recorded and replaced, not followed)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_wait_that_runs_out_is_reported_not_hung():
    """A test build of the decode-shaped product (short wait limit, a switch that makes the producer announce
    more bytes than it loads): with the switch on no stage of the ring ever fills, every wait of the kernel
    runs out, the kernel returns, and `check_status` raises; with the switch off again the same library gives
    the right product."""
    from picolm_b200 import ops
    from picolm_b200.csrc.build import load_library
    lib = load_library("gemm_tc_skinny@stall", ["-DPLM_WAIT_LIMIT=20000", "-DPLM_TEST_STALL"])
    vp, i, l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
    lib.plm_gemm_tc_skinny.argtypes = [vp, vp, vp, i, i, i, i, i, l, l, l, vp, vp]
    lib.plm_test_stall.argtypes = [i, vp]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    T, F, K = 8, 512, 1024
    torch.manual_seed(3)
    x = (torch.randn(T, K) / K ** 0.25).to(torch.bfloat16).to(DEV)
    w = (torch.randn(F, K) / K ** 0.25).to(torch.bfloat16).to(DEV)
    out = torch.zeros((T, F), dtype=torch.float32, device=DEV)
    status = ops.status_word(DEV)
    ops.check_status(DEV)                                        # clean before the test

    def product():
        return lib.plm_gemm_tc_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, 0, T, F, K, K, K, F,
                                      status.data_ptr(), stream)

    assert lib.plm_test_stall(1, stream) == 0
    assert product() == 0                                        # launched; it gives up on the device
    torch.cuda.synchronize()                                     # ... and returns
    assert int(status.item()) in (1, 2, 3)
    with pytest.raises(ops.KernelError, match="gave up waiting"):
        ops.check_status(DEV)
    ops.check_status(DEV)                                        # reading the status cleared it
    assert lib.plm_test_stall(0, stream) == 0
    assert product() == 0
    torch.cuda.synchronize()
    ops.check_status(DEV)
    ref = x.double().cpu() @ w.double().cpu().t()
    assert torch.allclose(out.double().cpu(), ref, atol=2e-3, rtol=1e-4)


CHECKED_SCRIPT = r'''
import os, sys, json
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import torch
from picolm_b200 import ops
from picolm_b200.ops import _lib
assert _lib.CHECKED
from picolm_b200.engine import Engine
from harness import run_batch, run_tail, run_whole
from plain import llama_plain as P
from util import assert_close, random_tokens
out = {}
# 1. the tiny models through the checked kernels, in both precisions and every cut: nothing is out of bounds
for d, vocab in ((sys.argv[2], 256), (sys.argv[3], 384)):
    cfg, w = P.load_model(d)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 12, max_seqs=4)
        a, b = random_tokens(100, vocab, 1), random_tokens(41, vocab, 2)
        act = torch.bfloat16 if dtype == "bfloat16" else None
        ra, rb = P.forward(cfg, w, a, act_dtype=act), P.forward(cfg, w, b, act_dtype=act)
        assert_close(run_whole(eng, a), ra, dtype, "whole")
        assert_close(run_tail(eng, b, tail=32), rb, dtype, "tail")
        for got, ref in zip(run_batch(eng, [a, b], [70, 5]), (ra, rb)):
            assert_close(got, ref, dtype, "batch")
        ops.check_status()
out["models"] = "clean"
# 2. a page table with a page number beyond the cache's pages (the tensors below have room to spare, so
#    that nothing could leave allocated memory even if the check did not act): recorded, not followed
G, hd, H = 2, 16, 4
cache_k = torch.randn(8, G, 64, hd, device="cuda")
cache_v = torch.randn(8, G, 64, hd, device="cuda")
q = torch.randn(1, H, hd, device="cuda")
pos = torch.tensor([70], dtype=torch.int32, device="cuda")
seq = torch.zeros(1, dtype=torch.int32, device="cuda")
good = torch.tensor([[1, 2, 0, 0]], dtype=torch.int32, device="cuda")
ops.attention_rows(q, cache_k[:5], cache_v[:5], pos, seq, good, G, 0.25)
torch.cuda.synchronize(); ops.check_status()
bad = torch.tensor([[1, 6, 0, 0]], dtype=torch.int32, device="cuda")          # page 6 of a cache of 5 pages
ops.attention_rows(q, cache_k[:5], cache_v[:5], pos, seq, bad, G, 0.25)
torch.cuda.synchronize()
try:
    ops.check_status()
    out["bad_page"] = "missed"
except ops.KernelError as e:
    out["bad_page"] = str(e)
far = torch.tensor([300], dtype=torch.int32, device="cuda")                   # position 300 of a table of 4 pages
ops.attention_rows(q, cache_k[:5], cache_v[:5], far, seq, good, G, 0.25)
torch.cuda.synchronize()
try:
    ops.check_status()
    out["bad_position"] = "missed"
except ops.KernelError as e:
    out["bad_position"] = str(e)
print(json.dumps(out))
'''


def test_the_checked_build_runs_clean_and_catches_a_bad_page(model_dirs):
    """A process of its own with PICOLM_B200_CHECK=1: the page-walking kernels are compiled with their
    bounds checks, the tiny models run through them in every cut with a clean status word, and a page number
    and a position outside their bounds are reported instead of followed."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PICOLM_B200_CHECK="1")
    r = subprocess.run([sys.executable, "-c", CHECKED_SCRIPT, root, model_dirs["A_sharp"], model_dirs["B_sharp"]],
                       capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["models"] == "clean"
    assert "page number outside its bounds" in out["bad_page"]
    assert "position outside its bounds" in out["bad_position"]
