"""The plain implementation itself (no device): against logits that
whoreson/picolm's own CPU code produced (tests/golden, made by
tests/golden/make_golden.py), and its parts against hand-computed values."""
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import llama_plain as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _weights(case):
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors
    return {k: v.float() for k, v in random_tensors(config_from_dict(case["config"]), case["seed"]).items()}


@pytest.mark.parametrize("name", ["tiny_a_half", "tiny_a_adjacent", "tiny_b_llama3"])
def test_plain_matches_the_reference_code(name):
    """The reference keeps K and V as fp16; with the same rounding the plain
    implementation agrees with it to float32 accuracy, at every position, for
    both pairings and with the injected llama3 table."""
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        case = json.load(f)
    cfg, toks = case["config"], case["tokens"]
    ref = torch.from_numpy(np.fromfile(os.path.join(GOLDEN, name + ".f32"), dtype="<f4").reshape(len(toks) + 1, -1).copy())
    step_by_step, prefill_last = ref[:-1], ref[-1]
    assert torch.equal(step_by_step[-1], prefill_last)           # the reference's two entry points agree exactly
    w = _weights(case)
    got = P.forward(cfg, w, toks, pairing=case["pairing"], kv_dtype=torch.float16)
    err = (got - step_by_step).abs().max().item()
    assert err < 5e-6, f"max |diff| {err:.2e}"
    # without the fp16 rounding the difference is the rounding's size, not more
    exact = P.forward(cfg, w, toks, pairing=case["pairing"])
    assert 0 < (exact - step_by_step).abs().max().item() < 2e-3
    # the other pairing gives other logits: the golden files tell the two apart
    other = P.forward(cfg, w, toks, pairing="adjacent" if case["pairing"] == "half" else "half", kv_dtype=torch.float16)
    assert (other - step_by_step).abs().max().item() > 1e-3


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    out = P.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.5)            # mean square 12.5, + eps = 13
    assert torch.allclose(out, torch.tensor([[6.0, 2.0]]) / math.sqrt(13.0))


def test_rope_pairings_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]]).repeat(2, 1, 1)
    cos, sin = P.rope_table(2, 4, 10000.0, None)
    half, adj = P.rope(x, cos, sin, "half"), P.rope(x, cos, sin, "adjacent")
    assert torch.equal(half[0], x[0]) and torch.equal(adj[0], x[0])              # position 0: no rotation
    c0, s0, c1, s1 = math.cos(1.0), math.sin(1.0), math.cos(0.01), math.sin(0.01)
    assert torch.allclose(half[1, 0], torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1]))
    assert torch.allclose(adj[1, 0], torch.tensor([1 * c0 - 2 * s0, 1 * s0 + 2 * c0, 3 * c1 - 4 * s1, 3 * s1 + 4 * c1]))


def test_llama3_scaling_regimes():
    sc = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base, scaled = P.rope_frequencies(32, 500000.0, None), P.rope_frequencies(32, 500000.0, sc)
    wl = 2 * math.pi / base
    for i in range(16):
        if wl[i] < 16:
            assert scaled[i] == base[i]
        elif wl[i] > 64:
            assert scaled[i] == base[i] / 4
        else:
            assert base[i] / 4 < scaled[i] < base[i]
    assert (wl < 16).any() and (wl > 64).any() and ((wl >= 16) & (wl <= 64)).any()


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    out = P.attention(q, k, v, 0.35)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[4], v2[4] = 9.0, 9.0                                                            # the future does not leak
    assert torch.equal(P.attention(q, k2, v2, 0.35)[:4], out[:4])
    # one row by the reference's running-max recurrence (picolm/model_attention.c:43-140)
    m, l, acc = -1e30, 0.0, torch.zeros(8)
    for t in range(4):
        s = float(q[3, 2] @ k[t, 1]) * 0.35
        if s > m:
            c = math.exp(m - s)
            l, acc, m = l * c + 1.0, acc * c + v[t, 1], s
        else:
            wgt = math.exp(s - m)
            l, acc = l + wgt, acc + wgt * v[t, 1]
    assert torch.allclose(out[3, 2], acc / l, atol=1e-6)
    win = P.attention(q, k, v, 0.35, window=2)
    assert torch.allclose(win[1], out[1]) and not torch.allclose(win[4], out[4])


def test_sampler_chain_by_hand():
    logits = torch.log(torch.tensor([0.5, 0.2, 0.15, 0.1, 0.05]))
    kept, w = P.sampling_weights(logits, 1.0, 0, 1.0, 0.0)
    assert kept == [0, 1, 2, 3, 4] and torch.allclose(w, torch.tensor([0.5, 0.2, 0.15, 0.1, 0.05]), atol=1e-6)
    assert P.sampling_weights(logits, 1.0, 2, 1.0, 0.0)[0] == [0, 1]                   # top-k
    assert P.sampling_weights(logits, 1.0, 0, 0.8, 0.0)[0] == [0, 1, 2]                # top-p: 0.5+0.2+0.15 >= 0.8
    assert P.sampling_weights(logits, 1.0, 0, 1.0, 0.25)[0] == [0, 1, 2]               # min-p: p >= 0.125
    kept, w = P.sampling_weights(logits, 0.5, 2, 1.0, 0.0)                             # p^(1/T) renormalised
    assert torch.allclose(w, torch.tensor([0.25, 0.04]) / 0.29, atol=1e-6)
    assert P.argmax(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    state, x = P.xorshift64(42)
    assert x == 45454805674 and P.rand_float(42)[1] == pytest.approx((45454805674 >> 11) / 2.0 ** 53)
    # both draw orders pick from the kept set and follow the same stream
    s1, a = P.sample_reference_order(logits, 1.0, 3, 1.0, 0.0, 7)
    s2, b = P.sample_index_order(logits, 1.0, 3, 1.0, 0.0, 7)
    assert s1 == s2 and a in (0, 1, 2) and b in (0, 1, 2)


def test_llama3_rule_on_the_tiny_configuration_by_hand():
    """The scaling rule on Tiny B's numbers (theta 500000, head size 32, factor 4, low 1, high 4, original
    context 64), against values worked out by hand from the published rule rather than by either
    implementation: the 16 wavelengths 2 pi theta^(i/16) start 6.28, 14.27, 32.40, 73.58; 6.28 and 14.27 lie
    below 64/4 = 16 and are kept; 73.58 and all later ones lie above 64/1 and are divided by 4; 32.40 lies
    between: smooth = (64/32.40 - 1) / (4 - 1) = 0.3251, so the frequency becomes
    (0.6749 / 4 + 0.3251) f = 0.49382 f.  The library's function (which builds the kernels' tables) must give
    the same as the plain one.  (No installed package's implementation of the rule is used as a mark: the
    packages' model code is not a source for this library.)"""
    from picolm_b200.parts.position import rope_inverse_frequencies
    sc = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    plain = P.rope_frequencies(32, 500000.0, sc)
    mine = torch.tensor(rope_inverse_frequencies(32, 500000.0, sc), dtype=torch.float64)
    assert torch.allclose(plain.double(), mine, rtol=1e-12, atol=0)
    base = [500000.0 ** (-i / 16.0) for i in range(16)]
    wl = [2 * math.pi / f for f in base]
    assert [round(x, 2) for x in wl[:4]] == [6.28, 14.27, 32.40, 73.58]
    ratio = [float(mine[i]) / base[i] for i in range(16)]
    assert ratio[0] == 1.0 and ratio[1] == 1.0
    smooth = (64.0 / wl[2] - 1.0) / 3.0
    assert smooth == pytest.approx(0.3251, abs=5e-5)
    assert ratio[2] == pytest.approx((1.0 - smooth) / 4.0 + smooth, rel=1e-12) and ratio[2] == pytest.approx(0.49382, abs=5e-6)
    assert all(r == pytest.approx(0.25, rel=1e-12) for r in ratio[3:])
    # the shapes the benchmarks use: every frequency is kept, divided by the factor, or in between, and the
    # rule is monotone (a longer wavelength is never scaled less)
    for hd, theta, factor, L0 in ((64, 500000.0, 32.0, 8192), (128, 500000.0, 8.0, 8192)):
        s = {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
             "original_max_position_embeddings": L0}
        a = rope_inverse_frequencies(hd, theta, None)
        b = rope_inverse_frequencies(hd, theta, s)
        r = [y / x for x, y in zip(a, b)]
        assert r[0] == 1.0 and r[-1] == pytest.approx(1.0 / factor) and all(r[i + 1] <= r[i] + 1e-15 for i in range(len(r) - 1))
        assert torch.allclose(P.rope_frequencies(hd, theta, s).double(), torch.tensor(b, dtype=torch.float64), rtol=1e-12, atol=0)


def test_the_draw_order_is_not_the_reference_s():
    """The engine's sampler walks the kept tokens in index order, the reference in descending probability
    (picolm/sampler.c:112-121): the same distribution, but not the same token for the same seed.  This case
    shows the difference, so that nobody reads the sampler's description as a promise of equal tokens."""
    logits = torch.log(torch.tensor([0.1, 0.2, 0.7]))
    s1, a = P.sample_reference_order(logits, 1.0, 0, 1.0, 0.0, 1)
    s2, b = P.sample_index_order(logits, 1.0, 0, 1.0, 0.0, 1)
    assert s1 == s2 and (a, b) == (2, 0)
