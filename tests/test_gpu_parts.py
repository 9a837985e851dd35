"""Each part of a layer alone, built from a PartSpec with sizes of its own and
run against the plain implementation's function for that part."""

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _runtime(dtype):
    from picolm_b200.runtime import Runtime
    return Runtime.create(dtype, DEV)


def _step_and_cache(rt, layer_specs, seq_tokens, starts=None):
    """A cache and the StepBatch of sequences that bring `seq_tokens` tokens each."""
    from picolm_b200.cache import SequenceCache
    from picolm_b200.engine.step_batch import build_step_batch
    cache = SequenceCache(layer_specs, max_tokens=64 * 16, max_seqs=4, kv_dtype=rt.dtype, device=rt.device)
    entries = []
    for n in seq_tokens:
        s = cache.allocate()
        entries.append((s, list(range(n))))
    cache.reserve([(s, len(t)) for s, t in entries])
    step = build_step_batch(entries, [[len(t) - 1] for _, t in entries], cache, rt.device)
    return cache, step


def _tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part_folds_the_pending_delta(dtype):
    from picolm_b200.config import PartSpec
    from picolm_b200.parts import ResidualStream, build_part
    rt = _runtime(dtype)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 120, "eps": 3e-4}), rt)
    assert norm.weight_specs()["weight"].shape == (120,)
    w = (1 + 0.2 * torch.randn(120)).to(DT[dtype])
    norm.load({"weight": w.to(DEV)})
    x, delta = torch.randn(6, 120), torch.randn(6, 120)
    stream = ResidualStream(x.to(DEV).clone(), delta.to(DEV))
    h = norm.forward(stream)
    assert stream.pending is None and torch.equal(stream.x.cpu(), x + delta)
    assert h.dtype == DT[dtype]
    assert torch.allclose(h.float().cpu(), P.rmsnorm(x + delta, w.float(), 3e-4), **_tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from picolm_b200 import ops
    from picolm_b200.config import PartSpec
    from picolm_b200.parts import build_part
    rt = _runtime(dtype)
    d, F = 80, 204
    ff = build_part("feed_forward", PartSpec("gated_mlp", {
        "hidden_size": d, "intermediate_size": F, "activation": "silu",
        "gate_name": "g.weight", "up_name": "u.weight", "down_name": "d.weight"}), rt)
    specs = ff.weight_specs()
    assert specs["g.weight"].shape == (F, d) and specs["d.weight"].shape == (d, F)
    w = {n: (torch.randn(s.shape) * 0.1).to(DT[dtype]) for n, s in specs.items()}
    ff.load({n: t.to(DEV) for n, t in w.items()})
    h = torch.randn(11, d).to(DT[dtype])
    out = ff.forward(h.to(DEV), None)
    assert out.dtype == torch.float32
    rnd = (lambda t: t.to(DT[dtype]).float())
    gate, up = rnd(P.linear(h.float(), w["g.weight"].float())), rnd(P.linear(h.float(), w["u.weight"].float()))
    ref = P.linear(rnd(P.swiglu(gate, up)), w["d.weight"].float())
    assert torch.allclose(out.cpu(), ref, **_tol(dtype))
    with pytest.raises(ValueError, match="activation"):
        build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8,
                                                          "activation": "relu"}), rt)
    # the reference's other activation (picolm/tensor.c:3317-3323), through the same part
    gelu = build_part("feed_forward", PartSpec("gated_mlp", {
        "hidden_size": d, "intermediate_size": F, "activation": "gelu_tanh",
        "gate_name": "g.weight", "up_name": "u.weight", "down_name": "d.weight"}), rt)
    gelu.load({n: t.to(DEV) for n, t in w.items()})
    act = 0.5 * gate * (1.0 + torch.tanh(0.79788456 * (gate + 0.044715 * gate ** 3))) * up
    ref_gelu = P.linear(rnd(act), w["d.weight"].float())
    got = gelu.forward(h.to(DEV), None)
    got = got.compute() if hasattr(got, "compute") else got
    assert torch.allclose(got.cpu(), ref_gelu, **_tol(dtype)) and not torch.allclose(ref_gelu, ref, atol=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pairing", ["half", "adjacent"])
def test_attention_part_with_rope_options(dtype, pairing):
    """An attention mixer with sizes and options of its own (partial rotary,
    a scale that is not 1/sqrt(hd), llama3 scaling, two sequences of unequal
    lengths in one step) against the plain parts."""
    from picolm_b200 import ops
    from picolm_b200.config import PartSpec
    from picolm_b200.parts import build_part
    rt = _runtime(dtype)
    d, H, G, hd, rot = 72, 6, 3, 24, 16
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 32}
    pos_spec = PartSpec("rope", {"head_dim": hd, "rotary_dim": rot, "theta": 777.0, "scaling": scaling,
                                 "pairing": pairing, "max_positions": 512})
    mixer = build_part("mixer", PartSpec("attention", {
        "hidden_size": d, "num_heads": H, "num_kv_heads": G, "head_dim": hd, "scale": 0.3, "window": None,
        "position": pos_spec, "q_name": "q", "k_name": "k", "v_name": "v", "o_name": "o"}), rt)
    specs = mixer.weight_specs()
    torch.manual_seed(4)
    w = {n: (torch.randn(s.shape) * 0.15).to(DT[dtype]) for n, s in specs.items()}
    mixer.load({n: t.to(DEV) for n, t in w.items()})
    lens = [40, 9]                                       # few enough rows for the last product to come back unrun
    cache, step = _step_and_cache(rt, [mixer.cache_spec()], lens)
    mixer.prepare(cache.max_seq_tokens)
    from picolm_b200.cache import KVLayerCache
    g = cache.kv_groups[0]
    view = KVLayerCache(g.k[0], g.v[0], step.block_tables[0], None, True)
    h = torch.randn(sum(lens), d).to(DT[dtype])
    out = mixer.forward(h.to(DEV), step, view)
    if dtype == "bfloat16":                              # a delta that the next norm may run (or anyone, by compute())
        assert isinstance(out, ops.PendingLinear)
        out = out.compute()
    out = out.cpu()
    rnd = (lambda t: t.to(DT[dtype]).float())
    cos, sin = P.rope_table(max(lens), rot, 777.0, scaling)
    cos, sin = cos.float(), sin.float()
    ref, o = [], 0
    for n in lens:
        hh = h[o:o + n].float()
        o += n
        q = rnd(P.linear(hh, w["q"].float())).reshape(n, H, hd)
        k = rnd(P.linear(hh, w["k"].float())).reshape(n, G, hd)
        v = rnd(P.linear(hh, w["v"].float())).reshape(n, G, hd)
        q[..., :rot] = P.rope(q[..., :rot].contiguous(), cos, sin, pairing)
        k[..., :rot] = P.rope(k[..., :rot].contiguous(), cos, sin, pairing)
        a = rnd(P.attention(rnd(q), rnd(k), v, 0.3)).reshape(n, H * hd)
        ref.append(P.linear(a, w["o"].float()))
    assert torch.allclose(out, torch.cat(ref), **_tol(dtype))


def test_rope_table_against_plain_in_all_three_llama3_regimes():
    from picolm_b200.parts.position import rope_inverse_frequencies
    scaling = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    ours = torch.tensor(rope_inverse_frequencies(32, 500000.0, scaling), dtype=torch.float64)
    plain = P.rope_frequencies(32, 500000.0, scaling)
    base = P.rope_frequencies(32, 500000.0, None)
    assert torch.allclose(ours, plain, rtol=1e-12, atol=0)
    ratio = (plain / base).tolist()
    assert any(r == 1.0 for r in ratio) and any(abs(r - 0.25) < 1e-12 for r in ratio)
    assert any(0.25 < r < 1.0 for r in ratio)                # kept, divided and blended all occur


def test_embedding_and_head_parts():
    from picolm_b200.config import PartSpec
    from picolm_b200.parts import build_part
    from types import SimpleNamespace
    rt = _runtime("bfloat16")
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 50, "hidden_size": 24, "name": "E"}), rt)
    head = build_part("head", PartSpec("lm_head", {"vocab_size": 50, "hidden_size": 24, "name": "E"}), rt)
    table = torch.randn(50, 24).to(torch.bfloat16)
    emb.load({"E": table.to(DEV)}), head.load({"E": table.to(DEV)})
    toks = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    x = emb.forward(SimpleNamespace(tok_ids=toks))
    assert torch.equal(x.cpu(), table.float()[[3, 49, 0]])
    h = torch.randn(4, 24).to(torch.bfloat16)
    logits = head.forward(h.to(DEV))
    assert logits.dtype == torch.float32
    assert torch.allclose(logits.cpu(), P.linear(h.float(), table.float()), atol=1e-4, rtol=1e-4)
