"""Another arrangement and a mixer with state that captured steps can run, defined here and registered
without touching a file of the library.  The arrangement has four norms a layer (one before and one after
each of mixer and feed-forward); the mixer keeps a decaying sum of its inputs per sequence and reaches its
state through the step's device buffers only, so decode steps are replayed from CUDA graphs.  A toy
architecture uses both; its logits are compared with a plain computation written out in this file: whole,
with the last 32 tokens one by one, and in batches of unequal lengths whose rows of padding must not touch
a live sequence's state."""
import dataclasses
import math
import os

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu

DECAY = 0.75


def _register():
    from picolm_b200 import register_architecture, register_part
    from picolm_b200.cache import CacheSpec
    from picolm_b200.config import LayerSpec, ModelSpec, PartSpec
    from picolm_b200.parts import Part, ResidualStream, WeightSpec
    from picolm_b200.parts.block import Arrangement

    @register_part("arrangement", "toy_four_norms")
    class FourNorms(Arrangement):
        """x += norm_out_a(mixer(norm_in_a(x))); x += norm_out_b(feed_forward(norm_in_b(x)))."""
        wants = ("norm_in_a", "mixer", "norm_out_a", "norm_in_b", "feed_forward", "norm_out_b")

        def forward(self, stream, step, caches):
            h = self.norm_in_a.forward(stream)
            stream.pending = self._after(self.norm_out_a, self.mixer.forward(h, step, caches[0]))
            h = self.norm_in_b.forward(stream)
            stream.pending = self._after(self.norm_out_b, self.feed_forward.forward(h, step))

        @staticmethod
        def _after(norm, delta):
            if hasattr(delta, "compute"):                       # a product handed back unrun
                delta = delta.compute()
            return norm.forward(ResidualStream(delta)).float()

    @register_part("mixer", "toy_decaying_sum")
    class DecayingSum(Part):
        """s_t = DECAY * s_(t-1) + x_t per sequence, out_t = W s_t.  The state s lives in the cache."""
        graph_safe = True

        def weight_specs(self):
            d = self.params["hidden_size"]
            return {"mix.weight": WeightSpec((d, d))}

        def load(self, tensors):
            self.w = tensors["mix.weight"].float()

        def cache_spec(self):
            return CacheSpec.state((self.params["hidden_size"],))

        def forward(self, h, step, cache):
            x = h.float()
            if step.is_decode:
                # one token per sequence; the sequences' slots are read from the device, so a captured
                # step follows whatever batch it is replayed for
                idx = step.seq_slot_long
                s = cache.state.index_select(0, idx) * DECAY + x
                cache.state.index_copy_(0, idx, s)
                return s @ self.w.t()
            out = torch.empty_like(x)
            o = 0
            for slot, n in zip(step.slots, step.new_lens):
                s = cache.state[slot].clone()
                for t in range(n):
                    s = s * DECAY + x[o + t]
                    out[o + t] = s
                cache.state[slot] = s
                o += n
            return out @ self.w.t()

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        architecture: str = "ToyFourNormsForCausalLM"

        @staticmethod
        def from_dict(d):
            return ToyConfig(d["vocab_size"], d["hidden_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}

    def toy_spec(cfg):
        d = cfg.hidden_size
        norm = {"size": d, "eps": 1e-5}
        ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": 2 * d, "activation": "silu",
                                    "gate_name": "gate.weight", "up_name": "up.weight", "down_name": "down.weight"},
                      prefix="ff")
        rope = PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "scaling": None,
                                 "pairing": "half", "max_positions": 256})
        attn = PartSpec("attention", {"hidden_size": d, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                      "scale": None, "window": None, "position": rope,
                                      "q_name": "q.weight", "k_name": "k.weight", "v_name": "v.weight",
                                      "o_name": "o.weight"}, prefix="attn")
        decay = PartSpec("toy_decaying_sum", {"hidden_size": d}, prefix="sum")

        def layer(i, mixer):
            n = {name: ("norm", PartSpec("rmsnorm", norm, prefix=name))
                 for name in ("norm_in_a", "norm_out_a", "norm_in_b", "norm_out_b")}
            return LayerSpec(f"blocks.{i}", "toy_four_norms",
                             dict(n, mixer=("mixer", mixer), feed_forward=("feed_forward", ff)))

        return ModelSpec(
            architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "emb.weight"}),
            layers=(layer(0, decay), layer(1, attn)), schedule=(0, 1),
            final_norm=PartSpec("rmsnorm", norm, prefix="final"),
            lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "head.weight"}),
            max_positions=256, stop_token_ids=(0,))

    register_architecture("ToyFourNormsForCausalLM", ToyConfig.from_dict, toy_spec)
    return ToyConfig


def _plain_logits(w, tokens):
    """The toy model, whole sequence, no cache, with the plain implementation's parts."""
    T, H, G, hd, eps = len(tokens), 4, 2, 16, 1e-5
    x = P.embed(tokens, w["emb.weight"])
    for l in range(2):
        p = f"blocks.{l}."
        h = P.rmsnorm(x, w[p + "norm_in_a.weight"], eps)
        if l == 0:
            s, rows = torch.zeros(x.shape[1]), []
            for t in range(T):
                s = s * DECAY + h[t]
                rows.append(s)
            delta = P.linear(torch.stack(rows), w[p + "sum.mix.weight"])
        else:
            q = P.linear(h, w[p + "attn.q.weight"]).reshape(T, H, hd)
            k = P.linear(h, w[p + "attn.k.weight"]).reshape(T, G, hd)
            v = P.linear(h, w[p + "attn.v.weight"]).reshape(T, G, hd)
            cos, sin = P.rope_table(T, hd, 10000.0, None)
            q, k = P.rope(q, cos.float(), sin.float(), "half"), P.rope(k, cos.float(), sin.float(), "half")
            delta = P.linear(P.attention(q, k, v, 1.0 / math.sqrt(hd)).reshape(T, H * hd), w[p + "attn.o.weight"])
        x = x + P.rmsnorm(delta, w[p + "norm_out_a.weight"], eps)
        h = P.rmsnorm(x, w[p + "norm_in_b.weight"], eps)
        delta = P.linear(P.swiglu(P.linear(h, w[p + "ff.gate.weight"]), P.linear(h, w[p + "ff.up.weight"])),
                         w[p + "ff.down.weight"])
        x = x + P.rmsnorm(delta, w[p + "norm_out_b.weight"], eps)
    return P.linear(P.rmsnorm(x, w["final.weight"], eps), w["head.weight"])


def test_four_norms_and_a_state_mixer_under_graphs(tmp_path):
    from harness import run_batch, run_tail, run_whole
    from picolm_b200.engine import Engine
    from picolm_b200.weights import write_random_model
    from util import assert_close, random_tokens
    ToyConfig = _register()
    d = write_random_model(ToyConfig(vocab_size=110, hidden_size=48), 17, str(tmp_path / "toy"), std=0.25)
    w = {k: v.float() for k, v in P.read_safetensors(os.path.join(d, "model.safetensors")).items()}
    assert sum(name.startswith("blocks.0.norm_") for name in w) == 4                # four norms a layer
    a, b, c = random_tokens(70, 110, 5), random_tokens(45, 110, 6), random_tokens(34, 110, 7)
    ref = {name: _plain_logits(w, toks) for name, toks in (("a", a), ("b", b), ("c", c))}
    eng = Engine.from_folder(d, dtype="float32", max_tokens=64 * 8, max_seqs=5)
    assert eng.use_graphs                                                        # every part said graph_safe
    assert sorted(eng.cache.state) == [0] and sorted(eng.cache.layer_group) == [1]
    assert torch.allclose(run_whole(eng, a), ref["a"], atol=3e-5)
    assert torch.allclose(run_tail(eng, b, tail=32), ref["b"], atol=3e-5)
    assert eng._graphs                                                           # the tail ran from a captured step
    # three sequences in a captured step of four rows: the row of padding has a state row of its own, so
    # slot 0 (a live sequence) keeps its sum; a and b go on after c has left
    outs = run_batch(eng, [c, a, b], [3, 40, 11])
    for got, name in zip(outs, "cab"):
        assert torch.allclose(got, ref[name], atol=3e-5), name
    assert 4 in {k[0] for k in eng._graphs}
    # the same slots again, from zeroed state
    outs = run_batch(eng, [b, c], [20, 2])
    assert torch.allclose(outs[0], ref["b"], atol=3e-5) and torch.allclose(outs[1], ref["c"], atol=3e-5)
    eng.cache.check()
    # in bfloat16, steps from graphs and steps launched kernel by kernel agree
    both = []
    for graphs in (True, False):
        e16 = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8, max_seqs=5, use_graphs=graphs)
        both.append(torch.cat(run_batch(e16, [c, a, b], [3, 40, 11])))
        assert bool(e16._graphs) == graphs
    assert_close(both[0], both[1], "bfloat16", "four norms, graphs against plain launches")
