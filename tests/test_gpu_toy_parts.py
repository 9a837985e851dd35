"""Two more toy parts, defined here and registered without touching a file of the
library: a feed-forward that routes every token to one of several experts, and a
position encoding that is not a rotation.  A toy architecture uses them in one
layer and the library's own parts in another; its logits are compared with a plain
computation written out in this file, whole, token by token and in batches."""
import dataclasses
import math

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu


def _wave(pos: torch.Tensor, head_dim: int) -> torch.Tensor:
    """The toy position encoding: a factor 1 + 0.5 sin(pos / (1 + i)) on component i of every query and key."""
    i = torch.arange(head_dim, device=pos.device, dtype=torch.float32)
    return 1.0 + 0.5 * torch.sin(pos.to(torch.float32)[:, None] / (1.0 + i)[None, :])


def _register():
    from picolm_b200 import ops, register_architecture, register_part
    from picolm_b200.config import ModelSpec, PartSpec
    from picolm_b200.parts.block import pre_norm_layer
    from picolm_b200.parts import Part, WeightSpec

    @register_part("feed_forward", "toy_routed")
    class Routed(Part):
        """params: hidden_size, intermediate_size, experts.  Each token goes to the expert whose router
        logit is largest; its output is weighted by the softmax probability of that expert."""

        def weight_specs(self):
            d, f, e = self.params["hidden_size"], self.params["intermediate_size"], self.params["experts"]
            specs = {"router.weight": WeightSpec((e, d))}
            for x in range(e):
                specs[f"experts.{x}.up.weight"] = WeightSpec((f, d))
                specs[f"experts.{x}.down.weight"] = WeightSpec((d, f))
            return specs

        def load(self, tensors):
            e = self.params["experts"]
            self.router = tensors["router.weight"]
            self.up = [tensors[f"experts.{x}.up.weight"] for x in range(e)]
            self.down = [tensors[f"experts.{x}.down.weight"] for x in range(e)]

        def forward(self, h, step):
            logits = ops.linear(h, self.router, torch.float32)                   # router logits in 32-bit
            prob = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)
            out = torch.zeros((h.shape[0], self.params["hidden_size"]), dtype=torch.float32, device=h.device)
            for x in range(self.params["experts"]):
                rows = torch.nonzero(choice == x).flatten()
                if rows.numel() == 0:
                    continue
                hx = h.index_select(0, rows).contiguous()
                mid = torch.relu(ops.linear(hx, self.up[x], h.dtype))
                out.index_copy_(0, rows, ops.linear(mid, self.down[x], torch.float32) * prob[rows, x][:, None])
            return out

    @register_part("position", "toy_wave")
    class Wave(Part):
        """Queries and keys are multiplied by a factor that depends on position and component."""

        def prepare(self, n_positions: int) -> None:
            pass

        def apply(self, qkv, q_out, kv, step, num_heads, num_kv_heads, head_dim) -> None:
            T = qkv.shape[0]
            f = _wave(step.tok_pos, head_dim)                                    # [T, hd]
            heads = qkv.view(T, num_heads + 2 * num_kv_heads, head_dim).float()
            heads[:, :num_heads + num_kv_heads] *= f[:, None, :]                 # queries and keys, not values
            scaled = heads.to(qkv.dtype).view(T, -1).contiguous()
            ops.rope_store(scaled, q_out, kv.k, kv.v, None, None, step.tok_pos, step.tok_seq, kv.block_table,
                           num_heads, num_kv_heads, head_dim, 0, "half", store=kv.writable)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        architecture: str = "ToyRoutedForCausalLM"

        @staticmethod
        def from_dict(d):
            return ToyConfig(d["vocab_size"], d["hidden_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}

    def toy_spec(cfg):
        d = cfg.hidden_size
        norm = {"size": d, "eps": 1e-5}

        def attn(position):
            return PartSpec("attention", {"hidden_size": d, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                          "scale": None, "window": None, "position": position,
                                          "q_name": "q.weight", "k_name": "k.weight", "v_name": "v.weight",
                                          "o_name": "o.weight"}, prefix="attn")

        routed = PartSpec("toy_routed", {"hidden_size": d, "intermediate_size": 40, "experts": 3}, prefix="moe")
        dense = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": 2 * d, "activation": "silu",
                                       "gate_name": "gate.weight", "up_name": "up.weight", "down_name": "down.weight"},
                         prefix="ff")
        rope = PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "scaling": None,
                                 "pairing": "half", "max_positions": 256})

        def layer(i, mixer, ff):
            return pre_norm_layer(f"blocks.{i}", mixer, ff, PartSpec("rmsnorm", norm, prefix="n1"),
                             PartSpec("rmsnorm", norm, prefix="n2"))

        return ModelSpec(
            architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "emb.weight"}),
            layers=(layer(0, attn(PartSpec("toy_wave")), routed), layer(1, attn(rope), dense)), schedule=(0, 1),
            final_norm=PartSpec("rmsnorm", norm, prefix="final"),
            lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "head.weight"}),
            max_positions=256, stop_token_ids=(0,))

    register_architecture("ToyRoutedForCausalLM", ToyConfig.from_dict, toy_spec)
    return ToyConfig


def _plain_logits(w, tokens):
    """The toy model, whole sequence, no cache: the same formulas with the plain implementation's parts."""
    T, H, G, hd, eps = len(tokens), 4, 2, 16, 1e-5
    pos = torch.arange(T)
    x = P.embed(tokens, w["emb.weight"])
    routed_rows = []
    for l in range(2):
        p = f"blocks.{l}."
        h = P.rmsnorm(x, w[p + "n1.weight"], eps)
        q = P.linear(h, w[p + "attn.q.weight"]).reshape(T, H, hd)
        k = P.linear(h, w[p + "attn.k.weight"]).reshape(T, G, hd)
        v = P.linear(h, w[p + "attn.v.weight"]).reshape(T, G, hd)
        if l == 0:
            f = _wave(pos, hd)
            q, k = q * f[:, None, :], k * f[:, None, :]
        else:
            cos, sin = P.rope_table(T, hd, 10000.0, None)
            q, k = P.rope(q, cos.float(), sin.float(), "half"), P.rope(k, cos.float(), sin.float(), "half")
        a = P.attention(q, k, v, 1.0 / math.sqrt(hd)).reshape(T, H * hd)
        x = x + P.linear(a, w[p + "attn.o.weight"])
        h = P.rmsnorm(x, w[p + "n2.weight"], eps)
        if l == 0:
            logits = P.linear(h, w[p + "moe.router.weight"])
            prob = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)
            routed_rows = choice.tolist()
            out = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                mid = torch.relu(P.linear(h[t:t + 1], w[p + f"moe.experts.{e}.up.weight"]))
                out[t] = P.linear(mid, w[p + f"moe.experts.{e}.down.weight"])[0] * prob[t, e]
            x = x + out
        else:
            x = x + P.linear(P.swiglu(P.linear(h, w[p + "ff.gate.weight"]), P.linear(h, w[p + "ff.up.weight"])),
                             w[p + "ff.down.weight"])
    return P.linear(P.rmsnorm(x, w["final.weight"], eps), w["head.weight"]), routed_rows


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    import os
    from harness import run_batch, run_tail, run_whole
    from picolm_b200.engine import Engine
    from picolm_b200.weights import write_random_model
    from util import random_tokens
    ToyConfig = _register()
    d = write_random_model(ToyConfig(vocab_size=120, hidden_size=48), 11, str(tmp_path / "toy"), std=0.25)
    w = {k: v.float() for k, v in P.read_safetensors(os.path.join(d, "model.safetensors")).items()}
    a, b, c = random_tokens(70, 120, 5), random_tokens(33, 120, 6), random_tokens(9, 120, 7)
    ref = {}
    for name, toks in (("a", a), ("b", b), ("c", c)):
        ref[name], routes = _plain_logits(w, toks)
        if name == "a":
            assert len(set(routes)) == 3                      # every expert gets tokens
    eng = Engine.from_folder(d, dtype="float32", max_tokens=64 * 8, max_seqs=4)
    assert torch.allclose(run_whole(eng, a), ref["a"], atol=3e-5)
    assert torch.allclose(run_tail(eng, b, tail=32), ref["b"], atol=3e-5)
    outs = run_batch(eng, [c, a, b], [3, 40, 11])
    for got, name in zip(outs, "cab"):
        assert torch.allclose(got, ref[name], atol=3e-5)
    eng.cache.check()
    # the same model in bfloat16 runs (the toy parts take whatever dtype the run has) and stays near
    eng16 = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8, max_seqs=4)
    got16 = run_whole(eng16, a)
    assert torch.isfinite(got16).all()
    assert (got16 - ref["a"]).abs().max() < 0.25 * ref["a"].std()
