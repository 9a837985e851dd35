"""A toy mixer with state of its own, and a toy architecture around it, are
defined here, registered, built, loaded and stepped without touching a file of
the library.  The toy keeps a running sum of its inputs per sequence (a fixed-size
state) and lets every token see the mean so far; one layer of the toy model uses
it, another uses the library's attention, the schedule runs that layer twice, and
a last layer reads the attention layer's cache instead of owning one."""
import dataclasses
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _register():
    from picolm_b200 import register_architecture, register_part
    from picolm_b200.cache import CacheSpec
    from picolm_b200.config import ModelSpec, PartSpec
    from picolm_b200.parts.block import pre_norm_layer
    from picolm_b200.parts import Part, WeightSpec

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Part):
        def weight_specs(self):
            d = self.params["hidden_size"]
            return {"mix.weight": WeightSpec((d, d))}

        def load(self, tensors):
            self.w = tensors["mix.weight"].float()

        def cache_spec(self):
            return CacheSpec.state((self.params["hidden_size"] + 1,))      # running sum and count

        def forward(self, h, step, cache):
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            o = 0
            for slot, n in zip(step.slots, step.new_lens):                 # tokens of a sequence in order
                st = cache.state[slot]
                x = h[o:o + n].float()
                sums = st[:-1] + torch.cumsum(x, dim=0)
                counts = st[-1] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                out[o:o + n] = (sums / counts[:, None]) @ self.w.t()
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
                o += n
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        architecture: str = "ToyForCausalLM"

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
        toy = PartSpec("toy_running_mean", {"hidden_size": d}, prefix="toy")
        attn = PartSpec("attention", {"hidden_size": d, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                      "scale": None, "window": None, "position": PartSpec("none"),
                                      "q_name": "q.weight", "k_name": "k.weight", "v_name": "v.weight",
                                      "o_name": "o.weight"}, prefix="attn")

        def layer(i, mixer, cache_of=None):
            return pre_norm_layer(f"blocks.{i}", mixer, ff, PartSpec("rmsnorm", norm, prefix="n1"),
                             PartSpec("rmsnorm", norm, prefix="n2"), cache_of=cache_of)

        return ModelSpec(
            architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "emb.weight"}),
            # layer 2 owns no cache: its queries read what the latest run of layer 1 wrote
            layers=(layer(0, toy), layer(1, attn), layer(2, attn, cache_of=1)), schedule=(0, 1, 1, 2),
            final_norm=PartSpec("rmsnorm", norm, prefix="final"),
            lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": d, "name": "emb.weight"}),
            max_positions=256, stop_token_ids=(0,))

    register_architecture("ToyForCausalLM", ToyConfig.from_dict, toy_spec)
    return ToyConfig


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from harness import run_batch, run_tail, run_whole
    from picolm_b200.config import read_config
    from picolm_b200.engine import Engine
    from picolm_b200.weights import write_random_model
    from util import random_tokens
    ToyConfig = _register()
    d = write_random_model(ToyConfig(vocab_size=90, hidden_size=32), 3, str(tmp_path / "toy"), std=0.2)
    assert read_config(d).hidden_size == 32                    # found through the registry by config.json alone
    eng = Engine.from_folder(d, dtype="float32", max_tokens=64 * 8, max_seqs=4)
    # the cache is kept per run of the schedule (0: toy state; 1 and 2: the two runs of the attention layer)
    assert sorted(eng.cache.state) == [0] and sorted(eng.cache.layer_group) == [1, 2]          # run 3 owns nothing
    assert eng.cache.state[0].shape == (5, 33) and eng.cache.kv_groups[0].k.shape[0] == 2
    a, b = random_tokens(50, 90, 1), random_tokens(21, 90, 2)
    whole_a, whole_b = run_whole(eng, a), run_whole(eng, b)
    assert torch.isfinite(whole_a).all() and whole_a.std() > 0
    # the state carries across steps, per sequence, and starts from zero in a slot that is used again
    assert torch.allclose(run_tail(eng, a, tail=32), whole_a, atol=2e-5)
    out_b, out_a = run_batch(eng, [b, a], [4, 17])
    assert torch.allclose(out_a, whole_a, atol=2e-5) and torch.allclose(out_b, whole_b, atol=2e-5)
    assert torch.allclose(run_whole(eng, b), whole_b, atol=0)
    # the toy layer matters: with its mixing weight zeroed the logits change
    eng.model.blocks[0].mixer.w.zero_()
    assert not torch.allclose(run_whole(eng, a), whole_a, atol=1e-3)
    eng.cache.check()
