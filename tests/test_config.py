"""Configuration and registry (no device)."""
import json

import pytest

from picolm_b200.config import (ConfigError, config_from_dict, read_config, registered_architectures,
                                spec_of)
from util import TINY


def test_reads_every_key_of_both_tiny_configs():
    a = config_from_dict(TINY["A"]["config"])
    b = config_from_dict(TINY["B"]["config"])
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps) == (172, 256, 10000.0, 1e-5)
    assert a.rope_scaling is None and not a.tie_word_embeddings and a.eos_token_id == (2,)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.tie_word_embeddings and b.eos_token_id == (3, 4) and b.max_position_embeddings == 256


def test_defaults_of_absent_keys_follow_the_reference():
    raw = {"architectures": ["LlamaForCausalLM"], "vocab_size": 10, "hidden_size": 24, "intermediate_size": 8,
           "num_hidden_layers": 1, "num_attention_heads": 3}
    c = config_from_dict(raw)
    assert c.head_dim == 8 and c.num_key_value_heads == 3
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.bos_token_id == 1 and c.eos_token_id == (2,)


def test_round_trip_through_json(tmp_path):
    c = config_from_dict(TINY["B"]["config"])
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert read_config(str(tmp_path)) == c


def test_text_config_is_unwrapped():
    inner = dict(TINY["A"]["config"])
    archs = inner.pop("architectures")
    c = config_from_dict({"architectures": archs, "text_config": inner})
    assert c.hidden_size == 64


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_scaling"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_unsupported_values_name_their_key(patch, word):
    raw = dict(TINY["A"]["config"])
    raw.update(patch)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_missing_key_is_named():
    raw = dict(TINY["A"]["config"])
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(raw)


def test_unknown_architecture_lists_the_known_ones():
    raw = dict(TINY["A"]["config"])
    raw["architectures"] = ["MambaForCausalLM"]
    with pytest.raises(KeyError) as e:
        config_from_dict(raw)
    assert "LlamaForCausalLM" in str(e.value)
    assert "LlamaForCausalLM" in registered_architectures()


def test_spec_is_data_layer_by_layer():
    c = config_from_dict(TINY["B"]["config"])
    s = spec_of(c)
    assert len(s.layers) == 3 and s.schedule == (0, 1, 2)
    assert s.layers[1].part("mixer").kind == "attention" and s.layers[1].part("feed_forward").kind == "gated_mlp"
    assert s.layers[2].part("mixer").params["num_kv_heads"] == 1
    assert s.layers[0].part("mixer").params["position"].params["scaling"]["factor"] == 4.0
    assert s.lm_head.params["name"] == "model.embed_tokens.weight"          # tied
    assert s.stop_token_ids == (3, 4)
    a = spec_of(config_from_dict(TINY["A"]["config"]))
    assert a.lm_head.params["name"] == "lm_head.weight"


def test_schedule_and_cache_sharing_are_validated():
    import dataclasses
    s = spec_of(config_from_dict(TINY["B"]["config"]))
    with pytest.raises(ValueError, match="schedule"):
        dataclasses.replace(s, schedule=(0, 5)).validate()
    layers = list(s.layers)
    layers[0] = dataclasses.replace(layers[0], cache_of=2)                   # reads a cache not yet written
    with pytest.raises(ValueError, match="before"):
        dataclasses.replace(s, layers=tuple(layers)).validate()
    layers = list(s.layers)
    layers[2] = dataclasses.replace(layers[2], cache_of=0)
    dataclasses.replace(s, layers=tuple(layers), schedule=(0, 1, 2, 1)).validate()


def test_layer_hook_brackets_every_run_of_the_schedule():
    """`Model.layer_hook` (the reference's per-layer benchmark callback) is called before and after every run
    of the schedule, in order, with the run and the layer; without a hook the forward is as before.  The parts
    are replaced by stand-ins that record when they run, so this needs no device."""
    from types import SimpleNamespace
    from picolm_b200.engine.model import Model
    import dataclasses
    spec = dataclasses.replace(spec_of(config_from_dict(TINY["A"]["config"])), schedule=(0, 1, 0))   # a layer run twice
    model = Model(spec, runtime=None)
    log = []

    class Block:
        def __init__(self, i):
            self.i = i

        def forward(self, stream, step, cache):
            log.append(("layer", self.i))

    model.embedding = SimpleNamespace(forward=lambda step: "x")
    model.blocks = [Block(i) for i in range(len(spec.layers))]
    model.final_norm = SimpleNamespace(forward=lambda stream, rows=None: "h")
    model.head = SimpleNamespace(forward=lambda h: "logits")
    model.layer_caches = lambda run, cache, step: []
    step = SimpleNamespace(n_want=1, want_rows=None)
    assert model.forward(step, None) == "logits"
    assert log == [("layer", 0), ("layer", 1), ("layer", 0)]
    log.clear()
    model.layer_hook = lambda run, layer, done: log.append(("hook", run, layer, done))
    assert model.forward(step, None) == "logits"
    assert log == [("hook", 0, 0, False), ("layer", 0), ("hook", 0, 0, True),
                   ("hook", 1, 1, False), ("layer", 1), ("hook", 1, 1, True),
                   ("hook", 2, 0, False), ("layer", 0), ("hook", 2, 0, True)]


def test_benchmark_layer_times_are_means_per_run():
    from picolm_b200.cli import build_parser, layer_times
    assert layer_times([(0, 1.0), (1, 2.0), (0, 3.0), (1, 4.0)], 3) == [2.0, 3.0, 0.0]
    args = build_parser().parse_args(["model", "-p", "1,2", "--benchmark", "-n", "4"])
    assert args.benchmark and not args.benchmark_ctx and args.max_tokens == 4


def test_one_sm_count_on_both_sides():
    """Plans (K splits, waves, cluster sizes) are made for the B200's SM count on the Python side and in the
    kernels' host code; both read it from one constant each, and the two agree."""
    import os
    import re
    from picolm_b200.ops._lib import SM_COUNT
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "picolm_b200", "csrc")
    with open(os.path.join(csrc, "common.cuh")) as f:
        assert int(re.search(r"#define PLM_SM_COUNT (\d+)", f.read()).group(1)) == SM_COUNT
    for name in os.listdir(csrc):
        if name.endswith((".cu", ".cuh")):
            with open(os.path.join(csrc, name)) as f:
                assert not re.search(r"\b148\b", re.sub(r"#define PLM_SM_COUNT 148", "", f.read())), name
