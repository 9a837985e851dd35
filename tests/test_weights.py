"""Weights: the container, the by-name check with its one error, random mode (no device)."""
import json
import os

import pytest
import torch

from picolm_b200.config import config_from_dict, spec_of
from picolm_b200.engine.model import Model
from picolm_b200.weights import (Checkpoint, SafetensorsError, WeightsError, check_checkpoint, random_tensors,
                                 save_safetensors, write_random_model)
from picolm_b200.weights.loader import to_run_dtype
from picolm_b200.parts import WeightSpec
from util import TINY


def _model(name):
    return Model(spec_of(config_from_dict(TINY[name]["config"])), runtime=None)


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(4, 2).to(torch.float16)}
    path = str(tmp_path / "model.safetensors")
    save_safetensors(path, t, metadata={"k": "v"})
    ck = Checkpoint(str(tmp_path))
    assert set(ck.names()) == set(t)
    for k, v in t.items():
        assert ck.entries[k].shape == tuple(v.shape)
        assert torch.equal(ck.tensor(k), v)
    assert ck.files[0].metadata == {"k": "v"}


def test_container_is_read_by_the_plain_reader_too(tmp_path):
    from plain import llama_plain
    t = {"x": torch.randn(4, 6).to(torch.bfloat16), "y": torch.randn(5)}
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    got = llama_plain.read_safetensors(str(tmp_path / "model.safetensors"))
    assert torch.equal(got["x"], t["x"].float()) and torch.equal(got["y"], t["y"])


def test_truncated_file_is_refused(tmp_path):
    save_safetensors(str(tmp_path / "model.safetensors"), {"x": torch.randn(8, 8)})
    raw = (tmp_path / "model.safetensors").read_bytes()
    (tmp_path / "model.safetensors").write_bytes(raw[:-16])
    with pytest.raises(SafetensorsError, match="outside the file"):
        Checkpoint(str(tmp_path))


def test_sharded_checkpoint(tmp_path):
    save_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {"a": torch.ones(2)})
    save_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    ck = Checkpoint(str(tmp_path))
    assert torch.equal(ck.tensor("a"), torch.ones(2)) and torch.equal(ck.tensor("b"), torch.zeros(3))


def test_expected_tensors_of_both_configs():
    a, b = _model("A").expected_tensors(), _model("B").expected_tensors()
    assert a["model.layers.1.mlp.down_proj.weight"].shape == (64, 172)
    assert a["model.layers.0.self_attn.k_proj.weight"].shape == (32, 64)
    assert a["lm_head.weight"].shape == (256, 64)
    assert "lm_head.weight" not in b and b["model.embed_tokens.weight"].shape == (384, 96)
    assert len(a) == 2 * 9 + 3 and len(b) == 3 * 9 + 2


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY["A"]["config"])
    t = random_tensors(cfg, 0)
    del t["model.layers.1.self_attn.v_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(64, 172, dtype=torch.bfloat16)     # transposed
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)                       # known, ignored
    t["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)                 # wrong type
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    m = _model("A")
    with pytest.raises(WeightsError) as e:
        check_checkpoint(m.expected_tensors(), Checkpoint(str(tmp_path)), m.spec.ignored_tensors)
    err = e.value
    assert [n for n, _ in err.missing] == ["model.layers.1.self_attn.v_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.mlp.up_proj.weight", (172, 64), (64, 172))]
    assert err.wrong_dtype[0][0] == "model.embed_tokens.weight"
    msg = str(err)
    for word in ("v_proj", "model.norm.weight", "extra.weight", "[172, 64]", "[64, 172]", "I32"):
        assert word in msg
    assert "inv_freq" not in msg


def test_untied_model_without_head_is_an_error_and_tied_ignores_a_stray_head(tmp_path):
    cfg = config_from_dict(TINY["A"]["config"])
    t = random_tensors(cfg, 0)
    del t["lm_head.weight"]
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    m = _model("A")
    with pytest.raises(WeightsError, match="lm_head.weight"):
        check_checkpoint(m.expected_tensors(), Checkpoint(str(tmp_path)), m.spec.ignored_tensors)
    cfgb = config_from_dict(TINY["B"]["config"])
    tb = random_tensors(cfgb, 1)
    tb["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.bfloat16)
    d = tmp_path / "b"
    d.mkdir()
    save_safetensors(str(d / "model.safetensors"), tb)
    mb = _model("B")
    check_checkpoint(mb.expected_tensors(), Checkpoint(str(d)), mb.spec.ignored_tensors)


def test_element_type_policy():
    ws, wi = WeightSpec((2,)), WeightSpec((2,), integer=True)
    f32, b16, f16 = torch.ones(2), torch.ones(2, dtype=torch.bfloat16), torch.ones(2, dtype=torch.float16)
    assert to_run_dtype(b16, ws, torch.bfloat16).dtype == torch.bfloat16
    assert to_run_dtype(f16, ws, torch.bfloat16).dtype == torch.bfloat16
    assert to_run_dtype(f32, ws, torch.bfloat16).dtype == torch.float32          # stored in 32 bits: stays so
    assert to_run_dtype(b16, ws, torch.float32).dtype == torch.float32
    assert to_run_dtype(torch.ones(2, dtype=torch.int64), wi, torch.bfloat16).dtype == torch.int32


def test_random_mode_writes_a_folder_and_is_seeded(tmp_path):
    cfg = config_from_dict(TINY["B"]["config"])
    d1 = write_random_model(cfg, 7, str(tmp_path / "m1"))
    d2 = write_random_model(cfg, 7, str(tmp_path / "m2"))
    d3 = write_random_model(cfg, 8, str(tmp_path / "m3"))
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    c1, c2, c3 = Checkpoint(d1), Checkpoint(d2), Checkpoint(d3)
    for n in c1.names():
        assert torch.equal(c1.tensor(n), c2.tensor(n))
    assert not torch.equal(c1.tensor("model.embed_tokens.weight"), c3.tensor("model.embed_tokens.weight"))
    w = c1.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert w.dtype == torch.float32 and abs(w.std().item() - 0.02) < 0.002
    n = c1.tensor("model.norm.weight").float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    from picolm_b200.config import read_config
    assert read_config(d1) == cfg
    m = _model("B")
    check_checkpoint(m.expected_tensors(), c1, m.spec.ignored_tensors)
