#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ from whoreson/picolm's own CPU
model code.

    python tests/golden/make_golden.py /path/to/picolm/picolm

It copies the reference's C sources into a temporary folder, compiles the model
objects unchanged with gcc, links them with ref_harness.c (the reference's own
CLI does not link without its GPU backend), writes each tiny model's weights as
fp32 into a flat file, runs the harness and stores what it printed:

    tests/golden/<case>.json   config, seed, tokens
    tests/golden/<case>.f32    logits [n_tokens + 1, vocab]: every position through
                               model_forward, then the last one through
                               model_forward_prefill

Cases: Tiny A with the half-split pairing (rope_type 1) and with the adjacent
pairing (rope_type 0), and Tiny B, whose llama3-scaled rotary table is injected
(the reference has no rotary scaling, so that rule itself rests on its formula).
The reference rounds K and V to fp16 in its cache; the test that reads these
files gives the plain implementation the same rounding.
"""
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

OBJECTS = ["model_core", "model_attention", "model_moe", "model_gemma3n", "model_ssm", "model_kv_cache",
           "model_gguf", "tensor", "quant", "csafetensors", "cJSON", "safetensors"]
CFLAGS = ["-O2", "-std=c11", "-D_GNU_SOURCE", "-fno-common", "-w"]


def build_harness(ref_src, work):
    for fn in os.listdir(ref_src):
        if fn.endswith((".c", ".h")):
            shutil.copy(os.path.join(ref_src, fn), work)
    shutil.copy(os.path.join(HERE, "ref_harness.c"), work)
    for o in OBJECTS + ["ref_harness"]:
        subprocess.run(["gcc", *CFLAGS, "-c", o + ".c", "-o", o + ".o"], cwd=work, check=True)
    subprocess.run(["gcc", "-o", "ref_harness", *[o + ".o" for o in OBJECTS + ["ref_harness"]], "-lm", "-lpthread"],
                   cwd=work, check=True)
    return os.path.join(work, "ref_harness")


def run_case(harness, work, case, cfg, seed, tokens, rope_type, inject_table):
    from plain import llama_plain as P
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors
    w = {k: v.float() for k, v in random_tensors(config_from_dict(cfg), seed).items()}
    d, F, H, G = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    L, V, S, hd = cfg["num_hidden_layers"], cfg["vocab_size"], cfg["max_position_embeddings"], cfg["head_dim"]
    tied = bool(cfg["tie_word_embeddings"])
    path_in, path_out = os.path.join(work, case + ".in"), os.path.join(work, case + ".out")
    with open(path_in, "wb") as f:
        f.write(struct.pack("<12i", d, F, H, G, L, V, S, hd, rope_type, int(tied), len(tokens), int(inject_table)))
        f.write(struct.pack("<2f", cfg["rope_theta"], cfg["rms_norm_eps"]))
        f.write(np.asarray(tokens, dtype="<i4").tobytes())

        def put(name):
            f.write(w[name].contiguous().numpy().astype("<f4").tobytes())

        put("model.embed_tokens.weight")
        for l in range(L):
            p = f"model.layers.{l}."
            for n in ("input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                      "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
                put(p + n + ".weight")
        put("model.norm.weight")
        if not tied:
            put("lm_head.weight")
        if inject_table:
            cos, sin = P.rope_table(S, hd, cfg["rope_theta"], cfg.get("rope_scaling"))
            f.write(cos.float().numpy().astype("<f4").tobytes())
            f.write(sin.float().numpy().astype("<f4").tobytes())
    subprocess.run([harness, path_in, path_out], check=True)
    shutil.copy(path_out, os.path.join(HERE, case + ".f32"))
    with open(os.path.join(HERE, case + ".json"), "w") as f:
        json.dump({"config": cfg, "seed": seed, "tokens": tokens, "rope_type": rope_type,
                   "pairing": "half" if rope_type == 1 else "adjacent", "table_injected": bool(inject_table)}, f, indent=1)


def main():
    from util import TINY, random_tokens
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <the reference's source folder (the one with model_core.c)>")
    ref_src = sys.argv[1]
    with tempfile.TemporaryDirectory() as work:
        harness = build_harness(ref_src, work)
        a, b = TINY["A"], TINY["B"]
        run_case(harness, work, "tiny_a_half", a["config"], a["seed"], random_tokens(11, 256, 900), 1, False)
        run_case(harness, work, "tiny_a_adjacent", a["config"], a["seed"], random_tokens(11, 256, 901), 0, False)
        run_case(harness, work, "tiny_b_llama3", b["config"], b["seed"], random_tokens(40, 384, 902), 1, True)
    print("golden files written to", HERE)


if __name__ == "__main__":
    main()
