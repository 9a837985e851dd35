"""The engine at further sizes than the two tiny configurations: head sizes in steps of 16 up to 256,
many query heads per KV head (more than one row group of the decode kernel), as many KV heads as heads,
a projection width H * head_dim that differs from the hidden size, widths and vocabularies that are no
multiple of 8 (which sends products to the CUDA-core kernel) next to ones the tensor cores take.  Each
shape: whole, the last tokens one by one, and an unequal batch, in both dtypes, against the plain
implementation."""
import pytest
import torch

from harness import run_batch, run_tail, run_whole
from plain import llama_plain as P
from util import assert_close, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu

#        layers d    H   G   hd   F    vocab theta    eps   tied
SHAPES = {
    "hd48_mha":      (1, 96,  2,  2,  48, 200, 301, 10000.0, 1e-5, False),
    "hd80_gqa":      (2, 160, 4,  2,  80, 416, 512, 50000.0, 1e-6, True),
    "hd112_wide_qk": (1, 64,  3,  1, 112, 192, 250, 10000.0, 1e-5, False),      # H * hd = 336, hidden 64
    "hd256":         (1, 128, 2,  1, 256, 256, 128, 10000.0, 1e-5, True),
    "mqa_20_heads":  (1, 320, 20, 1,  16, 320, 264, 10000.0, 1e-5, False),      # 20 query heads on one KV head
    "odd_widths":    (2, 72,  3,  3,  24, 100, 97,  10000.0, 1e-5, False),      # F = 100: not a multiple of 8
    "hd40":          (1, 80,  2,  1,  40, 160, 130, 10000.0, 1e-5, False),      # no multiple of 16: CUDA-core attention
}


def _config(shape):
    L, d, H, G, hd, F, V, theta, eps, tied = shape
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": L, "hidden_size": d,
            "num_attention_heads": H, "num_key_value_heads": G, "head_dim": hd, "intermediate_size": F,
            "vocab_size": V, "rope_theta": theta, "rope_scaling": None, "rms_norm_eps": eps,
            "max_position_embeddings": 512, "tie_word_embeddings": tied, "hidden_act": "silu",
            "bos_token_id": 1, "eos_token_id": 2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_shape_in_every_cut(tmp_path, name, dtype):
    from picolm_b200.engine import Engine
    cfg_dict = _config(SHAPES[name])
    d = make_model_dir(str(tmp_path / name), cfg_dict, 40 + len(name), sharpen=3.0)
    cfg, w = P.load_model(d)
    V = cfg_dict["vocab_size"]
    toks = {n: random_tokens(n, V, 900 + n) for n in (150, 70, 9)}
    act = torch.bfloat16 if dtype == "bfloat16" else None
    ref = {n: P.forward(cfg, w, t, act_dtype=act) for n, t in toks.items()}
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 12, max_seqs=4)
    assert_close(run_whole(eng, toks[150]), ref[150], dtype, f"{name} {dtype} whole")
    assert_close(run_tail(eng, toks[70], tail=32), ref[70], dtype, f"{name} {dtype} tail")
    outs = run_batch(eng, [toks[9], toks[150], toks[70]], [2, 100, 38])
    for n, got in zip((9, 150, 70), outs):
        assert_close(got, ref[n], dtype, f"{name} {dtype} batch {n}")
    eng.cache.check()
    if dtype == "bfloat16":
        from picolm_b200 import ops
        ops.check_status()


def test_head_size_beyond_the_kernels_is_refused(tmp_path):
    """A head of 272 is more than any attention kernel takes: a clear error at the first step, no result."""
    from picolm_b200.engine import Engine
    from picolm_b200.ops import KernelError
    cfg_dict = _config((1, 64, 1, 1, 272, 64, 50, 10000.0, 1e-5, False))
    d = make_model_dir(str(tmp_path / "hd272"), cfg_dict, 3)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(d, dtype=dtype, max_tokens=128, max_seqs=1)
        s = eng.new_sequence()
        with pytest.raises(KernelError, match="head_dim 272 exceeds 256"):
            eng.step([(s, [1, 2, 3])])
        eng.end_sequence(s)
