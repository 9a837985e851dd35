"""Shared helpers of the tests: the tiny configurations, model folders with
random weights, and error measures."""
import json
import os

import torch

# Two tiny Llama configurations that differ in every size and option: layers,
# width, heads, KV heads (GQA / MQA), head size, intermediate size (172 is no
# multiple of 8), vocabulary, theta, rotary scaling, eps, context, tied or not.
TINY = {
    "A": {
        "seed": 0,
        "config": {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
            "head_dim": 16, "intermediate_size": 172, "vocab_size": 256, "rope_theta": 10000.0,
            "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 128,
            "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
        },
        "prompts": [5, 11, 17], "decode": 8,
    },
    "B": {
        "seed": 1,
        "config": {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
            "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 64},
            "rms_norm_eps": 1e-6, "max_position_embeddings": 256,
            "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 0, "eos_token_id": [3, 4],
        },
        "prompts": [1, 40], "decode": 12,
    },
}


def make_model_dir(path, config_dict, seed, sharpen=None, std=0.02, norm_std=0.1):
    """Write a random model folder.  `sharpen` multiplies the query and key
    projections so that attention is peaked: with N(0, 0.02) weights every key
    gets nearly the same probability and a wrong key or position would barely
    show in the logits."""
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors, save_safetensors
    cfg = config_from_dict(config_dict)
    tensors = random_tensors(cfg, seed, std=std, norm_std=norm_std)
    if sharpen:
        for name in tensors:
            if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
            elif name.endswith("_proj.weight") or name.endswith("embed_tokens.weight") or name == "lm_head.weight":
                tensors[name] = (tensors[name].float() * 2.0).to(tensors[name].dtype)
    os.makedirs(path, exist_ok=True)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    return path


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Tolerances, fixed from the arithmetic and not from what a run happened to give.
# float32: both sides accumulate in fp32 in different orders; errors are a few
# ulps of values of order one.
FP32_ATOL = 2e-5
# bfloat16: activations are rounded to 8 bits of mantissa (relative step 2^-8)
# at every matrix product; against the plain implementation with the same
# rounding points the remaining difference is accumulation order and single-ulp
# flips of activations.
BF16_REL_RMS = 0.02
BF16_MAX_OVER_STD = 0.12


def assert_close_fp32(got, ref, what=""):
    err = (got.double() - ref.double()).abs().max().item()
    scale = max(1.0, ref.abs().max().item())
    assert err <= FP32_ATOL * scale, f"{what}: max |diff| {err:.3e} exceeds {FP32_ATOL * scale:.1e}"


def assert_close_bf16(got, ref, what=""):
    diff = got.double() - ref.double()
    rel_rms = diff.pow(2).mean().sqrt().item() / max(ref.double().pow(2).mean().sqrt().item(), 1e-12)
    worst = diff.abs().max().item() / max(ref.double().std().item(), 1e-12)
    assert rel_rms <= BF16_REL_RMS, f"{what}: relative rms error {rel_rms:.4f} exceeds {BF16_REL_RMS}"
    assert worst <= BF16_MAX_OVER_STD, f"{what}: max |diff| is {worst:.4f} of the logits' std, limit {BF16_MAX_OVER_STD}"


def assert_close(got, ref, dtype, what=""):
    if dtype == "float32":
        assert_close_fp32(got, ref, what)
    else:
        assert_close_bf16(got, ref, what)


def gemm_tc_workspace(a, w, out_dtype):
    """out = a @ w^T through `plm_gemm_tc`, the exported split-K product for at most 64 rows that takes a
    caller-allocated fp32 workspace (csrc/gemm_tc.cu), called through its C symbol with a workspace from
    torch.  The engine does not use it; `plm_gemm_tc_static` is its twin without the workspace."""
    import ctypes
    from picolm_b200.csrc.build import load_library
    lib = load_library("gemm_tc")
    vp, i, l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
    lib.plm_gemm_tc.argtypes = [vp, vp, vp, i, i, i, i, l, l, l, vp, vp, vp]
    lib.plm_gemm_tc_plan.argtypes = [i, i, i, ctypes.POINTER(i), ctypes.POINTER(l)]
    M, K = a.shape
    N = w.shape[0]
    splits, elems = i(0), l(0)
    lib.plm_gemm_tc_plan(M, N, K, ctypes.byref(splits), ctypes.byref(elems))
    ws = torch.empty((max(elems.value, 1),), dtype=torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    rc = lib.plm_gemm_tc(a.data_ptr(), w.data_ptr(), out.data_ptr(), 0 if out_dtype == torch.float32 else 1, M, N, K,
                         K, K, N, ws.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"plm_gemm_tc returned {rc}"
    assert int(status.item()) == 0
    return out
