"""Llama dense decoder as a layout of parts.

Layer order as the reference runs it (picolm/model_core.c:1797-2210):
`x += Attention(RMSNorm(x)); x += SwiGLU(RMSNorm(x))` for every layer, then the
final RMSNorm and the LM head (picolm/model_core.c:2213-2220).  Tensor names are
the safetensors names the reference looks up (picolm/safetensors.c:236-330).
This file is everything that is specific to the architecture: it only fills
`PartSpec`s from `LlamaConfig`; the parts themselves know nothing of Llama.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec
from ..parts.block import pre_norm_layer


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
    position = PartSpec("rope", {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.head_dim,            # the reference rotates the whole head (picolm/safetensors.c:128-130)
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        # safetensors checkpoints pair x[i] with x[i + half]; the reference's GGUF
        # files are permuted to adjacent pairs instead (picolm/tensor.c:3216-3304).
        "pairing": "half",
        "max_positions": cfg.max_position_embeddings,
    })
    attention = PartSpec("attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "scale": None,                          # 1/sqrt(head_dim) (picolm/model_core.c:2077)
        "window": None,                         # the reference's Llama path has no sliding window
        "position": position,
        "q_name": "q_proj.weight", "k_name": "k_proj.weight",
        "v_name": "v_proj.weight", "o_name": "o_proj.weight",
    }, prefix="self_attn")
    swiglu = PartSpec("gated_mlp", {
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
        "activation": cfg.hidden_act,
        "gate_name": "gate_proj.weight", "up_name": "up_proj.weight", "down_name": "down_proj.weight",
    }, prefix="mlp")
    layers = tuple(
        pre_norm_layer(
            prefix=f"model.layers.{i}",
            mixer=attention,
            feed_forward=swiglu,
            mixer_norm=PartSpec("rmsnorm", norm, prefix="input_layernorm"),
            feed_forward_norm=PartSpec("rmsnorm", norm, prefix="post_attention_layernorm"),
        )
        for i in range(cfg.num_hidden_layers)
    )
    ignored = [r".*rotary_emb\.inv_freq$"]
    if cfg.tie_word_embeddings:
        # A tied checkpoint may still carry a copy of the head; the embedding is used.
        ignored.append(r"^lm_head\.weight$")
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "name": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=tuple(range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", norm, prefix="model.norm"),
        lm_head=PartSpec("lm_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            # tied: the head is the embedding matrix (picolm/safetensors.c:248-251)
            "name": "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"}),
        max_positions=cfg.max_position_embeddings,
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id,
        ignored_tensors=tuple(ignored),
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)
