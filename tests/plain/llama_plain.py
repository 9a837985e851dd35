"""A plain, slow Llama decoder written from the reference's formulas: whole
sequences, no cache, no batching, one function for each part, float32 (or
float64) on the CPU.  It shares no code with picolm_b200: it reads config.json
and the safetensors file itself.

Each function cites the lines of whoreson/picolm it restates.  The llama3
rotary scaling is not in the reference; `rope_frequencies` states the rule that
Llama-3 checkpoints carry in `rope_scaling`.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# ----------------------------------------------------------------- the folder
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_safetensors(path):
    """name -> float32 torch tensor.  Container: picolm/csafetensors.h:49-79."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = raw[8 + hlen + b:8 + hlen + e]
        if info["dtype"] == "BF16":
            # bf16 is the upper half of a float32 (picolm/quant.c:133-153)
            u16 = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4")
        elif info["dtype"] == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float32)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = torch.from_numpy(arr.copy()).reshape(info["shape"])
    return out


def load_model(model_dir, dtype=torch.float32):
    cfg = read_config(model_dir)
    w = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


# ------------------------------------------------------------------ the parts
def embed(tokens, table):
    """x[t] = float(table[token[t]]), no scale.  picolm/model_core.c:1785-1786, :2758-2762."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x, weight, eps):
    """ss = sum x^2; r = 1/sqrt(ss/size + eps); out = x*r*w.  picolm/tensor.c:2942-3064 (:3001, :3062)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * r * weight


def linear(x, w):
    """out[o] = sum_i w[o, i] * x[i]; w is [out, in] row-major.  picolm/tensor.c:1394-1418."""
    return x @ w.t()


def rope_frequencies(head_dim, theta, scaling):
    """inv_freq[i] = theta^(-2i/head_dim)  (picolm/model_core.c:314-326 divides the
    position by theta^(2i/rope_dim)).  llama3 rule (not in the reference): with
    wavelen = 2 pi / inv_freq and L0 the original context, keep inv_freq when
    wavelen < L0/high, divide by factor when wavelen > L0/low, else blend with
    smooth = (L0/wavelen - low) / (high - low)."""
    inv = [theta ** (-(2.0 * i) / head_dim) for i in range(head_dim // 2)]
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        fac, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
        L0 = scaling["original_max_position_embeddings"]
        scaled = []
        for f in inv:
            wl = 2.0 * math.pi / f
            if wl < L0 / high:
                scaled.append(f)
            elif wl > L0 / low:
                scaled.append(f / fac)
            else:
                s = (L0 / wl - low) / (high - low)
                scaled.append((1 - s) * f / fac + s * f)
        inv = scaled
    return torch.tensor(inv, dtype=torch.float64)


def rope_table(n_pos, head_dim, theta, scaling):
    """cos/sin[pos][i] of pos * inv_freq[i].  picolm/model_core.c:314-326."""
    ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * rope_frequencies(head_dim, theta, scaling)[None, :]
    return ang.cos(), ang.sin()


def rope(x, cos, sin, pairing="half"):
    """x: [T, heads, hd].  half: pairs (x[i], x[i+hd/2]); adjacent: (x[2i], x[2i+1]);
    (x0, x1) -> (x0 c - x1 s, x0 s + x1 c).  picolm/tensor.c:3216-3304."""
    T, nh, hd = x.shape
    c = cos[:T].to(x.dtype)[:, None, :]
    s = sin[:T].to(x.dtype)[:, None, :]
    out = torch.empty_like(x)
    if pairing == "half":
        x0, x1 = x[..., :hd // 2], x[..., hd // 2:]
        out[..., :hd // 2] = x0 * c - x1 * s
        out[..., hd // 2:] = x0 * s + x1 * c
    else:
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
    return out


def attention(q, k, v, scale, window=None):
    """q: [T, H, hd], k/v: [T, G, hd].  For query t and head h with g = h // (H/G):
    s_u = (q . k_u) * scale for u <= t, softmax, out = sum p_u v_u.
    picolm/model_attention.c:43-140 (one query), picolm/model_core.c:2066-2095 (g, scale)."""
    T, H, hd = q.shape
    G = k.shape[1]
    out = torch.empty_like(q)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h, :] @ k[:, g, :].t()) * scale                    # [T, T]
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] < idx[:, None] - window + 1)
        s = s.masked_fill(mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate, up):
    """silu(g) * u with silu(g) = g / (1 + exp(-g)).  picolm/tensor.c:3306-3315, picolm/model_core.c:2192-2193."""
    return gate / (1.0 + torch.exp(-gate)) * up


# ----------------------------------------------------------------- the model
def forward(cfg, w, tokens, pairing="half", window=None, return_hidden=False, act_dtype=None, kv_dtype=None):
    """Logits [T, vocab] of one whole sequence.  Layer order: picolm/model_core.c:1797-2220.
    `act_dtype=torch.bfloat16` rounds the activations where a bfloat16 run keeps them
    in 16 bits (norm outputs, projections, rotated q/k, v, attention output, the
    activated branch); the residual stream and its deltas stay float32.
    `kv_dtype=torch.float16` rounds only the cached keys and values, as the reference
    does (picolm/model_core.c:1943-1955, :2003-2015)."""
    def rnd(t):
        return t if act_dtype is None else t.to(act_dtype).to(t.dtype)

    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads") or H
    d = cfg["hidden_size"]
    hd = cfg.get("head_dim") or d // H
    eps = cfg["rms_norm_eps"]
    T = len(tokens)
    cos, sin = rope_table(T, hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    cos, sin = cos.to(torch.float32), sin.to(torch.float32)
    x = embed(tokens, w["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = rnd(rmsnorm(x, w[p + "input_layernorm.weight"], eps))
        q = rnd(linear(h, w[p + "self_attn.q_proj.weight"])).reshape(T, H, hd)
        k = rnd(linear(h, w[p + "self_attn.k_proj.weight"])).reshape(T, G, hd)
        v = rnd(linear(h, w[p + "self_attn.v_proj.weight"])).reshape(T, G, hd)
        q, k = rnd(rope(q, cos, sin, pairing)), rnd(rope(k, cos, sin, pairing))
        if kv_dtype is not None:
            k, v = k.to(kv_dtype).to(x.dtype), v.to(kv_dtype).to(x.dtype)
        a = rnd(attention(q, k, v, 1.0 / math.sqrt(hd), window)).reshape(T, H * hd)
        x = x + linear(a, w[p + "self_attn.o_proj.weight"])
        h = rnd(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps))
        gate = rnd(linear(h, w[p + "mlp.gate_proj.weight"]))
        up = rnd(linear(h, w[p + "mlp.up_proj.weight"]))
        x = x + linear(rnd(swiglu(gate, up)), w[p + "mlp.down_proj.weight"])
    hidden = rnd(rmsnorm(x, w["model.norm.weight"], eps))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    logits = linear(hidden, head)
    return (logits, hidden) if return_hidden else logits


def greedy(cfg, w, prompt, n_new, stop=()):
    """Greedy generation by re-running the whole sequence for every token."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = argmax(forward(cfg, w, toks)[-1])
        out.append(nxt)
        if nxt in stop:
            break
        toks.append(nxt)
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits):
    """First index of the maximum (strict > scan).  picolm/sampler.c:50-56."""
    best = 0
    vals = logits.tolist()
    for i in range(1, len(vals)):
        if vals[i] > vals[best]:
            best = i
    return best


def xorshift64(state):
    """picolm/sampler.c:10-17.  Returns (new state, value)."""
    m = (1 << 64) - 1
    x = state
    x ^= (x << 13) & m
    x ^= x >> 7
    x ^= (x << 17) & m
    return x, x


def rand_float(state):
    """(float)(x >> 11) / 2^53 in float32.  picolm/sampler.c:19-21."""
    state, x = xorshift64(state)
    return state, float(np.float32(x >> 11) / np.float32(2.0 ** 53))


def sampling_weights(logits, temperature, top_k, top_p, min_p):
    """The kept tokens and their renormalised weights p^(1/T), as the reference
    finds them: softmax, sort descending, cut to top_k, cut where the cumulative
    probability reaches top_p, drop p < min_p * p_max, p^(1/T), renormalise.
    picolm/sampler.c:58-109.  Returns (indices in sorted order, weights)."""
    x = logits.to(torch.float32)
    p = torch.exp(x - x.max())
    p = p / p.sum()                                   # picolm/tensor.c:3066-3076
    order = sorted(range(len(p)), key=lambda i: (-float(p[i]), i))
    V = len(order)
    k_limit = top_k if 0 < top_k < V else V
    cum, cutoff = np.float32(0.0), 0
    for j in range(k_limit):
        cum = np.float32(cum + np.float32(p[order[j]]))
        cutoff = j + 1
        if cum >= np.float32(top_p):
            break
    if min_p > 0 and cutoff > 1:
        thr = np.float32(min_p) * np.float32(p[order[0]])
        new_cut = 0
        for j in range(cutoff):
            if np.float32(p[order[j]]) >= thr:
                new_cut = j + 1
        cutoff = max(new_cut, 1)
    kept = order[:cutoff]
    wts = torch.tensor([float(p[i]) for i in kept], dtype=torch.float32) ** (1.0 / temperature)
    wts = wts / wts.sum()
    return kept, wts


def sample_reference_order(logits, temperature, top_k, top_p, min_p, state):
    """The reference's draw: walk the kept tokens in sorted order until the
    cumulative weight exceeds r.  picolm/sampler.c:111-121."""
    if temperature <= 0:
        return state, argmax(logits)
    kept, wts = sampling_weights(logits, temperature, top_k, top_p, min_p)
    state, r = rand_float(state)
    acc = np.float32(0.0)
    for i, wgt in zip(kept, wts.tolist()):
        acc = np.float32(acc + np.float32(wgt))
        if acc > r:
            return state, i
    return state, kept[0]


def sample_index_order(logits, temperature, top_k, top_p, min_p, state):
    """The same kept set and weights, walked in index order (what the engine's
    kernel does; the distribution is the reference's)."""
    if temperature <= 0:
        return state, argmax(logits)
    kept, wts = sampling_weights(logits, temperature, top_k, top_p, min_p)
    state, r = rand_float(state)
    pairs = sorted(zip(kept, wts.tolist()))
    acc = np.float32(0.0)
    for i, wgt in pairs:
        acc = np.float32(acc + np.float32(wgt))
        if acc > r:
            return state, i
    return state, kept[0]
