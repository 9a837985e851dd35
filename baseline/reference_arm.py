"""The reference arm of bench.py: whoreson/picolm itself, unmodified, timed on the same GPU.

The reference is a C program with a CUDA backend, not a Python package, so "installing" it means copying
its source folder to `baseline/_ref/picolm` and building its stock command line with its own Makefile
(`make cuda CUDA_ARCH=sm_100`, picolm/Makefile:309-333).  It reads GGUF files with a vocabulary in their
metadata, so this module writes one: random bfloat16 weights at the benchmark's shape under the tensor
names its loader looks up (picolm/model_gguf.c:1190-1251), the `llama.*` keys it reads
(picolm/model_gguf.c:755-922) and a vocabulary whose first entries are single letters, so that a prompt of
N letters is N tokens (picolm/tokenizer.c:155-290: characters are looked up one by one, then merged where
the merged string is a token; none is).  Then it runs the stock binary with `PICOLM_GPU=1`
(picolm/model_core.c:1143-1154) and reads the `Prefill:` / `Generation:` lines that it prints
(picolm/picolm.c:1629-1636), which is how the reference's own bench script measures (picolm/bench.zsh).

Nothing of picolm_b200 runs on this path except torch's random numbers for the weights.
"""
from __future__ import annotations

import os
import re
import shutil
import struct
import subprocess
import sys
import time
from typing import Dict, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref", "picolm")
# where the reference's checkout is looked for: beside this repository, unless the variable says otherwise
SOURCE = os.environ.get("PICOLM_REFERENCE_SOURCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "picolm")

GGUF_F32, GGUF_BF16 = 0, 30
META_U32, META_F32, META_BOOL, META_STR, META_ARRAY = 4, 6, 7, 8, 9
ALIGN = 32


class Unavailable(RuntimeError):
    """The reference cannot be run here; the message is the one line that bench.py prints."""


def _say(msg: str) -> None:
    print(f"[reference] {msg}", file=sys.stderr, flush=True)


# ------------------------------------------------------------------ install and build
def install() -> str:
    """Copy the reference's source folder under baseline/_ref (once); returns the folder."""
    if os.path.isfile(os.path.join(REF_DIR, "Makefile")):
        return REF_DIR
    if not os.path.isfile(os.path.join(SOURCE, "Makefile")):
        raise Unavailable(f"the reference's sources are neither under baseline/_ref/picolm nor under {SOURCE}")
    os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
    shutil.copytree(SOURCE, REF_DIR, ignore=shutil.ignore_patterns("*.o", "picolm", "*.gguf"))
    _say(f"copied {SOURCE} -> {REF_DIR}")
    return REF_DIR


def _runs(binary: str) -> bool:
    """Whether the binary starts on this machine (it is built with -march=native: one built on another CPU
    may not)."""
    try:
        r = subprocess.run([binary], capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.TimeoutExpired):
        return False
    return "Usage:" in r.stdout + r.stderr


def build() -> str:
    """The reference's stock CUDA command line, built by its own Makefile; returns the binary's path."""
    folder = install()
    binary = os.path.join(folder, "picolm")
    if os.path.isfile(binary) and _runs(binary):
        return binary
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    log = os.path.join(folder, "build.log")
    _say("building the reference: make cuda CUDA_ARCH=sm_100 ...")
    t0 = time.time()
    with open(log, "w") as f:
        subprocess.run(["make", "clean"], cwd=folder, stdout=f, stderr=subprocess.STDOUT)
        r = subprocess.run(["make", "cuda", "CUDA_ARCH=sm_100", f"CC={cc}", "-j8"], cwd=folder, stdout=f,
                           stderr=subprocess.STDOUT)
    if r.returncode != 0 or not _runs(binary):
        raise Unavailable(f"the reference's `make cuda CUDA_ARCH=sm_100` failed here (log: {log})")
    _say(f"built in {time.time() - t0:.0f} s")
    return binary


# ------------------------------------------------------------------------------ GGUF
def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def letters_vocab(vocab_size: int):
    """Token strings: 0 `<unk>`, 1 `<s>`, 2 `</s>`, 3..28 the letters a..z, then names that no text spells."""
    names = ["<unk>", "<s>", "</s>"] + [chr(ord("a") + i) for i in range(26)]
    names += [f"<t{i}>" for i in range(len(names), vocab_size)]
    return names[:vocab_size]


def write_gguf(path: str, cfg: Dict, seed: int) -> int:
    """A GGUF v3 file of a Llama model with random weights N(0, 0.02) in bfloat16 and norm weights 1 in
    float32.  `cfg` has config.json's keys.  Returns the file's size."""
    import torch
    d, F, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    H, G, hd, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    tensors = [("token_embd.weight", (V, d), GGUF_BF16), ("output_norm.weight", (d,), GGUF_F32)]
    if not cfg.get("tie_word_embeddings"):
        tensors.append(("output.weight", (V, d), GGUF_BF16))
    for l in range(L):
        p = f"blk.{l}."
        tensors += [(p + "attn_norm.weight", (d,), GGUF_F32), (p + "attn_q.weight", (H * hd, d), GGUF_BF16),
                    (p + "attn_k.weight", (G * hd, d), GGUF_BF16), (p + "attn_v.weight", (G * hd, d), GGUF_BF16),
                    (p + "attn_output.weight", (d, H * hd), GGUF_BF16), (p + "ffn_norm.weight", (d,), GGUF_F32),
                    (p + "ffn_gate.weight", (F, d), GGUF_BF16), (p + "ffn_up.weight", (F, d), GGUF_BF16),
                    (p + "ffn_down.weight", (d, F), GGUF_BF16)]
    vocab = letters_vocab(V)
    u32 = lambda v: struct.pack("<I", v)                                                    # noqa: E731
    meta = [
        _kv("general.architecture", META_STR, _s("llama")),
        _kv("general.alignment", META_U32, u32(ALIGN)),
        _kv("llama.embedding_length", META_U32, u32(d)),
        _kv("llama.feed_forward_length", META_U32, u32(F)),
        _kv("llama.attention.head_count", META_U32, u32(H)),
        _kv("llama.attention.head_count_kv", META_U32, u32(G)),
        _kv("attention.key_length", META_U32, u32(hd)),
        _kv("llama.block_count", META_U32, u32(L)),
        _kv("llama.context_length", META_U32, u32(int(cfg.get("context", 4096)))),
        _kv("llama.rope.freq_base", META_F32, struct.pack("<f", float(cfg.get("rope_theta", 10000.0)))),
        _kv("llama.attention.layer_norm_rms_epsilon", META_F32, struct.pack("<f", float(cfg["rms_norm_eps"]))),
        _kv("llama.vocab_size", META_U32, u32(V)),
        _kv("tokenizer.ggml.model", META_STR, _s("llama")),
        _kv("tokenizer.ggml.bos_token_id", META_U32, u32(1)),
        _kv("tokenizer.ggml.eos_token_id", META_U32, u32(2)),
        _kv("tokenizer.ggml.add_bos_token", META_BOOL, b"\x01"),
        _kv("tokenizer.ggml.add_space_prefix", META_BOOL, b"\x00"),
        _kv("tokenizer.ggml.tokens", META_ARRAY, u32(META_STR) + struct.pack("<Q", V) + b"".join(_s(t) for t in vocab)),
        _kv("tokenizer.ggml.scores", META_ARRAY, u32(META_F32) + struct.pack("<Q", V) + b"\x00" * (4 * V)),
    ]
    infos, offset = [], 0
    for name, shape, typ in tensors:
        n = 1
        for s in shape:
            n *= s
        dims = tuple(reversed(shape))                        # GGUF lists the innermost dimension first
        infos.append(_s(name) + u32(len(dims)) + b"".join(struct.pack("<Q", x) for x in dims) + u32(typ)
                     + struct.pack("<Q", offset))
        offset += (n * (4 if typ == GGUF_F32 else 2) + ALIGN - 1) // ALIGN * ALIGN
    head = b"GGUF" + u32(3) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(meta)) + b"".join(meta) + b"".join(infos)
    g = torch.Generator().manual_seed(seed)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\x00" * ((len(head) + ALIGN - 1) // ALIGN * ALIGN - len(head)))
        for name, shape, typ in tensors:
            if typ == GGUF_F32:
                raw = torch.ones(shape, dtype=torch.float32).numpy().tobytes()
            else:
                t = torch.empty(shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g).to(torch.bfloat16)
                raw = t.view(torch.int16).numpy().tobytes()
            f.write(raw)
            f.write(b"\x00" * ((len(raw) + ALIGN - 1) // ALIGN * ALIGN - len(raw)))
    return os.path.getsize(path)


# ------------------------------------------------------------------------------- run
_LINE = re.compile(r"^(Prefill|Generation): (\d+) tokens in ([0-9.]+)s \(([0-9.]+) tok/s\)", re.M)


def letters_prompt(n_tokens: int, seed: int) -> str:
    """A text that the letters vocabulary reads as `n_tokens` tokens, the BOS token that the command line
    puts in front included."""
    import random
    r = random.Random(seed)
    return "".join(chr(ord("a") + r.randrange(26)) for _ in range(max(n_tokens - 1, 1)))


def run(binary: str, gguf: str, prompt_tokens: int, new_tokens: int, context: int, gpu: bool = True,
        seed: int = 42, timeout: float = 600.0) -> Dict:
    """One run of the stock command line, greedy (`-t 0 -s 42`, as picolm/bench.zsh runs it).  Returns the
    numbers of its two timing lines and which backend ran."""
    env = dict(os.environ)
    if gpu:
        env["PICOLM_GPU"] = "1"
    else:
        env.pop("PICOLM_GPU", None)
    cmd = [binary, gguf, "-p", letters_prompt(prompt_tokens, seed), "-n", str(new_tokens), "-t", "0", "-s", str(seed),
           "-c", str(context)]
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout, errors="replace")
    wall = time.time() - t0
    found = {m.group(1): (int(m.group(2)), float(m.group(3)), float(m.group(4))) for m in _LINE.finditer(r.stderr)}
    if r.returncode != 0 or "Prefill" not in found or "Generation" not in found:
        tail = " | ".join(r.stderr.strip().splitlines()[-4:])[-400:]
        raise Unavailable(f"the reference's command line ended with code {r.returncode} without its timing lines: {tail}")
    on_gpu = "INFO: GPU initialized" in r.stderr
    return {"prefill_tokens": found["Prefill"][0], "prefill_s": found["Prefill"][1], "prefill_tok_s": found["Prefill"][2],
            "gen_tokens": found["Generation"][0], "gen_s": found["Generation"][1], "gen_tok_s": found["Generation"][2],
            "backend": "cuda" if on_gpu else "cpu", "wall_s": round(wall, 2),
            "stderr_head": [ln for ln in r.stderr.splitlines() if ln.startswith(("INFO", "WARN", "ERROR"))][:8]}
