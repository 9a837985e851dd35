"""The Python entry point, in the manner of the reference's `model.h` and
`picolm.c`: `model_load` / `model_free` around a model (picolm/model.h:504-582),
and `generate` with the command line's option names and defaults (`-n` max
tokens 256, `-t` temperature 0.8, `--top-p` 0.9, `-k` top-k 40, `-s` seed 42,
`-c` context; picolm/picolm.c:140-196, :774-776).  Prompts and results are lists
of token ids on the host: the reference's tokenizer is not part of this library.
"""
from __future__ import annotations

from typing import Optional, Sequence

from .engine.engine import Engine
from .engine.generate import generate as _generate
from .sampling import SamplingParams


def model_load(model_dir: str, dtype: str = "bfloat16", context: Optional[int] = None,
               max_batch: int = 8, max_tokens: Optional[int] = None, device: str = "cuda:0") -> Engine:
    """Load a model folder (config.json + safetensors).  `context` bounds the
    length of one sequence (the reference's `-c`, default: the model's own
    limit); the cache is sized for `max_batch` sequences of that length unless
    `max_tokens` (tokens held by all live sequences together) says otherwise."""
    from .config.registry import read_config
    cfg = read_config(model_dir)
    limit = getattr(cfg, "max_position_embeddings", None) or 2048
    ctx = min(context or limit, limit)
    ctx_pages = (ctx + 63) // 64 * 64
    total = max_tokens or ctx_pages * max_batch
    return Engine.from_folder(model_dir, dtype=dtype, max_tokens=total, max_seqs=max(max_batch, 1),
                              max_seq_tokens=ctx, device=device)


def model_free(engine: Engine) -> None:
    """Drop the model's device memory (weights and cache)."""
    import gc
    import torch
    engine.cache = None
    engine.model = None
    gc.collect()
    torch.cuda.empty_cache()


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256, temperature: float = 0.8,
             top_p: float = 0.9, top_k: int = 40, min_p: float = 0.05, seed: int = 42,
             stop_ids: Optional[Sequence[int]] = None, max_batch: Optional[int] = None,
             return_stats: bool = False, steps_per_sync: int = 3):
    """Generate for every prompt (a list of token ids); returns the new tokens
    of each.  `temperature` 0 is greedy.  Prompts are batched as the cache
    allows, batches run one after another.  `steps_per_sync`: how many decode steps may
    be in flight before the host looks at the first one's tokens (1: it waits for every step)."""
    params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p, seed=seed)
    outputs, stats = _generate(engine, prompts, max_tokens=max_tokens, sampling=params, stop_ids=stop_ids,
                               max_batch=max_batch, steps_per_sync=steps_per_sync)
    return (outputs, stats) if return_stats else outputs
