"""What stands behind the C functions of plm.h inside the interpreter: handles for models and contexts,
and the calls themselves on the library's one engine.  Arguments arrive as plain ints, strings and
memoryviews over the caller's arrays; nothing here computes anything of its own.

The reference's counterparts are `model_load` / `model_forward` / `model_forward_prefill` / `model_free`
(picolm/model.h:504-551); its one sequence per model becomes a context with slots here.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np

_models: Dict[int, object] = {}
_contexts: Dict[int, "Context"] = {}
_next_handle = [1]


def _new_handle(table: dict, obj) -> int:
    h = _next_handle[0]
    _next_handle[0] += 1
    table[h] = obj
    return h


def _ints(mv, n: Optional[int] = None) -> np.ndarray:
    a = np.frombuffer(mv, dtype=np.int32)
    return a if n is None else a[:n]


class LoadedModel:
    def __init__(self, model, config):
        self.model, self.config = model, config


class Context:
    """An engine over one model, and which of the caller's slot numbers holds which sequence of the cache."""

    def __init__(self, engine, n_slots: int):
        self.engine, self.n_slots = engine, n_slots
        self.held: Dict[int, int] = {}                  # the caller's slot -> the cache's slot

    def cache_slot(self, slot: int, create: bool) -> Optional[int]:
        if not 0 <= slot < self.n_slots:
            raise ValueError(f"slot {slot} is outside [0, {self.n_slots})")
        if slot not in self.held and create:
            self.held[slot] = self.engine.new_sequence()
        return self.held.get(slot)

    def reset(self, slot: int) -> None:
        s = self.cache_slot(slot, create=False)
        if s is not None:
            self.engine.end_sequence(s)
            del self.held[slot]


# ------------------------------------------------------------------------------- configuration
def config_json(path: str) -> str:
    from .. import architectures  # noqa: F401
    from ..config.registry import read_config
    return json.dumps(read_config(path).to_dict())


# -------------------------------------------------------------------------------------- models
def _load(model_dir: str, dtype: str) -> int:
    from .. import architectures  # noqa: F401
    from ..config.registry import read_config, spec_of
    from ..engine.model import Model
    from ..runtime import Runtime
    from ..weights.loader import load_weights
    config = read_config(model_dir)
    model = Model(spec_of(config), Runtime.create(dtype, "cuda:0"))
    load_weights(model, model_dir)
    return _new_handle(_models, LoadedModel(model, config))


def model_load(model_dir: str, dtype: str) -> int:
    return _load(model_dir, dtype)


def model_random(config_path: str, seed: int, dtype: str, out_dir: str) -> int:
    from .. import architectures  # noqa: F401
    from ..config.registry import read_config
    from ..weights import write_random_model
    write_random_model(read_config(config_path), int(seed), out_dir)
    return _load(out_dir, dtype)


def model_free(handle: int) -> None:
    import gc
    import torch
    m = _models.pop(handle)
    for h in [h for h, c in _contexts.items() if c.engine.model is m.model]:
        ctx_free(h)
    del m
    gc.collect()
    torch.cuda.empty_cache()


def model_vocab_size(handle: int) -> int:
    return int(_models[handle].model.spec.vocab_size)


# ------------------------------------------------------------------------------------ contexts
def ctx_create(model_handle: int, n_slots: int, max_context: int) -> int:
    from ..engine.engine import Engine
    if n_slots <= 0:
        raise ValueError("n_slots must be positive")
    m = _models[model_handle]
    limit = m.model.spec.max_positions
    ctx = min(max_context or limit, limit)
    engine = Engine(m.model, max_tokens=n_slots * ((ctx + 63) // 64 * 64), max_seqs=n_slots, max_seq_tokens=ctx)
    engine.config = m.config
    return _new_handle(_contexts, Context(engine, n_slots))


def ctx_free(handle: int) -> None:
    import gc
    c = _contexts.pop(handle)
    c.engine.cache = None
    del c
    gc.collect()


def slot_reset(handle: int, slot: int) -> None:
    _contexts[handle].reset(slot)


def slot_length(handle: int, slot: int) -> int:
    c = _contexts[handle]
    s = c.cache_slot(slot, create=False)
    return 0 if s is None else c.engine.length(s)


# ---------------------------------------------------------------------------------------- step
def step(handle: int, n_seqs: int, slots_mv, n_new_mv, tokens_mv, rows_mv, n_rows: int, logits_mv) -> None:
    c = _contexts[handle]
    slots, n_new = _ints(slots_mv, n_seqs).tolist(), _ints(n_new_mv, n_seqs).tolist()
    if any(n <= 0 for n in n_new):
        raise ValueError("every sequence must bring at least one token")
    tokens = _ints(tokens_mv, sum(n_new)).tolist()
    if len(set(slots)) != len(slots):
        raise ValueError("a slot occurs twice in one step")
    offs = [0]
    for n in n_new:
        offs.append(offs[-1] + n)
    if rows_mv is None:
        wants = [[n - 1] for n in n_new]
    else:
        wants: List[List[int]] = [[] for _ in slots]
        rows = _ints(rows_mv, n_rows).tolist()
        if rows != sorted(rows):
            raise ValueError("logit_rows must be in ascending order")
        for r in rows:
            if not 0 <= r < offs[-1]:
                raise ValueError(f"logit row {r} is outside the step's {offs[-1]} tokens")
            i = next(i for i in range(len(slots)) if r < offs[i + 1])
            wants[i].append(r - offs[i])
    fresh = [s for s in slots if s not in c.held]
    entries = [(c.cache_slot(s, create=True), tokens[offs[i]:offs[i + 1]]) for i, s in enumerate(slots)]
    try:
        logits = c.engine.step(entries, wants)
    except Exception:
        for s in fresh:                                    # the step changed nothing: neither do the slots
            c.reset(s)
        raise
    if logits is not None:
        out = np.frombuffer(logits_mv, dtype=np.float32)
        flat = logits.reshape(-1).cpu().numpy()
        if out.size < flat.size:
            raise ValueError("logits_out is too small")
        out[:flat.size] = flat


def sample(handle: int, logits_mv, rows: int, temperature: float, top_k: int, top_p: float, min_p: float,
           rng_mv, out_mv) -> None:
    import torch
    from .. import ops
    c = _contexts[handle]
    vocab = c.engine.vocab_size
    dev = c.engine.runtime.device
    logits = torch.from_numpy(np.frombuffer(logits_mv, dtype=np.float32)[:rows * vocab].reshape(rows, vocab).copy()).to(dev)
    if temperature <= 0.0:
        toks = ops.argmax(logits)
    else:
        rng = np.frombuffer(rng_mv, dtype=np.int64)[:rows]
        state = torch.from_numpy(rng.copy()).to(dev)
        toks = ops.sample(logits, state, temperature, top_k, top_p, min_p)
        rng[:] = state.cpu().numpy()
    np.frombuffer(out_mv, dtype=np.int32)[:rows] = toks.cpu().numpy()


def generate(handle: int, prompt_mvs, max_new: int, temperature: float, top_k: int, top_p: float, min_p: float,
             seed: int, stop_mv, n_stop: int, out_mvs, out_lens_mv) -> None:
    from ..engine.generate import generate as run
    from ..sampling import SamplingParams
    c = _contexts[handle]
    if c.held:
        raise ValueError("plm_generate needs a context whose slots are all empty")
    prompts = [_ints(mv).tolist() for mv in prompt_mvs]
    stop = None if stop_mv is None else _ints(stop_mv, n_stop).tolist()
    params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p, seed=seed)
    outputs, _ = run(c.engine, prompts, max_tokens=max_new, sampling=params, stop_ids=stop, max_batch=c.n_slots)
    lens = np.frombuffer(out_lens_mv, dtype=np.int32)
    for i, (toks, mv) in enumerate(zip(outputs, out_mvs)):
        np.frombuffer(mv, dtype=np.int32)[:len(toks)] = toks
        lens[i] = len(toks)


def classify(exc: BaseException) -> int:
    """The C API's code for an exception."""
    from ..cache.allocator import CacheFull
    if isinstance(exc, CacheFull):
        return 2
    if isinstance(exc, (ValueError, IndexError, KeyError, TypeError)):
        return 3
    return 1
