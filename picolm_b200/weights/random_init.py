"""Random-weights mode: write a model folder (config.json, model.safetensors)
from a typed configuration and a seed.

Matrices are N(0, std), norm weights 1 + N(0, norm_std), drawn on the CPU from
one seeded generator in the sorted order of the tensor names, then stored as
bfloat16 (or float32).  The reference has no such mode (its only random tensors
are in its kernel self-tests, picolm/picolm.c:577-593).
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..config.registry import spec_of
from .safetensors_io import save_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(config, seed: int, std: float = 0.02, norm_std: float = 0.1,
                   store_dtype: str = "bfloat16") -> Dict[str, torch.Tensor]:
    from ..engine.model import Model
    model = Model(spec_of(config), runtime=None)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    dt = _STORE[store_dtype]
    out: Dict[str, torch.Tensor] = {}
    expected = model.expected_tensors()
    for name in sorted(expected):
        ws = expected[name]
        if ws.integer or ws.init == "zeros":
            out[name] = torch.zeros(ws.shape, dtype=torch.int32 if ws.integer else dt)
        elif ws.init == "ones_normal":
            out[name] = (1.0 + norm_std * torch.randn(ws.shape, generator=gen, dtype=torch.float32)).to(dt)
        elif ws.init == "normal":
            out[name] = (std * torch.randn(ws.shape, generator=gen, dtype=torch.float32)).to(dt)
        else:
            raise ValueError(f"tensor {name!r}: unknown init {ws.init!r}")
    return out


def write_random_model(config, seed: int, out_dir: str, std: float = 0.02, norm_std: float = 0.1,
                       store_dtype: str = "bfloat16") -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors`; returns out_dir."""
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(config, seed, std, norm_std, store_dtype)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_std": str(norm_std)})
    cfg = config.to_dict()
    cfg["torch_dtype"] = store_dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    return out_dir
