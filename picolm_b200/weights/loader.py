"""Weights by tensor name from a model folder's safetensors files.

Every tensor that the model's parts name must be there with the exact shape;
what is missing, what has another shape or an unusable element type, and what the
folder holds beyond that are all reported in one error.  (The reference checks
only that layer 0's attention tensors exist and never a shape,
picolm/safetensors.c:509-512, and silently ties a missing head to the embedding,
picolm/safetensors.c:248-251.)

Element types.  In a bfloat16 run BF16 tensors are used as stored, F16 tensors
are rounded to bfloat16, F32 tensors stay float32, integer tables become int32.
In a float32 run every floating tensor is widened to float32, which is exact.
Two parts that name the same tensor (tied embeddings) get the same device buffer.
"""
from __future__ import annotations

import re
from typing import Dict

import torch

from ..parts import WeightSpec
from .safetensors_io import Checkpoint

_FLOATS = {"BF16", "F16", "F32"}
_INTS = {"I64", "I32", "I16", "I8", "U8"}


class WeightsError(ValueError):
    """The checkpoint does not match the model.  `missing`, `unexpected`,
    `wrong_shape` and `wrong_dtype` hold the details that the message lists."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n}  expected shape {list(s)}" for n, s in self.missing]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {n}  expected {list(e)}, found {list(g)}" for n, e, g in self.wrong_shape]
        if self.wrong_dtype:
            lines.append(f"  unusable element types ({len(self.wrong_dtype)}):")
            lines += [f"    {n}  found {d}, {why}" for n, d, why in self.wrong_dtype]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}" for n in self.unexpected]
        super().__init__("\n".join(lines))


def check_checkpoint(expected: Dict[str, WeightSpec], ckpt: Checkpoint, ignored=()) -> None:
    """Raise one `WeightsError` that lists every mismatch, or return."""
    ignore = [re.compile(p) for p in ignored]
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, ws in expected.items():
        ent = ckpt.entries.get(name)
        if ent is None:
            missing.append((name, ws.shape))
            continue
        if tuple(ent.shape) != tuple(ws.shape):
            wrong_shape.append((name, ws.shape, ent.shape))
        if ws.integer and ent.dtype not in _INTS:
            wrong_dtype.append((name, ent.dtype, "an integer table is expected"))
        elif not ws.integer and ent.dtype not in _FLOATS:
            wrong_dtype.append((name, ent.dtype, "BF16, F16 or F32 is expected"))
    unexpected = sorted(n for n in ckpt.names() if n not in expected and not any(p.search(n) for p in ignore))
    if missing or wrong_shape or wrong_dtype or unexpected:
        raise WeightsError(ckpt.model_dir, missing, unexpected, wrong_shape, wrong_dtype)


def to_run_dtype(t: torch.Tensor, ws: WeightSpec, run_dtype: torch.dtype) -> torch.Tensor:
    if ws.integer:
        return t.to(torch.int32)
    if run_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype == torch.float32:
        return t                              # stored in 32 bits: stays so
    return t.to(torch.bfloat16)


def load_weights(model, model_dir: str) -> None:
    """Check the folder against `model.expected_tensors()` and hand the tensors
    to the model's parts on its device."""
    ckpt = Checkpoint(model_dir)
    try:
        expected = model.expected_tensors()
        check_checkpoint(expected, ckpt, model.spec.ignored_tensors)
        rt = model.runtime
        on_device: Dict[str, torch.Tensor] = {}

        def get(name: str) -> torch.Tensor:
            t = on_device.get(name)
            if t is None:
                t = to_run_dtype(ckpt.tensor(name), expected[name], rt.dtype).to(rt.device).contiguous()
                on_device[name] = t
            return t

        model.load_tensors(get)
    finally:
        ckpt.close()
