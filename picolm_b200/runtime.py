"""What every part is given besides its own parameters: the device and the
precision of the run.

`bfloat16` is the serving precision: bf16 weights, activations and cache, with
an fp32 residual stream and fp32 statistics.  `float32` is the true 32-bit path:
everything is fp32 and every matrix product runs as plain FFMA (the reference
keeps activations in fp32 but rounds K/V to fp16, picolm/model_core.c:1943-1955,
so it has no such path).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported (bfloat16 or float32)") from None


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype                 # activations, cache and 16-bit weights

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32

    @staticmethod
    def create(dtype="bfloat16", device="cuda:0") -> "Runtime":
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError(
                f"picolm_b200 runs on a CUDA device only (asked for {dev}); there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("picolm_b200 needs a CUDA device and none is available; there is no CPU path")
        return Runtime(dev, parse_dtype(dtype))
