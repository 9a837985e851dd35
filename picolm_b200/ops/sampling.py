"""Token selection on the device: argmax and the reference's sampling chain."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, _check, _dev, _fn, _p, _stream


def _token_out(out: Optional[torch.Tensor], n: int, like: torch.Tensor, what: str) -> torch.Tensor:
    """The int32 [n] result tensor of a sampling kernel: `out` if it is one, on the logits' device."""
    if out is None:
        return torch.empty((n,), dtype=torch.int32, device=like.device)
    if (out.dtype != torch.int32 or out.dim() != 1 or out.numel() != n or out.device != like.device
            or not out.is_contiguous()):
        raise KernelError(f"{what}: out must be a contiguous int32 [{n}] tensor on {like.device}, got "
                          f"{out.dtype} {tuple(out.shape)} on {out.device}")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum, int32 [rows]."""
    _dev(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("logits must be float32")
    n, V = logits.shape
    out = _token_out(out, n, logits, "argmax")
    _check(_fn("sampling", "plm_argmax")(_p(logits), V, n, V, _p(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, rng_state: torch.Tensor, temperature: float, top_k: int, top_p: float,
           min_p: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row by the reference's chain (top-k, top-p, min-p, p^(1/T));
    `rng_state` (int64 [rows], xorshift64 states) is advanced in place."""
    _dev(logits, "logits"), _dev(rng_state, "rng_state")
    if logits.dtype != torch.float32 or rng_state.dtype != torch.int64:
        raise KernelError("sample: logits must be float32 and rng_state int64")
    n, V = logits.shape
    if rng_state.numel() != n:
        raise KernelError("sample: one rng state per row is needed")
    if V > 8 * 40 * 1024:
        raise KernelError(f"sample: a vocabulary of {V} exceeds {8 * 40 * 1024}, the most the sampling kernel keeps "
                          f"in the shared memory of its eight CTAs")
    out = _token_out(out, n, logits, "sample")
    _check(_fn("sampling", "plm_sample")(
        _p(logits), V, n, V, float(temperature), int(top_k), float(top_p), float(min_p), _p(rng_state), _p(out),
        _stream()), "sample")
    return out
