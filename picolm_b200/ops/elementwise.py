"""Embedding, RMSNorm, SwiGLU, rotary encoding with the cache write."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import PAGE_TOKENS, KernelError, _check, _dev, _dt, _fn, _i32, _p, _stream, set_bounds


def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, :] = float(table[tokens[t], :]) as the fp32 residual stream."""
    _i32(tokens, "tokens")
    _dev(table, "table")
    n, (vocab, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, d), dtype=torch.float32, device=table.device)
    _check(_fn("elementwise", "plm_embed")(_p(tokens), _p(table), _dt(table, "table"), _p(out), n, d, vocab, _stream()),
           "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the fp32 stream `x` [T, d].  With `delta` the sum x + delta is
    normalised and, unless `rows` gathers, written back to x.  `rows` (int32)
    picks the source rows; the output then has len(rows) rows."""
    _dev(x, "x")
    _dev(weight, "weight")
    if x.dtype != torch.float32:
        raise KernelError("the residual stream must be float32")
    T, d = x.shape
    if weight.shape != (d,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, the stream is {d} wide")
    if hasattr(delta, "compute"):                          # a product that has not run yet (gemm.PendingLinear)
        if rows is None and delta.adds_in_place(x):        # many rows: the add in the product's epilogue
            delta.add_into(x)
            delta = None
        else:
            delta = delta.compute()
    if delta is not None:
        _dev(delta, "delta")
        if delta.dtype != torch.float32 or delta.shape != x.shape:
            raise KernelError("delta must be float32 and shaped like x")
    n_rows = T
    if rows is not None:
        _i32(rows, "rows")
        n_rows = rows.numel()
    if out is None:
        out = torch.empty((n_rows, d), dtype=out_dtype, device=x.device)
    set_bounds("elementwise", n_rows=T, device=x.device)
    _check(_fn("elementwise", "plm_rmsnorm")(
        _p(x), _p(delta), _p(weight), _dt(weight, "weight"), _p(out), _dt(out, "out"), _p(rows), n_rows, d,
        float(eps), _stream()), f"rmsnorm rows={n_rows} d={d}",
        nbytes=n_rows * d * (4 + (8 if delta is not None else 0) + out.element_size()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """x[rows] for a 2-D `x` with contiguous rows and int32 `rows` on the device: [len(rows), x.shape[1]]."""
    _i32(rows, "rows")
    if not x.is_cuda:
        raise KernelError(f"x is on {x.device}; picolm_b200 kernels run on a CUDA device only")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gather_rows takes a matrix with contiguous rows")
    n, d = rows.numel(), x.shape[1]
    out = torch.empty((n, d), dtype=x.dtype, device=x.device)
    set_bounds("elementwise", n_rows=x.shape[0], device=x.device)
    _check(_fn("elementwise", "plm_gather_rows")(_p(x), _p(out), _p(rows), n, d * x.element_size(),
                                                x.stride(0) * x.element_size(), _stream()),
           f"gather_rows {n} of {x.shape[0]}", nbytes=2 * n * d * x.element_size())
    return out


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """gate_up [T, 2F] (gate columns first) -> act(gate) * up, [T, F]; `activation` "silu" or "gelu_tanh"
    (the reference's two: picolm/tensor.c:3306-3323)."""
    _dev(gate_up, "gate_up")
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"activation {activation!r} has no kernel; known: {', '.join(GATE_ACTIVATIONS)}")
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("gate_up must have an even number of columns")
    if out is None:
        out = torch.empty((T, F2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", "plm_swiglu")(_p(gate_up), _p(out), _dt(gate_up, "gate_up"),
                                            GATE_ACTIVATIONS[activation], T, F2 // 2, _stream()), "swiglu")
    return out


def rope_store(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
               num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, pairing: str,
               store: bool = True) -> None:
    """Rotate the query and key heads of `qkv` [T, (H+2G)*hd] by their tokens'
    positions; write queries to `q_out` [T, H, hd] and keys/values into the paged
    cache [pages, G, PAGE_TOKENS, hd]."""
    _dev(qkv, "qkv")
    _dev(q_out, "q_out")
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if qkv.shape[1] != (H + 2 * G) * hd or q_out.shape != (T, H, hd) or q_out.dtype != qkv.dtype:
        raise KernelError("rope_store: qkv / q_out shapes do not match the head counts")
    if store:
        for c, n in ((k_cache, "k_cache"), (v_cache, "v_cache")):
            _dev(c, n)
            if c.dtype != q_out.dtype or c.shape[1:] != (G, PAGE_TOKENS, hd):
                raise KernelError(f"rope_store: {n} must be [pages, {G}, {PAGE_TOKENS}, {hd}] of {q_out.dtype}")
    if cos is not None:
        _dev(cos, "cos"), _dev(sin, "sin")
        if cos.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rope_store: cos/sin tables must be float32 [positions, rotary_dim/2]")
    if pairing not in ("half", "adjacent"):
        raise KernelError(f"rope_store: unknown pairing {pairing!r}")
    set_bounds("elementwise", n_pages=k_cache.shape[0] if store else 0, n_seqs=block_table.shape[0],
               n_positions=block_table.shape[1] * PAGE_TOKENS, device=qkv.device)
    _check(_fn("elementwise", "plm_rope_store")(
        _p(qkv), _p(q_out), _p(k_cache) if store else None, _p(v_cache) if store else None, _dt(qkv, "qkv"),
        _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(block_table), block_table.shape[1], T, H, G, hd,
        rotary_dim, 0 if pairing == "half" else 1, 1 if store else 0, _stream()), "rope_store")
