"""Products of a decode step that have not run yet and feed one another, run together by one persistent
kernel (csrc/decode_chain.cu): a layer's output projection with the residual add and the next norm's
weight, the gate/up projection with SwiGLU, the down projection with the residual add, and the next
layer's query/key/value projection are four launches when run one by one and one when run as a chain.

The parts do not know: a mixer or feed-forward hands back its last product unrun (`PendingLinear`), a norm
that may leave its scale to the next product returns `ScaledRows`, and a feed-forward may get `LazyRows`
back from `linear_swiglu(..., defer=True)`; while such objects are only handed on to other products, the
products collect in a `Chain`, and the first caller that needs a tensor runs it.

Chains are OFF unless PICOLM_B200_CHAIN=1 is set (or a test switches `ENABLED` on): measured inside a captured
step at the Llama-3.2-1B widths the four products take 34 us launched one by one and 66 us as a chain.  The chain's
results are right and do not depend on the batch (tests/test_gpu_chain.py); its time goes to the seven meetings
of all CTAs at a counter in global memory and the sums between them, each a dependent round trip through the
second-level cache of 2 to 4 us while the weights stream, and to a producer thread that asks for a block every
0.45 us; profiles/decode_chain_1b_t8.md has the trace."""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from ._lib import KernelError, _check, _fn, _p, _stream, status_word

RESIDUAL, SWIGLU, SCALED, PLAIN = 0, 1, 2, 3
MAX_PHASES = 4
MAX_TOKENS = int(os.environ.get("PICOLM_B200_CHAIN_TOKENS", "64"))     # chains are built for steps of at most this many tokens
ENABLED = os.environ.get("PICOLM_B200_CHAIN", "0") == "1"


class _Phase(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("w", ctypes.c_void_p), ("ldw", ctypes.c_longlong),
                ("a", ctypes.c_void_p), ("lda", ctypes.c_longlong),
                ("out", ctypes.c_void_p), ("ldo", ctypes.c_longlong),
                ("resid", ctypes.c_void_p), ("ld_resid", ctypes.c_longlong),
                ("norm_w", ctypes.c_void_p), ("ss_out", ctypes.c_void_p), ("ss_in", ctypes.c_void_p),
                ("size", ctypes.c_int), ("eps", ctypes.c_float)]


LAUNCHES = [0]                    # chains launched so far (tests and the launch counter read it)
_configured = False
_n_ctas = 0
_sync = {}
_scratch_floats = {}


def _library():
    global _configured, _n_ctas
    lib_fn = _fn("decode_chain", "plm_decode_chain")
    if not _configured:
        ctas = _fn("decode_chain", "plm_decode_chain_ctas")
        _n_ctas = int(ctas())
        scratch = _fn("decode_chain", "plm_decode_chain_scratch")
        scratch.restype = ctypes.c_longlong
        _configured = True
    return lib_fn


def n_ctas() -> int:
    """CTAs of the chain kernel: the rows of a table of partial sums of squares that it writes."""
    _library()
    return _n_ctas


def wanted(n_tokens: int) -> bool:
    """Whether the products of a step of `n_tokens` tokens are collected in chains."""
    return ENABLED and 0 < n_tokens <= MAX_TOKENS


def _scratch(N: int, K: int, T: int) -> int:
    key = (N, K, 16 if T <= 16 else (32 if T <= 32 else 64))
    v = _scratch_floats.get(key)
    if v is None:
        _library()
        v = int(_fn("decode_chain", "plm_decode_chain_scratch")(N, K, T))
        _scratch_floats[key] = v
    return v


class Chain:
    def __init__(self, a: torch.Tensor):
        """`a`: the first product's input, bfloat16 [T, K], contiguous, on the device."""
        self.a = a
        self.T = a.shape[0]
        self.phases: List[dict] = []
        self.launched = 0

    @property
    def pending(self) -> bool:
        return bool(self.phases)

    def _input(self) -> torch.Tensor:
        return self.phases[-1]["out"] if self.phases else self.a

    def _add(self, **phase) -> None:
        if len(self.phases) == MAX_PHASES:                # the kernel takes four: run them, go on from their output
            last = self.phases[-1]["out"]
            self.run()
            self.a = last
        phase["a"] = self._input()
        if phase["a"].dtype != torch.bfloat16 or phase["a"].shape != (self.T, phase["w"].shape[1]):
            raise KernelError(f"chain: a product of {tuple(phase['w'].shape)} cannot take rows {tuple(phase['a'].shape)} "
                              f"of {phase['a'].dtype}")
        self.phases.append(phase)

    def add_residual(self, w: torch.Tensor, x: torch.Tensor, norm_w: torch.Tensor):
        """x += a @ w^T in place; returns (bf16(x * norm_w), the table of partial sums of squares)."""
        N = w.shape[0]
        xw = torch.empty((self.T, N), dtype=torch.bfloat16, device=x.device)
        parts = torch.empty((n_ctas(), 64), dtype=torch.float32, device=x.device)
        self._add(kind=RESIDUAL, w=w, out=xw, resid=x, norm_w=norm_w, ss_out=parts)
        return xw, parts

    def add_swiglu(self, w_gate_up: torch.Tensor, parts: torch.Tensor, size: int, eps: float) -> torch.Tensor:
        out = torch.empty((self.T, w_gate_up.shape[0] // 2), dtype=torch.bfloat16, device=w_gate_up.device)
        self._add(kind=SWIGLU, w=w_gate_up, out=out, ss_in=parts, size=size, eps=eps)
        return out

    def add_scaled(self, w: torch.Tensor, parts: torch.Tensor, size: int, eps: float) -> torch.Tensor:
        out = torch.empty((self.T, w.shape[0]), dtype=torch.bfloat16, device=w.device)
        self._add(kind=SCALED, w=w, out=out, ss_in=parts, size=size, eps=eps)
        return out

    def add_plain(self, w: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.T, w.shape[0]), dtype=torch.float32, device=w.device)
        self._add(kind=PLAIN, w=w, out=out)
        return out

    def run(self) -> None:
        """Launch what has collected (nothing, if nothing has)."""
        if not self.phases:
            return
        fn = _library()
        dev = self.a.device
        arr = (_Phase * len(self.phases))()
        floats = 0
        for i, ph in enumerate(self.phases):
            w, a, out = ph["w"], ph["a"], ph["out"]
            N, K = w.shape
            floats = max(floats, _scratch(N, K, self.T))
            p = arr[i]
            p.kind, p.N, p.K = ph["kind"], N, K
            p.w, p.ldw = w.data_ptr(), w.stride(0)
            p.a, p.lda = a.data_ptr(), a.stride(0)
            p.out, p.ldo = out.data_ptr(), out.stride(0)
            resid = ph.get("resid")
            p.resid, p.ld_resid = (resid.data_ptr(), resid.stride(0)) if resid is not None else (None, 0)
            p.norm_w = ph["norm_w"].data_ptr() if ph.get("norm_w") is not None else None
            p.ss_out = ph["ss_out"].data_ptr() if ph.get("ss_out") is not None else None
            p.ss_in = ph["ss_in"].data_ptr() if ph.get("ss_in") is not None else None
            p.size, p.eps = int(ph.get("size", 0)), float(ph.get("eps", 0.0))
        partial = torch.empty((floats,), dtype=torch.float32, device=dev)
        sync = _sync.get(dev)
        if sync is None:
            sync = _sync[dev] = torch.zeros(2, dtype=torch.int32, device=dev)
        n = len(self.phases)
        keep = self.phases                                    # the operands stay alive until the launch is queued
        self.phases = []
        _check(fn(arr, n, self.T, _p(partial), _p(sync), _p(status_word(dev)), _stream()), "decode_chain")
        self.launched += 1
        LAUNCHES[0] += 1
        del keep


class LazyRows:
    """The bfloat16 rows [T, F] that a product of a chain writes when the chain runs.  Handed to another
    product (`linear(..., defer=True)`) they stay unrun; `materialize()` runs the chain and gives the tensor."""
    __slots__ = ("chain", "rows")

    def __init__(self, chain: Chain, rows: torch.Tensor):
        self.chain, self.rows = chain, rows

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device

    def materialize(self) -> torch.Tensor:
        self.chain.run()
        return self.rows
