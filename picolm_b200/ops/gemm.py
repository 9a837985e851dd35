"""Matrix products: the CUDA-core kernel, the tcgen05 kernels for decode-shaped and prompt-shaped
problems, the pieces of an RMSNorm that two products share, and the dispatcher `linear`."""
from __future__ import annotations

from typing import Optional

import torch

from . import chain as _chain
from ._lib import (SM_COUNT, KernelError, _check, _dev, _dt, _fn, _p, _stream, status_word, stream_space,
                   stream_space_enabled)
from .chain import LazyRows


def _work(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, extra: int = 0) -> dict:
    """What a product has to move and compute: both operands and the result once, 2 M N K flops."""
    return {"nbytes": a.numel() * a.element_size() + w.numel() * w.element_size() + out.numel() * out.element_size() + extra,
            "flops": 2 * a.shape[0] * w.shape[0] * w.shape[1]}


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores, fp32 accumulation."""
    _dev(a, "a"), _dev(w, "w")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is [{M}, {K}] but w is [{N}, {K2}]")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _check(_fn("gemm_simt", "plm_gemm_simt")(
        _p(a), _dt(a, "a"), _p(w), _dt(w, "w"), _p(out), _dt(out, "out"), M, N, K, K, K, N, _stream()),
        f"gemm_simt {M}x{N}x{K}", **_work(a, w, out))
    return out


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes a @ w^T: both bfloat16, K a multiple of
    8 (rows start on 16-byte boundaries, as TMA needs) and at least one K block."""
    if isinstance(a, LazyRows):
        a = a.rows
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    (M, K), (N, K2) = a.shape, w.shape
    if K != K2 or K < 64:
        return False
    # TMA's rule (the kernels check it again): rows start on 16-byte boundaries
    return (M > 0 and N > 0 and K % 8 == 0 and a.is_contiguous() and w.is_contiguous()
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_skinny(a, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decode-shaped tensor-core product: a [M <= 64, K] @ w [N, K]^T with the weights on the MMA's 128
    rows and K split over a thread-block cluster whose CTAs add their partial tiles up through distributed
    shared memory.  With `swiglu`, w holds tiles of 64 gate rows followed by their 64 up rows (see
    `interleave_gate_up`) and the result is silu(gate) * up, [M, N/2] in bfloat16.  `a` may be `ScaledRows`
    (an RMSNorm whose scale is still due): the epilogue then scales each row of the result, in bfloat16."""
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
        scaled.ready()
        a = scaled.x
        if out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc_skinny: rows with a scale that is still due give a bfloat16 result only")
    _dev(a, "a"), _dev(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if M > 64 or not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc_skinny: needs a supported bfloat16 problem with at most 64 rows")
    if swiglu:
        if N % 128:
            raise KernelError("gemm_tc_skinny: the interleaved gate/up matrix must have a multiple of 128 rows")
        out_dtype = torch.bfloat16
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=a.device)
    if scaled is not None:
        _check(_fn("gemm_tc_skinny", "plm_gemm_tc_skinny_scaled")(
            _p(a), _p(w), _p(out), 1 if swiglu else 0, M, N, K, K, K, n_out, _p(scaled.parts), scaled.parts.shape[0],
            scaled.parts.shape[1], scaled.size, float(scaled.eps), _p(status_word(a.device)), _stream()),
            f"gemm_tc_skinny{'_swiglu' if swiglu else ''}_scaled {M}x{N}x{K}", **_work(a, w, out))
        return out
    _check(_fn("gemm_tc_skinny", "plm_gemm_tc_skinny")(
        _p(a), _p(w), _p(out), _dt(out, "out"), 1 if swiglu else 0, M, N, K, K, K, n_out,
        _p(status_word(a.device)), _stream()), f"gemm_tc_skinny{'_swiglu' if swiglu else ''} {M}x{N}x{K}", **_work(a, w, out))
    return out


class PendingLinear:
    """a [M, K] @ w [N, K]^T in float32 that has not run yet: the last product of a mixer or a
    feed-forward, whose result is a delta for the residual stream.  The norm that follows may run it
    with the residual add and its own weight in the epilogue (`linear_residual_norm`); anything else
    calls `compute()`."""
    __slots__ = ("a", "w")

    def __init__(self, a, w: torch.Tensor):
        self.a, self.w = a, w                  # a: a tensor, or `LazyRows` of a chain that has not run

    @property
    def shape(self):
        return (self.a.shape[0], self.w.shape[0])

    def compute(self) -> torch.Tensor:
        if isinstance(self.a, LazyRows):       # the chain's last product, with a plain fp32 result
            out = self.a.chain.add_plain(self.w)
            self.a.chain.run()
            return out
        return linear(self.a, self.w, torch.float32)

    def adds_in_place(self, x: torch.Tensor) -> bool:
        """Whether `add_into(x)` runs as one kernel: a product of more than 64 rows for the tensor cores
        with enough tiles for the SMs, and an fp32 stream of its shape."""
        if (isinstance(self.a, LazyRows) or self.a.shape[0] <= 64 or x.dtype != torch.float32
                or not x.is_contiguous() or tuple(x.shape) != tuple(self.shape) or x.data_ptr() % 16):
            return False
        # where the tiles are few the plain product cuts K into parts through scratch memory, which this epilogue cannot
        return _fn("gemm_tc_wide", "plm_gemm_tc_wide_splits")(self.a.shape[0], self.w.shape[0], self.a.shape[1]) == 1

    def add_into(self, x: torch.Tensor) -> None:
        """x += a @ w^T in place, the add in the product's epilogue: the delta never goes through memory."""
        if not self.adds_in_place(x):
            x.add_(self.compute())
            return
        gemm_tc_wide(self.a, self.w, torch.float32, out=x, add=True,
                     pair=pair_pays(self.a.shape[0], self.w.shape[0], self.a.shape[1], 2))


class ScaledRows:
    """An RMSNorm whose scale is still due: `x` [T, size] in bfloat16 holds row * norm weight, and
    `parts` [n, >= T] partial sums of squares of the rows (column t for row t), so that the normalised
    row t is x[t] / sqrt(sum(parts[:, t]) / size + eps).  A product takes it as its left operand and
    applies the scale to its result (`linear`, `linear_swiglu`); `materialize()` gives the rows."""
    __slots__ = ("x", "parts", "size", "eps", "chain")

    def __init__(self, x: torch.Tensor, parts: torch.Tensor, size: int, eps: float, chain=None):
        self.x, self.parts, self.size, self.eps = x, parts, size, eps
        self.chain = chain                     # a chain whose run writes x and parts (None: they are written)

    def ready(self) -> None:
        """Run the chain that writes these rows, if it has not run."""
        if self.chain is not None:
            self.chain.run()
            self.chain = None

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    @property
    def dtype(self):
        return self.x.dtype

    def materialize(self) -> torch.Tensor:
        self.ready()
        out = torch.empty_like(self.x)
        T, d = self.x.shape
        _check(_fn("elementwise", "plm_scale_rows")(
            _p(self.x), _p(self.parts), self.parts.shape[0], self.parts.shape[1], self.size, float(self.eps),
            _p(out), T, d, _stream()), "scale_rows")
        return out


def residual_norm_supported(pending, x: torch.Tensor, norm_weight: torch.Tensor) -> bool:
    """Whether `linear_residual_norm` takes this case: a pending product of at most 64 rows that the
    cluster kernel takes, an fp32 stream of its shape and a bfloat16 norm weight.  (For more rows the
    fused epilogue was measured slower than a norm kernel of its own: there a thread of the epilogue
    holds a row of the tile, and its read-modify-write of the stream does not coalesce.)"""
    return (isinstance(pending, PendingLinear) and pending.a.shape[0] <= 64 and gemm_tc_supported(pending.a, pending.w)
            and x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == tuple(pending.shape)
            and norm_weight.dtype == torch.bfloat16 and norm_weight.shape == (x.shape[1],))


def linear_residual_norm(pending: PendingLinear, x: torch.Tensor, norm_weight: torch.Tensor, eps: float) -> ScaledRows:
    """x += pending (in place, the fp32 residual stream; done when the returned rows are made `ready()`,
    which every product that takes them does) and the RMSNorm of the new x as `ScaledRows`:
    one tensor-core product whose epilogue does the add, applies the norm weight and leaves the rows'
    sums of squares; the scale itself is applied by the product that takes the result."""
    if not residual_norm_supported(pending, x, norm_weight):
        raise KernelError("linear_residual_norm: not a case the fused kernel takes")
    a, w = pending.a, pending.w
    if _chain.wanted(a.shape[0]) and a.shape[0] * (w.shape[0] // SM_COUNT + 2) <= 4096:
        # collected, not run: the product that takes the result decides when (see ops/chain.py)
        ch = a.chain if isinstance(a, LazyRows) else _chain.Chain(a)
        xw, parts = ch.add_residual(w, x, norm_weight)
        return ScaledRows(xw, parts, w.shape[0], eps, chain=ch)
    if isinstance(a, LazyRows):
        a = a.materialize()
    _dev(a, "a"), _dev(w, "w"), _dev(x, "x"), _dev(norm_weight, "norm_weight")
    M, K = a.shape
    N = w.shape[0]
    xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    n_parts = _fn("gemm_tc_skinny", "plm_gemm_tc_skinny_residual_parts")(N, K)
    parts = torch.empty((n_parts, 64), dtype=torch.float32, device=x.device)
    _check(_fn("gemm_tc_skinny", "plm_gemm_tc_skinny_residual")(
        _p(a), _p(w), _p(x), _p(norm_weight), _p(xw), _p(parts), M, N, K, K, K, N, N,
        _p(status_word(x.device)), _stream()), f"gemm_tc_skinny_residual {M}x{N}x{K}", **_work(a, w, x, extra=x.numel() * 4))
    return ScaledRows(xw, parts, N, eps)


def gemm_tc_wide(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                 out: Optional[torch.Tensor] = None, pair: bool = False, add: bool = False) -> torch.Tensor:
    """The prompt-shaped tensor-core product: a [M > 64, K] @ w [N, K]^T by a persistent tcgen05 kernel
    (one CTA per SM, two accumulators in tensor memory so that a tile's epilogue overlaps the next
    tile's main loop; where the tiles do not fill one round over the SMs and K is long, the K blocks of all
    tiles are handed out as one stream, cut into equal ranges).  With `swiglu`, w comes from `interleave_gate_up`
    and the result is silu(gate) * up, [M, N/2] in bfloat16.  With `add`, `out` (float32) += the product.
    `pair`: the same by pairs of CTAs on tiles of 256 x 256 (`tcgen05.mma.cta_group::2`: each CTA of a pair
    loads half of the weight tile)."""
    _dev(a, "a"), _dev(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc_wide: needs bfloat16 operands that TMA can address")
    if swiglu:
        if N % 128:
            raise KernelError("gemm_tc_wide: the interleaved gate/up matrix must have a multiple of 128 rows")
        out_dtype = torch.bfloat16
    n_out = N // 2 if swiglu else N
    if add:
        if swiglu or out is None or out.dtype != torch.float32 or tuple(out.shape) != (M, N) or not out.is_contiguous():
            raise KernelError("gemm_tc_wide: `add` needs a contiguous float32 `out` of the product's shape")
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=a.device)
    epilogue = 2 if add else 1 if swiglu else 0
    name = f"{'_swiglu' if swiglu else '_residual' if add else ''} {M}x{N}x{K}"
    work = _work(a, w, out, extra=out.numel() * 4 if add else 0)
    # Shapes whose tiles leave most SMs idle walk K as one stream: that code is in a build variant of the library
    # (compiled when the first such shape comes), with a workspace; everything else runs the plain build.
    STREAM_LIB = ("gemm_tc_wide@stream", ("-DPLM_WIDE_STREAM",))
    if pair:
        streamed = K % 64 == 0 and stream_space_enabled() and _pair_streamed(M, N, K) > 0
        parts, flags, slots = stream_space(a.device) if streamed else (None, None, 0)
        lib = STREAM_LIB if streamed else ("gemm_tc_wide", ())
        _check(_fn(lib[0], "plm_gemm_tc_pair_space", lib[1])(
            _p(a), _p(w), _p(out), _dt(out, "out"), epilogue, M, N, K, K, K, n_out, _p(parts), _p(flags), slots,
            _p(status_word(a.device)), _stream()), "gemm_tc_pair" + (" (stream)" if streamed else "") + name, **work)
        return out
    scratch, kernels = None, 1
    how = wide_how(M, N, K, epilogue)
    if epilogue == 0 and how[1] > 1:
        # few tiles (a prompt of a few hundred tokens): K is cut into parts that pass through scratch memory
        k_splits = how[1]
        scratch = torch.empty((k_splits, M, N), dtype=torch.float32, device=a.device)
        name = f"(K in {k_splits} parts)" + name
        work = _work(a, w, out, extra=2 * scratch.numel() * 4)
        kernels = 2
    streamed = how[2] > 0
    parts, flags, slots = stream_space(a.device) if streamed else (None, None, 0)
    lib = STREAM_LIB if streamed else ("gemm_tc_wide", ())
    _check(_fn(lib[0], "plm_gemm_tc_wide_space", lib[1])(
        _p(a), _p(w), _p(out), _dt(out, "out"), epilogue, M, N, K, K, K, n_out, _p(scratch), _p(parts), _p(flags), slots,
        _p(status_word(a.device)), _stream()), "gemm_tc_wide" + (" (stream)" if streamed else "") + name, kernels=kernels, **work)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate | up] as one matrix whose rows come in tiles of 64 gate rows followed by the 64 up rows of
    the same features, so that a 128-row MMA tile holds both branches of 64 outputs and the product's
    epilogue can apply SwiGLU.  Needs a number of features that is a multiple of 64."""
    F, K = gate.shape
    if up.shape != gate.shape or F % 64:
        raise KernelError("interleave_gate_up: gate and up must have the same shape with a multiple of 64 rows")
    return torch.stack([gate.view(F // 64, 64, K), up.view(F // 64, 64, K)], dim=1).reshape(2 * F, K).contiguous()


_how_cache = {}
_pair_streamed_cache = {}


def _pair_streamed(m: int, n: int, k: int) -> int:
    """How many pairs walk the stages of (m, n, k)'s tiles as one stream (0: whole tiles)."""
    key = (m, n, k)
    v = _pair_streamed_cache.get(key)
    if v is None:
        v = _pair_streamed_cache[key] = _fn("gemm_tc_wide", "plm_gemm_tc_pair_streamed")(m, n, k, SM_COUNT)
    return v


def wide_how(m: int, n: int, k: int, epilogue: int = 0):
    """(tile width, parts of K through scratch memory, CTAs of the stream walk or 0) of the single-CTA form of the
    prompt-shaped product for this shape; epilogue 0 store, 1 SwiGLU, 2 add."""
    key = (m, n, k, epilogue)
    how = _how_cache.get(key)
    if how is None:
        import ctypes
        out = (ctypes.c_int * 3)()
        slots = SM_COUNT if stream_space_enabled() else 0
        _fn("gemm_tc_wide", "plm_gemm_tc_wide_how")(m, n, k, epilogue, slots, ctypes.cast(out, ctypes.c_void_p))
        how = _how_cache[key] = tuple(out)
    return how


def pair_pays(m: int, n: int, k: int = 0, epilogue: int = 0) -> bool:
    """Whether the prompt-shaped product runs as pairs of CTAs on tiles of 256 x 256: from half a round of
    such tiles for the 74 pairs on (measured faster than single CTAs there: the pairs take two tiles of K per copy,
    and the copies bound the single CTAs), and below that where the pairs can walk the tiles' stages of K as one
    stream (with `k` given: K a multiple of 64, enough stages).  `epilogue` 0 store, 1 SwiGLU, 2 add."""
    if m < 256 or n < 256 or (k and k % 64):
        return False
    tiles = ((m + 255) // 256) * ((n + 255) // 256)
    if tiles >= SM_COUNT // 4:
        return True
    if not k or not stream_space_enabled():
        return False
    if epilogue == 0 and wide_how(m, n, k, 0)[1] > 1:
        return False                            # few tiles, store: the single CTAs cut K through scratch memory
    return _pair_streamed(m, n, k) > 0


def linear_swiglu(a, w_gate_up: torch.Tensor, defer: bool = False):
    """silu(a @ gate^T) * (a @ up^T) with `w_gate_up` from `interleave_gate_up`: one tensor-core product
    whose epilogue applies the activation; [M, F] in bfloat16.  `a` may be `ScaledRows`.  With `defer` (the
    caller hands the result to `linear(..., defer=True)` and nowhere else) the result may be `LazyRows`."""
    if isinstance(a, ScaledRows) and a.chain is not None and a.chain.pending:
        if gemm_tc_supported(a.x, w_gate_up) and w_gate_up.shape[0] % 128 == 0:
            ch = a.chain
            rows = ch.add_swiglu(w_gate_up, a.parts, a.size, a.eps)
            if defer:
                return LazyRows(ch, rows)
            ch.run()
            return rows
        a.ready()
    if isinstance(a, ScaledRows) and not (a.shape[0] <= 64 and gemm_tc_supported(a.x, w_gate_up)):
        a = a.materialize()
    x = a.x if isinstance(a, ScaledRows) else a
    _dev(x, "a"), _dev(w_gate_up, "w_gate_up")
    M, K = x.shape
    N = w_gate_up.shape[0]
    if not gemm_tc_supported(x, w_gate_up) or N % 128:
        raise KernelError("linear_swiglu: needs bfloat16 operands the tensor-core kernel takes and N % 128 == 0")
    if M <= 64:
        return gemm_tc_skinny(a, w_gate_up, torch.bfloat16, swiglu=True)
    return gemm_tc_wide(a, w_gate_up, torch.bfloat16, swiglu=True, pair=pair_pays(M, N, K, 1))


def linear(a, w: torch.Tensor, out_dtype: torch.dtype, defer: bool = False):
    """a [M, K] times w [N, K]^T -> [M, N].  The kernel is chosen by element
    types and shape, never by the model: the tensor cores for bfloat16 operands
    that TMA can address (the cluster kernel for up to 64 rows, the wide kernel
    beyond), the CUDA cores for everything else.

    `a` may be `ScaledRows`.  With `defer` (a float32 delta for the residual stream) the product may
    come back as a `PendingLinear` for the next norm to run; whoever cannot use that calls `compute()`."""
    if isinstance(a, ScaledRows):
        if a.chain is not None and a.chain.pending and out_dtype == torch.bfloat16 and gemm_tc_supported(a.x, w):
            ch = a.chain                           # the chain's last product: run it all
            out = ch.add_scaled(w, a.parts, a.size, a.eps)
            ch.run()
            return out
        if a.shape[0] <= 64 and out_dtype == torch.bfloat16 and gemm_tc_supported(a.x, w):
            return gemm_tc_skinny(a, w, out_dtype)
        a = a.materialize()
    if isinstance(a, LazyRows):
        if defer and out_dtype == torch.float32 and gemm_tc_supported(a, w):
            return PendingLinear(a, w)
        a = a.materialize()
    if defer and out_dtype == torch.float32 and gemm_tc_supported(a, w):
        return PendingLinear(a, w)
    if gemm_tc_supported(a, w):
        if a.shape[0] <= 64:
            return gemm_tc_skinny(a, w, out_dtype)
        return gemm_tc_wide(a, w, out_dtype, pair=pair_pays(a.shape[0], w.shape[0], a.shape[1], 0))
    return gemm_simt(a, w, out_dtype)
