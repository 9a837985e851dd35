"""Python faces of the CUDA kernels.  Every function checks what it is given
(device, dtype, shape, contiguity), launches on the current CUDA stream and
raises `KernelError` if the kernel library refuses or fails.  There is no CPU
path: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import attention_variant, load_library

PAGE_TOKENS = 64            # tokens per cache page; PLM_PAGE in csrc/common.cuh

_DT = {torch.float32: 0, torch.bfloat16: 1}

_vp, _i, _l, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float

_SIGNATURES = {
    "plm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "plm_rmsnorm": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _f, _vp],
    "plm_swiglu": [_vp, _vp, _i, _i, _i, _vp],
    "plm_rope_store": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "plm_gemm_tc_skinny": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_skinny_residual": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _l, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_skinny_residual_parts": [_i, _i],
    "plm_gemm_tc_skinny_scaled": [_vp, _vp, _vp, _i, _i, _i, _i, _l, _l, _l, _vp, _i, _i, _i, _f, _vp, _vp],
    "plm_scale_rows": [_vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp],
    "plm_gemm_tc_wide": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_pair": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _l, _l, _l, _vp],
    "plm_gemm_tc": [_vp, _vp, _vp, _i, _i, _i, _i, _l, _l, _l, _vp, _vp, _vp],
    "plm_gemm_tc_plan": [_i, _i, _i, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_long)],
    "plm_gemm_tc_supported": [_vp, _vp, _i, _i, _i, _l, _l],
    "plm_attention_rows": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
    "plm_attn_prefill": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
    "plm_attn_tc_prefill": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp],
    "plm_attn_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp],
    "plm_attn_decode_rope": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _vp],
    "plm_argmax": [_vp, _l, _i, _i, _vp, _vp],
    "plm_sample": [_vp, _l, _i, _i, _f, _i, _f, _f, _vp, _vp, _vp],
}
_fn_cache = {}


class KernelError(RuntimeError):
    pass


_CODES = {-1: "unsupported element type", -2: "bad shape", -3: "bad alignment", -4: "unsupported option",
          -5: "the device wait ran out (see the status word)"}


def _fn(library: str, name: str, extra_flags=()):
    key = (library, name, tuple(extra_flags))
    f = _fn_cache.get(key)
    if f is None:
        lib = load_library(library, extra_flags)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        _fn_cache[key] = f
    return f


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (one per successful call of
    an entry point that launches one kernel)."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels that ran (or did not run) outside `_check`: the replays of a CUDA graph."""
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: refused ({_CODES.get(code, code)})")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        return torch.cuda.cudart().cudaGetErrorString(code)  # type: ignore[attr-defined]
    except Exception:
        return "see cudaError_t"


def _dev(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; picolm_b200 kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name} has dtype {t.dtype}; float32 and bfloat16 are supported")
    return _DT[t.dtype]


def _i32(t: torch.Tensor, name: str) -> None:
    _dev(t, name)
    if t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


# ---------------------------------------------------------------- elementwise
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
    if isinstance(delta, PendingLinear):
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
    _check(_fn("elementwise", "plm_rmsnorm")(
        _p(x), _p(delta), _p(weight), _dt(weight, "weight"), _p(out), _dt(out, "out"), _p(rows), n_rows, d,
        float(eps), _stream()), "rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gate_up [T, 2F] (gate columns first) -> silu(gate) * up, [T, F]."""
    _dev(gate_up, "gate_up")
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("gate_up must have an even number of columns")
    if out is None:
        out = torch.empty((T, F2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", "plm_swiglu")(_p(gate_up), _p(out), _dt(gate_up, "gate_up"), T, F2 // 2, _stream()),
           "swiglu")
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
    _check(_fn("elementwise", "plm_rope_store")(
        _p(qkv), _p(q_out), _p(k_cache) if store else None, _p(v_cache) if store else None, _dt(qkv, "qkv"),
        _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(block_table), block_table.shape[1], T, H, G, hd,
        rotary_dim, 0 if pairing == "half" else 1, 1 if store else 0, _stream()), "rope_store")


# ----------------------------------------------------------------------- GEMM
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
        _p(a), _dt(a, "a"), _p(w), _dt(w, "w"), _p(out), _dt(out, "out"), M, N, K, K, K, N, _stream()), "gemm_simt")
    return out


_status = {}


def status_word(device) -> torch.Tensor:
    """The device int that kernels with bounded waits write to when a wait runs
    out (0: all well).  One per device."""
    key = torch.device(device)
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=key)
        _status[key] = t
    return t


def check_status(device="cuda:0") -> None:
    """Raise if a kernel gave up a bounded wait since the last check (this
    synchronises with the device)."""
    t = _status.get(torch.device(device))
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        where = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue"}.get(code, str(code))
        raise KernelError(f"a tensor-core kernel gave up waiting on an mbarrier ({where}); its output is not valid")


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes a @ w^T: both bfloat16, K a multiple of
    8 (rows start on 16-byte boundaries, as TMA needs) and at least one K block."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    (M, K), (N, K2) = a.shape, w.shape
    if K != K2 or K < 64:
        return False
    return bool(_fn("gemm_tc", "plm_gemm_tc_supported")(_p(a), _p(w), M, N, K, K, K))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bf16 in, fp32
    accumulate).  With M <= 64 the weights take the 128-row side of the MMA and K
    is split; the fp32 partial sums pass through a scratch buffer."""
    _dev(a, "a"), _dev(w, "w")
    if not gemm_tc_supported(a, w):
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} {a.dtype} @ w {tuple(w.shape)} {w.dtype} is not supported "
                          f"(bfloat16, K a multiple of 8 and >= 64, 16-byte aligned)")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    splits, ws_elems = ctypes.c_int(0), ctypes.c_long(0)
    _fn("gemm_tc", "plm_gemm_tc_plan")(M, N, K, ctypes.byref(splits), ctypes.byref(ws_elems))
    ws = torch.empty((ws_elems.value,), dtype=torch.float32, device=a.device) if ws_elems.value else None
    _check(_fn("gemm_tc", "plm_gemm_tc")(
        _p(a), _p(w), _p(out), _dt(out, "out"), M, N, K, K, K, N, _p(ws), _p(status_word(a.device)), _stream()),
        "gemm_tc", kernels=2 if ws is not None else 1)
    return out


def gemm_tc_skinny(a, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decode-shaped tensor-core product: a [M <= 64, K] @ w [N, K]^T with the weights on the MMA's 128
    rows and K split over a thread-block cluster whose CTAs add their partial tiles up through distributed
    shared memory.  With `swiglu`, w holds tiles of 64 gate rows followed by their 64 up rows (see
    `interleave_gate_up`) and the result is silu(gate) * up, [M, N/2] in bfloat16.  `a` may be `ScaledRows`
    (an RMSNorm whose scale is still due): the epilogue then scales each row of the result, in bfloat16."""
    scaled = a if isinstance(a, ScaledRows) else None
    if scaled is not None:
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
            "gemm_tc_skinny_scaled")
        return out
    _check(_fn("gemm_tc_skinny", "plm_gemm_tc_skinny")(
        _p(a), _p(w), _p(out), _dt(out, "out"), 1 if swiglu else 0, M, N, K, K, K, n_out,
        _p(status_word(a.device)), _stream()), "gemm_tc_skinny")
    return out


class PendingLinear:
    """a [M, K] @ w [N, K]^T in float32 that has not run yet: the last product of a mixer or a
    feed-forward, whose result is a delta for the residual stream.  The norm that follows may run it
    with the residual add and its own weight in the epilogue (`linear_residual_norm`); anything else
    calls `compute()`."""
    __slots__ = ("a", "w")

    def __init__(self, a: torch.Tensor, w: torch.Tensor):
        self.a, self.w = a, w

    @property
    def shape(self):
        return (self.a.shape[0], self.w.shape[0])

    def compute(self) -> torch.Tensor:
        return linear(self.a, self.w, torch.float32)


class ScaledRows:
    """An RMSNorm whose scale is still due: `x` [T, size] in bfloat16 holds row * norm weight, and
    `parts` [n, >= T] partial sums of squares of the rows (column t for row t), so that the normalised
    row t is x[t] / sqrt(sum(parts[:, t]) / size + eps).  A product takes it as its left operand and
    applies the scale to its result (`linear`, `linear_swiglu`); `materialize()` gives the rows."""
    __slots__ = ("x", "parts", "size", "eps")

    def __init__(self, x: torch.Tensor, parts: torch.Tensor, size: int, eps: float):
        self.x, self.parts, self.size, self.eps = x, parts, size, eps

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
    """x += pending (in place, the fp32 residual stream) and the RMSNorm of the new x as `ScaledRows`:
    one tensor-core product whose epilogue does the add, applies the norm weight and leaves the rows'
    sums of squares; the scale itself is applied by the product that takes the result."""
    if not residual_norm_supported(pending, x, norm_weight):
        raise KernelError("linear_residual_norm: not a case the fused kernel takes")
    a, w = pending.a, pending.w
    _dev(a, "a"), _dev(w, "w"), _dev(x, "x"), _dev(norm_weight, "norm_weight")
    M, K = a.shape
    N = w.shape[0]
    xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    n_parts = _fn("gemm_tc_skinny", "plm_gemm_tc_skinny_residual_parts")(N, K)
    parts = torch.empty((n_parts, 64), dtype=torch.float32, device=x.device)
    _check(_fn("gemm_tc_skinny", "plm_gemm_tc_skinny_residual")(
        _p(a), _p(w), _p(x), _p(norm_weight), _p(xw), _p(parts), M, N, K, K, K, N, N,
        _p(status_word(x.device)), _stream()), "gemm_tc_skinny_residual")
    return ScaledRows(xw, parts, N, eps)


def gemm_tc_wide(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                 out: Optional[torch.Tensor] = None, pair: bool = False) -> torch.Tensor:
    """The prompt-shaped tensor-core product: a [M > 64, K] @ w [N, K]^T by a persistent tcgen05 kernel
    (one CTA per SM, two accumulators in tensor memory so that a tile's epilogue overlaps the next
    tile's main loop).  With `swiglu`, w comes from `interleave_gate_up` and the result is
    silu(gate) * up, [M, N/2] in bfloat16.  `pair`: the same by pairs of CTAs on tiles of 256 x 256
    (`tcgen05.mma.cta_group::2`: each CTA of a pair loads half of the weight tile)."""
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
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=a.device)
    _check(_fn("gemm_tc_wide", "plm_gemm_tc_pair" if pair else "plm_gemm_tc_wide")(
        _p(a), _p(w), _p(out), _dt(out, "out"), 1 if swiglu else 0, M, N, K, K, K, n_out,
        _p(status_word(a.device)), _stream()), "gemm_tc_pair" if pair else "gemm_tc_wide")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate | up] as one matrix whose rows come in tiles of 64 gate rows followed by the 64 up rows of
    the same features, so that a 128-row MMA tile holds both branches of 64 outputs and the product's
    epilogue can apply SwiGLU.  Needs a number of features that is a multiple of 64."""
    F, K = gate.shape
    if up.shape != gate.shape or F % 64:
        raise KernelError("interleave_gate_up: gate and up must have the same shape with a multiple of 64 rows")
    return torch.stack([gate.view(F // 64, 64, K), up.view(F // 64, 64, K)], dim=1).reshape(2 * F, K).contiguous()


def pair_pays(m: int, n: int) -> bool:
    """Whether the prompt-shaped product runs as pairs of CTAs on tiles of 256 x 256: measured 3..5 % faster
    than single CTAs on tiles of 128 x 256 where there are at least two rounds of tiles for the 74 pairs,
    and no faster or slower (a ragged last round of larger tiles) below that."""
    return m >= 256 and n >= 256 and ((m + 255) // 256) * ((n + 255) // 256) >= _SM_COUNT


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(a @ gate^T) * (a @ up^T) with `w_gate_up` from `interleave_gate_up`: one tensor-core product
    whose epilogue applies the activation; [M, F] in bfloat16.  `a` may be `ScaledRows`."""
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
    return gemm_tc_wide(a, w_gate_up, torch.bfloat16, swiglu=True, pair=pair_pays(M, N))


# ------------------------------------------------------------------ attention
def attention_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor,
                   tok_seq: torch.Tensor, block_table: torch.Tensor, num_kv_heads: int, scale: float,
                   window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of q [T, H, hd] over the paged cache; returns [T, H*hd]."""
    _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    T, H, hd = q.shape
    G = num_kv_heads
    if k_cache.dtype != q.dtype or k_cache.shape[1:] != (G, PAGE_TOKENS, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: the cache must be [pages, {G}, {PAGE_TOKENS}, {hd}] of {q.dtype}")
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} exceeds 256, the largest this kernel takes")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    _check(_fn("attention_simt", "plm_attention_rows")(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _dt(q, "q"), _p(tok_pos), _p(tok_seq), _p(block_table),
        block_table.shape[1], T, H, G, hd, float(scale), int(window or 0), _stream()), "attention_rows")
    return out


def attention_mma_supported(q: torch.Tensor) -> bool:
    """The tensor-core attention takes bfloat16 and head sizes that are multiples of 16 up to 256."""
    hd = q.shape[-1]
    return q.dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 256


def _attn_check(q, k_cache, v_cache, num_kv_heads):
    _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    T, H, hd = q.shape
    if not attention_mma_supported(q):
        raise KernelError(f"attention: {q.dtype} with head_dim {hd} is not supported by the tensor-core kernel "
                          f"(bfloat16, head_dim a multiple of 16 up to 256)")
    if k_cache.dtype != q.dtype or k_cache.shape[1:] != (num_kv_heads, PAGE_TOKENS, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: the cache must be [pages, {num_kv_heads}, {PAGE_TOKENS}, {hd}] of {q.dtype}")
    if H % num_kv_heads:
        raise KernelError("attention: the number of heads is not a multiple of the number of KV heads")
    return T, H, hd


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                      seq_kv_len: torch.Tensor, block_table: torch.Tensor, max_new: int, num_kv_heads: int,
                      scale: float, window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every sequence's new tokens (rows seq_start[b]..seq_start[b+1] of q [T, H, hd])
    over its keys 0..seq_kv_len[b]-1 in the paged cache; returns [T, H*hd]."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    _i32(seq_start, "seq_start"), _i32(seq_kv_len, "seq_kv_len"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    lib, flags = attention_variant(hd)
    _check(_fn(lib, "plm_attn_prefill", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(seq_start), _p(seq_kv_len), _p(block_table),
        block_table.shape[1], seq_kv_len.numel(), int(max_new), H, num_kv_heads, float(scale), int(window or 0),
        _stream()), "attention_prefill")
    return out


def attention_tc_supported(q: torch.Tensor) -> bool:
    """The tcgen05 prefill attention takes bfloat16 and head sizes 64 and 128."""
    return q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                         seq_kv_len: torch.Tensor, block_table: torch.Tensor, max_new: int, num_kv_heads: int,
                         scale: float, window: Optional[int] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`attention_prefill` on the tcgen05 tensor cores (scores and the page's output in tensor memory,
    operands by TMA): same arguments, same result up to rounding; head sizes 64 and 128."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    if not attention_tc_supported(q):
        raise KernelError(f"attention_prefill_tc: head_dim {hd} of {q.dtype} is not supported (bfloat16, 64 or 128)")
    _i32(seq_start, "seq_start"), _i32(seq_kv_len, "seq_kv_len"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    lib, flags = attention_variant(hd, "attention_tc")
    _check(_fn(lib, "plm_attn_tc_prefill", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(seq_start), _p(seq_kv_len), _p(block_table),
        block_table.shape[1], k_cache.shape[0], T, seq_kv_len.numel(), int(max_new), H, num_kv_heads, float(scale),
        int(window or 0), _p(status_word(q.device)), _stream()), "attention_prefill_tc")
    return out


_SM_COUNT = 148


DECODE_CLUSTER_SPLITS = 8       # up to this many ranges merge inside a thread-block cluster, without scratch


def decode_splits(n_tokens: int, num_heads: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Into how many ranges the decode kernel cuts each sequence's keys.  Where the whole grid runs at once
    (three CTAs an SM), as many ranges as that allows, up to the eight that merge inside a cluster, each of
    at least two pages.  Otherwise, and for long contexts (whose ranges would get too long for one wave
    of CTAs), about eight pages a range, more when that leaves SMs without a CTA (measured at batch 1, 8
    and 64 with 2,048 keys)."""
    row_groups = (num_heads // num_kv_heads + 15) // 16
    ctas = max(1, n_tokens * num_kv_heads * row_groups)
    pages = max(1, (max_kv_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
    in_cluster = min(DECODE_CLUSTER_SPLITS, (3 * _SM_COUNT) // ctas, max(1, pages // 2))
    if in_cluster >= 2 and pages <= (16 if ctas * in_cluster >= _SM_COUNT else 8) * in_cluster:
        return in_cluster
    splits = (pages + 7) // 8
    if ctas * splits < _SM_COUNT:
        splits = max(splits, min(max(1, pages // 2), (_SM_COUNT + ctas - 1) // ctas))
    return max(1, min(pages, splits))


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor,
                     tok_seq: torch.Tensor, block_table: torch.Tensor, num_kv_heads: int, scale: float,
                     n_splits: int, window: Optional[int] = None, out: Optional[torch.Tensor] = None,
                     scratch: Optional[bool] = None) -> torch.Tensor:
    """Attention of single query tokens (one per row of q [T, H, hd], at position tok_pos[t] of sequence
    tok_seq[t]) over the paged cache, the keys of each cut into `n_splits` ranges.  Up to eight ranges are the
    CTAs of a thread-block cluster and merge through its shared memory; more ranges, or more CTAs than
    run at once, pass their partial results through a scratch buffer and a second kernel (`scratch` forces
    one way or the other).  Returns [T, H*hd]."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    # Clusters are scheduled as a whole: past one wave of CTAs that costs more than the second kernel saves.
    ctas = T * num_kv_heads * ((H // num_kv_heads + 15) // 16) * n_splits
    if scratch is None:
        scratch = ctas > 3 * _SM_COUNT
    scratch = n_splits > 1 and (scratch or n_splits > DECODE_CLUSTER_SPLITS)
    ws = torch.empty((T * H * n_splits * (hd + 2),), dtype=torch.float32, device=q.device) if scratch else None
    lib, flags = attention_variant(hd)
    _check(_fn(lib, "plm_attn_decode", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(ws), _p(tok_pos), _p(tok_seq), _p(block_table),
        block_table.shape[1], T, H, num_kv_heads, float(scale), int(window or 0), int(n_splits), _stream()),
        "attention_decode", kernels=2 if scratch else 1)
    return out


class Rotation:
    """A rotary encoding as the kernels take it: cos / sin tables [positions, rotary_dim / 2] in float32,
    how many leading components of a head are rotated, and how they pair up ("half" or "adjacent")."""
    __slots__ = ("cos", "sin", "rotary_dim", "pairing")

    def __init__(self, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int, pairing: str):
        self.cos, self.sin, self.rotary_dim, self.pairing = cos, sin, rotary_dim, pairing


def attention_decode_rope_supported(qkv: torch.Tensor, kv, rotation: Optional[Rotation], head_dim: int) -> bool:
    """Whether the decode kernel can do this rotation and the cache write itself: bfloat16, a head size it
    takes, the whole head rotated in half-split pairs, a cache that this layer writes."""
    return (rotation is not None and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and rotation.rotary_dim == head_dim and rotation.pairing == "half" and kv.writable
            and kv.k.dtype == torch.bfloat16 and rotation.cos is not None)


def attention_decode_rope(qkv: torch.Tensor, kv, step, num_heads: int, num_kv_heads: int, head_dim: int,
                          scale: float, rotation: Rotation, scratch: Optional[bool] = None) -> torch.Tensor:
    """A decode step's attention with the rotary encoding and the cache write folded in: `qkv`
    [T, (H + 2G) * hd] is the output of the QKV projection; queries and the new keys are rotated inside
    the kernel, the new keys and values are written to the cache at the tokens' positions, and the
    queries attend to everything up to and including them.  Returns [T, H * hd]."""
    _dev(qkv, "qkv"), _dev(kv.k, "k_cache"), _dev(kv.v, "v_cache")
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if not attention_decode_rope_supported(qkv, kv, rotation, hd):
        raise KernelError("attention_decode_rope: not a case the fused kernel takes")
    if qkv.shape[1] != (H + 2 * G) * hd or kv.k.shape[1:] != (G, PAGE_TOKENS, hd) or kv.v.shape != kv.k.shape:
        raise KernelError("attention_decode_rope: qkv or the cache does not have the shape the heads imply")
    if step.max_position >= rotation.cos.shape[0]:
        raise KernelError(f"position {step.max_position} lies beyond the rotary table")
    n_splits = decode_splits(T, H, G, step.max_position + 1)
    ctas = T * G * ((H // G + 15) // 16) * n_splits
    if scratch is None:
        scratch = ctas > 3 * _SM_COUNT
    scratch = n_splits > 1 and (scratch or n_splits > DECODE_CLUSTER_SPLITS)
    out = torch.empty((T, H * hd), dtype=qkv.dtype, device=qkv.device)
    ws = torch.empty((T * H * n_splits * (hd + 2),), dtype=torch.float32, device=qkv.device) if scratch else None
    lib, flags = attention_variant(hd)
    _check(_fn(lib, "plm_attn_decode_rope", flags)(
        _p(qkv), _p(kv.k), _p(kv.v), _p(out), _p(ws), _p(rotation.cos), _p(rotation.sin), _p(step.tok_pos),
        _p(step.tok_seq), _p(kv.block_table), kv.block_table.shape[1], T, H, G, float(scale), int(kv.window or 0),
        int(n_splits), _stream()), "attention_decode_rope", kernels=2 if scratch else 1)
    return out


# ------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum, int32 [rows]."""
    _dev(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("logits must be float32")
    n, V = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
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
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "plm_sample")(
        _p(logits), V, n, V, float(temperature), int(top_k), float(top_p), float(min_p), _p(rng_state), _p(out),
        _stream()), "sample")
    return out


# ---------------------------------------------------------------- dispatchers
def linear(a, w: torch.Tensor, out_dtype: torch.dtype, defer: bool = False):
    """a [M, K] times w [N, K]^T -> [M, N].  The kernel is chosen by element
    types and shape, never by the model: the tensor cores for bfloat16 operands
    that TMA can address (the cluster kernel for up to 64 rows, the wide kernel
    beyond), the CUDA cores for everything else.

    `a` may be `ScaledRows`.  With `defer` (a float32 delta for the residual stream) the product may
    come back as a `PendingLinear` for the next norm to run; whoever cannot use that calls `compute()`."""
    if isinstance(a, ScaledRows):
        if a.shape[0] <= 64 and out_dtype == torch.bfloat16 and gemm_tc_supported(a.x, w):
            return gemm_tc_skinny(a, w, out_dtype)
        a = a.materialize()
    if defer and out_dtype == torch.float32 and a.shape[0] <= 64 and gemm_tc_supported(a, w):
        return PendingLinear(a, w)
    if gemm_tc_supported(a, w):
        if a.shape[0] <= 64:
            return gemm_tc_skinny(a, w, out_dtype)
        return gemm_tc_wide(a, w, out_dtype, pair=pair_pays(a.shape[0], w.shape[0]))
    return gemm_simt(a, w, out_dtype)


def attention(q: torch.Tensor, kv, step, num_kv_heads: int, scale: float) -> torch.Tensor:
    """Causal attention of the step's queries over their sequences' cached keys
    and values (`kv` is a `KVLayerCache`)."""
    if attention_mma_supported(q):
        if step.is_decode:
            splits = decode_splits(q.shape[0], q.shape[1], num_kv_heads, step.max_position + 1)
            return attention_decode(q, kv.k, kv.v, step.tok_pos, step.tok_seq, kv.block_table, num_kv_heads, scale,
                                    splits, window=kv.window)
        prefill = attention_prefill_tc if attention_tc_supported(q) else attention_prefill
        return prefill(q, kv.k, kv.v, step.seq_start, step.seq_kv_len, kv.block_table, max(step.new_lens),
                       num_kv_heads, scale, window=kv.window)
    return attention_rows(q, kv.k, kv.v, step.tok_pos, step.tok_seq, kv.block_table, num_kv_heads, scale,
                          window=kv.window)
