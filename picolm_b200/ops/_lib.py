"""The plumbing under the kernels' Python faces: the C signatures, loading a library's entry point,
error codes, the launch counter, argument helpers and the device status word of the bounded waits."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library

PAGE_TOKENS = 64            # tokens per cache page; PLM_PAGE in csrc/common.cuh

_DT = {torch.float32: 0, torch.bfloat16: 1}

_vp, _i, _l, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float

_SIGNATURES = {
    "plm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "plm_rmsnorm": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _f, _vp],
    "plm_swiglu": [_vp, _vp, _i, _i, _i, _i, _vp],
    "plm_rope_store": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "plm_gemm_tc_skinny": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_skinny_residual": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _l, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_skinny_residual_parts": [_i, _i],
    "plm_gemm_tc_skinny_scaled": [_vp, _vp, _vp, _i, _i, _i, _i, _l, _l, _l, _vp, _i, _i, _i, _f, _vp, _vp],
    "plm_scale_rows": [_vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp],
    "plm_gather_rows": [_vp, _vp, _vp, _i, _l, _l, _vp],
    "plm_gemm_tc_wide": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_tc_wide_space": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp, _vp, _i, _vp, _vp],
    "plm_gemm_tc_pair_space": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp, _i, _vp, _vp],
    "plm_gemm_tc_pair_streamed": [_i, _i, _i, _i],
    "plm_gemm_tc_wide_slot_floats": [],
    "plm_gemm_tc_wide_pieces": [_i, _i, _i, _i, _vp, _i],
    "plm_gemm_tc_wide_how": [_i, _i, _i, _i, _i, _vp],
    "plm_gemm_tc_wide_splits": [_i, _i, _i],
    "plm_gemm_tc_pair": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _l, _l, _l, _vp, _vp],
    "plm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _l, _l, _l, _vp],
    "plm_attention_rows": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
    "plm_attn_prefill": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
    "plm_attn_tc_prefill": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp],
    "plm_attn_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp],
    "plm_attn_decode_rope": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp],
    "plm_check_bounds": [_i, _i, _i, _i, _vp, _vp],
    "plm_decode_chain": [_vp, _i, _i, _vp, _vp, _vp, _vp],
    "plm_decode_chain_ctas": [],
    "plm_decode_chain_scratch": [_i, _i, _i],
    "plm_argmax": [_vp, _l, _i, _i, _vp, _vp],
    "plm_sample": [_vp, _l, _i, _i, _f, _i, _f, _f, _vp, _vp, _vp],
}
_fn_cache = {}

# The checked build of the kernels that follow host-computed indices (csrc/common.cuh, PLM_CHECK): with
# PICOLM_B200_CHECK=1 in the environment these libraries are compiled with -DPLM_CHECK, and the faces in
# this package hand them the bounds before every launch.  An index outside its bound is then recorded in
# the status word (`check_status` raises) instead of being followed.
CHECKED = os.environ.get("PICOLM_B200_CHECK", "") == "1"
CHECKED_LIBRARIES = ("elementwise", "attention_simt", "attention_mma", "attention_tc")


class KernelError(RuntimeError):
    pass


_CODES = {-1: "unsupported element type", -2: "bad shape", -3: "bad alignment", -4: "unsupported option",
          -5: "the device wait ran out (see the status word)"}


# library -> (variant name, compile flags): a measuring build that stands in for a library in this process
# (`bench_kernels --stations` puts the prompt-shaped product's trace build here)
VARIANT_OF = {}


def _fn(library: str, name: str, extra_flags=()):
    if library in VARIANT_OF:
        library, more = VARIANT_OF[library]
        extra_flags = tuple(extra_flags) + tuple(more)
    if CHECKED and library.split("@")[0] in CHECKED_LIBRARIES:
        library = library + ("_check" if "@" in library else "@check")
        extra_flags = tuple(extra_flags) + ("-DPLM_CHECK",)
    key = (library, name, tuple(extra_flags))
    f = _fn_cache.get(key)
    if f is None:
        lib = load_library(library, extra_flags)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        if TRACED:
            f = _traced(f)
        _fn_cache[key] = f
    return f


# ------------------------------------------------------------------ the per-kernel table
# With PICOLM_B200_TRACE=1 every entry point is called between two CUDA events, and when the process ends (or
# `trace_report()` is called) a table goes to stderr: per kind of launch its count, its device time, the bytes
# and flops its face in this package declared for it, and what fraction of the memory's or the tensor cores'
# rate that is.  Steps are launched kernel by kernel while tracing (no graphs).  The reference's counterpart is
# the per-layer table of its --benchmark (picolm/picolm.c:251-383); this one is per kernel.
TRACED = os.environ.get("PICOLM_B200_TRACE", "") == "1"
PEAK_GBS = float(os.environ.get("PICOLM_B200_PEAK_GBS", "6535.7"))        # a B200's copy bandwidth as measured
PEAK_TFLOPS = float(os.environ.get("PICOLM_B200_PEAK_TFLOPS", "1636.8"))  # and its cuBLAS bf16 rate
_trace_open = []          # (start, stop) of launches whose `_check` has not run yet
_trace_rows = []          # (what, start, stop, bytes, flops)


def _traced(f):
    def call(*args):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # Keep the device busy for some tens of microseconds first, so that the first event, the launch and the
        # second event are all queued before the device reaches them: the time between the events is then the
        # kernel's, not the host's time to enqueue it on an idle device.
        torch.cuda._sleep(120000)
        a.record()
        code = f(*args)
        b.record()
        _trace_open.append((a, b))
        return code
    return call


def trace_report(file=None, reset: bool = True):
    """The per-kernel table of what ran since the last report (needs PICOLM_B200_TRACE=1).  Returns the rows."""
    import sys
    torch.cuda.synchronize()
    agg = {}
    for what, a, b, nbytes, flops in _trace_rows:
        r = agg.setdefault(what, [0, 0.0, 0, 0])
        r[0] += 1
        r[1] += a.elapsed_time(b)
        r[2] += nbytes
        r[3] += flops
    rows = sorted(agg.items(), key=lambda kv: -kv[1][1])
    total = sum(r[1] for _, r in rows) or 1.0
    out = file or sys.stderr
    print(f"{'launch':44s} {'count':>6s} {'ms':>9s} {'share':>6s} {'GB/s':>8s} {'of peak':>7s} {'TFLOP/s':>8s} {'of peak':>7s}", file=out)
    for what, (n, ms, nbytes, flops) in rows:
        gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        tf = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        print(f"{what[:44]:44s} {n:6d} {ms:9.3f} {ms / total:6.1%} {gbs:8.0f} {gbs / PEAK_GBS:7.2f} {tf:8.1f} {tf / PEAK_TFLOPS:7.2f}",
              file=out)
    if reset:
        _trace_rows.clear()
    return rows


if TRACED:
    import atexit

    @atexit.register
    def _report_at_exit():
        if _trace_rows:
            try:
                trace_report()
            except Exception:
                pass


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (one per successful call of
    an entry point that launches one kernel)."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels that ran (or did not run) outside `_check`: the replays of a CUDA graph."""
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1, nbytes: int = 0, flops: int = 0) -> None:
    """After an entry point returned `code`: count its launches, or raise.  `nbytes` and `flops` are what the
    launch has to move and compute (for the per-kernel table)."""
    global _launches
    if TRACED and _trace_open:
        a, b = _trace_open.pop()
        _trace_open.clear()
        if code == 0:
            _trace_rows.append((what, a, b, int(nbytes), int(flops)))
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


_bound_stream = None


def _stream():
    if _bound_stream is not None:
        return _bound_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Within this scope every kernel goes to the stream that is current at its entry: asking torch for the
    current stream costs a few microseconds, and a step launches a hundred kernels.  Whoever changes the
    current stream inside (a CUDA graph capture does) opens a scope of its own there."""

    def __enter__(self):
        global _bound_stream
        self.outer = _bound_stream
        _bound_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self.outer
        return False


def _dt(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name} has dtype {t.dtype}; float32 and bfloat16 are supported")
    return _DT[t.dtype]


def _i32(t: torch.Tensor, name: str) -> None:
    _dev(t, name)
    if t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


SM_COUNT = 148              # SMs of a B200: what grids are sized for; PLM_SM_COUNT in csrc/common.cuh

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


_stream_space = {}
STREAM_WALK = os.environ.get("PICOLM_B200_STREAM_WALK", "1") != "0"   # 0: the prompt-shaped product hands out whole tiles only


def stream_space_enabled() -> bool:
    return STREAM_WALK


def stream_space(device):
    """(parts, flags, slots): the workspace with which the prompt-shaped product hands the K blocks of all
    tiles out as one stream, a slot and a flag per CTA.  One per device, for launches of one stream at a
    time; the kernels leave the flags zero."""
    if not STREAM_WALK:
        return None, None, 0
    key = torch.device(device)
    t = _stream_space.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the product's workspace must exist before a graph is captured: run the step once first")
        slot = _fn("gemm_tc_wide", "plm_gemm_tc_wide_slot_floats")()
        t = (torch.empty(SM_COUNT * slot, dtype=torch.float32, device=key),
             torch.zeros(SM_COUNT, dtype=torch.int32, device=key), SM_COUNT)
        _stream_space[key] = t
    return t


def set_bounds(library: str, extra_flags=(), *, n_pages: int = 0, n_seqs: int = 0, n_positions: int = 0,
               n_rows: int = 0, device=None) -> None:
    """In the checked build: tell `library` the bounds of the indices that its next launches follow (pages
    of the cache, sequences of the step, positions a sequence may have, rows that may be gathered; 0: not
    checked).  Nothing happens in the serving build."""
    if not CHECKED or library.split("@")[0] not in CHECKED_LIBRARIES:
        return
    code = _fn(library, "plm_check_bounds", extra_flags)(
        int(n_pages), int(n_seqs), int(n_positions), int(n_rows), _p(status_word(device or "cuda:0")), _stream())
    if code:
        raise KernelError(f"plm_check_bounds: CUDA error {code}")


def check_status(device="cuda:0") -> None:
    """Raise if a kernel gave up a bounded wait since the last check (this
    synchronises with the device)."""
    t = _status.get(torch.device(device))
    if t is None:
        return
    code = int(t.item())
    if code:
        t.zero_()
        if code >= 16:
            what = {16: "page number", 17: "sequence index", 18: "position", 19: "row index"}.get(code, str(code))
            raise KernelError(f"a kernel of the checked build met a {what} outside its bounds and did not follow it; "
                              f"its output is not valid")
        where = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "the CTAs' meeting"}.get(code, str(code))
        raise KernelError(f"a tensor-core kernel gave up waiting on an mbarrier ({where}); its output is not valid")

