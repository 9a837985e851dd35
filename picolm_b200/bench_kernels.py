"""Times one kernel at given sizes with CUDA events and prints what it achieved
against the bytes it has to move or the flops it has to do.

    python -m picolm_b200.bench_kernels gemm --m 8 --n 16384 --k 2048
    python -m picolm_b200.bench_kernels attention_decode --batch 8 --ctx 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m picolm_b200.bench_kernels attention_prefill --tokens 2048 --heads 32 --kv-heads 8 --head-dim 64
    python -m picolm_b200.bench_kernels sample --batch 8 --vocab 128256 --temperature 0.8 --top-k 40 --top-p 0.9
    python -m picolm_b200.bench_kernels gemm --m 8 --n 2048 --k 8192 --residual      (the product with the norm's half)
    python -m picolm_b200.bench_kernels gemm --m 2048 --n 2048 --k 8192 --residual   (the product added to the stream)

Operands rotate through copies that together exceed the L2 cache, so every
timed launch reads its weights or its cache from HBM.  `--iters` launches are
timed after `--warmup` untimed ones; `--once` runs a single launch (for a
profiler).
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

L2_BYTES = 126 * 1024 * 1024


USE_GRAPH = False


def _time(fn, n_variants, iters, warmup):
    """Seconds per launch.  With USE_GRAPH the `iters` launches are captured into one CUDA graph and
    the graph's replay is timed: launch overhead from Python (some 20 us a call) then does not hide
    kernels that are shorter than it."""
    for i in range(warmup):
        fn(i % n_variants)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if USE_GRAPH:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i % n_variants)
        g.replay()
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e-3
    a.record()
    for i in range(iters):
        fn(i % n_variants)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def bench_gemm(args):
    from . import ops
    M, N, K = args.m, args.n, args.k
    w_bytes = N * K * 2
    copies = args.copies or min(24, max(2, math.ceil(2 * L2_BYTES / w_bytes)))
    ws = [torch.randn(N, K, device="cuda").to(torch.bfloat16) * 0.02 for _ in range(copies)]
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    out_dtype = torch.float32 if args.out == "float32" else torch.bfloat16

    if args.residual:                                        # EPI_RESIDUAL: stream += product, norm weight, sums of squares
        x = torch.randn(M, N, device="cuda")
        nw = torch.ones(N, device="cuda", dtype=torch.bfloat16)

    def run(i):
        if args.library:                                     # the library's product of the same operands (bf16 out)
            y = torch.matmul(a, ws[i].t())
            if args.swiglu:                                  # rows in this kernel's order: tiles of 64 gate, 64 up rows
                y = y.view(M, N // 128, 2, 64)
                torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]
        elif args.residual and M > 64:                      # the add to the stream in the prompt-shaped product's epilogue
            ops.PendingLinear(a, ws[i]).add_into(x)
        elif args.residual:
            ops.linear_residual_norm(ops.PendingLinear(a, ws[i]), x, nw, 1e-5)
        elif args.pair:
            ops.gemm_tc_wide(a, ws[i], out_dtype, swiglu=args.swiglu, pair=True)
        elif args.swiglu:
            ops.linear_swiglu(a, ws[i])
        else:
            ops.linear(a, ws[i], out_dtype)

    sec = _time(run, len(ws), 1 if args.once else args.iters, 0 if args.once else args.warmup)
    ops.check_status()
    if args.stations:
        _print_stations()
    bytes_moved = w_bytes + M * K * 2 + M * N * (4 if out_dtype == torch.float32 else 2)
    flops = 2.0 * M * N * K
    return {"kernel": "torch.matmul (library)" if args.library else "linear (tensor cores)", "m": M, "n": N, "k": K,
            "us": round(sec * 1e6, 2),
            "GB/s": round(bytes_moved / sec / 1e9, 1), "TFLOP/s": round(flops / sec / 1e12, 2), "weight_copies": len(ws)}


def _print_stations():
    """The last launch of the prompt-shaped product's trace build (`-DPLM_WIDE_TRACE`): when its CTAs passed
    their stations (microseconds after the first CTA's entry) and, for CTAs with one piece of work, how many
    cycles the loading thread waited for a free stage and the MMA thread for loads to land."""
    import ctypes

    import numpy as np

    from .csrc.build import load_library
    from .ops import _lib
    name, flags = _lib.VARIANT_OF["gemm_tc_wide"]
    lib = load_library(name, flags)
    buf = (ctypes.c_ulonglong * (16 * _lib.SM_COUNT))()
    lib.plm_gemm_tc_wide_trace_read.argtypes = [ctypes.c_void_p]
    if lib.plm_gemm_tc_wide_trace_read(buf):
        raise RuntimeError("the trace could not be read")
    t = np.frombuffer(buf, dtype=np.uint64).reshape(_lib.SM_COUNT, 16).astype(np.int64)
    used = t[:, 0] > 0
    t0 = t[used, 0].min()
    for i, what in ((0, "entry"), (1, "activations may be read"), (2, "all loads issued"), (3, "all MMAs issued"),
                    (5, "first piece: accumulator ready"), (13, "first piece: 32 columns in registers"),
                    (14, "first piece: 32 columns written"), (6, "first piece: written")):
        ok = used & (t[:, i] >= t0)
        if ok.any():
            c = (t[ok, i] - t0) / 1e3
            print(f"{what:40s} CTAs {int(ok.sum()):3d}  min {c.min():7.2f}  median {np.median(c):7.2f}  max {c.max():7.2f} us",
                  file=sys.stderr)
    ok = used & (t[:, 10] > 0)
    if ok.any():
        print(f"loading thread: {np.median(t[ok, 7]):.0f} of {np.median(t[ok, 8]):.0f} cycles waiting for a free stage; "
              f"MMA thread: {np.median(t[ok, 9]):.0f} of {np.median(t[ok, 10]):.0f} cycles waiting for loads "
              f"(medians over {int(ok.sum())} CTAs)", file=sys.stderr)


def _print_attention_stations(hd):
    """The last launch of the prefill attention's trace build (`-DPLM_ATTN_TRACE`): how many cycles the first
    softmax warp and the issuing thread of the CTA that starts first spent between their stations, page by
    page (means over pages 8 to 120, where the pipeline is in its steady state)."""
    import ctypes

    import numpy as np

    from .csrc.build import load_library
    from .ops import _lib
    name, flags = _lib.VARIANT_OF[f"attention_tc@hd{hd}"]
    lib = load_library(name, (f"-DPLM_HD={hd}",) + tuple(flags))
    buf = (ctypes.c_longlong * (5 * 128 * 8))()
    lib.plm_attn_tc_trace_read.argtypes = [ctypes.c_void_p]
    if lib.plm_attn_tc_trace_read(buf):
        raise RuntimeError("the trace could not be read")
    t = np.frombuffer(buf, dtype=np.int64).reshape(5, 128, 8)
    mma = t[4]
    lo, hi = 8, 120
    if mma[hi, 2] == 0:
        print("the first CTA had fewer than 121 pages: no steady state to show", file=sys.stderr)
        return

    def mean(x):
        return float(np.mean(x[lo:hi]))

    for w in range(4):
        sm = t[w]
        print(f"softmax warp {w}, cycles a page: period {mean(sm[1:, 0] - sm[:-1, 0]):.0f} = "
              f"scores to registers {mean(sm[:, 1] - sm[:, 0]):.0f} + maximum and P's place {mean(sm[:, 2] - sm[:, 1]):.0f} + "
              f"exponentials {mean(sm[:, 3] - sm[:, 2]):.0f} + P to tensor memory {mean(sm[:, 4] - sm[:, 3]):.0f} + "
              f"arrive {mean(sm[:, 5] - sm[:, 4]):.0f} + wait for the next scores {mean(sm[1:, 0] - sm[:-1, 5]):.0f}; "
              f"its arrival to the issuing thread seeing everybody's {mean(mma[:, 0] - sm[:, 5]):.0f}", file=sys.stderr)
    print(f"issuing thread, cycles a page: period {mean(mma[1:, 0] - mma[:-1, 0]):.0f} = "
          f"first group of MMAs {mean(mma[:, 1] - mma[:, 0]):.0f} + second group and commits {mean(mma[:, 2] - mma[:, 1]):.0f} + "
          f"wait for the next page's arrivals {mean(mma[1:, 0] - mma[:-1, 2]):.0f}; from everybody's arrival to the "
          f"scores of the page after next seen by warp 0 {mean(t[0][2:, 0] - mma[:-2, 0]):.0f}", file=sys.stderr)


def _paged_cache(batch, ctx, G, hd, n_copies):
    pages_per_seq = (ctx + 63) // 64
    n_pages = batch * pages_per_seq + 1
    caches = []
    for _ in range(n_copies):
        caches.append((torch.randn(n_pages, G, 64, hd, device="cuda").to(torch.bfloat16),
                       torch.randn(n_pages, G, 64, hd, device="cuda").to(torch.bfloat16)))
    table = (torch.arange(batch * pages_per_seq, dtype=torch.int32, device="cuda") + 1).view(batch, pages_per_seq)
    return caches, table.contiguous()


def bench_attention_decode(args):
    from . import ops
    B, C, H, G, hd = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim
    kv_bytes = B * C * G * hd * 2 * 2
    caches, table = _paged_cache(B, C, G, hd, min(16, max(2, math.ceil(2 * L2_BYTES / kv_bytes))))
    q = torch.randn(B, H, hd, device="cuda").to(torch.bfloat16)
    pos = torch.full((B,), C - 1, dtype=torch.int32, device="cuda")
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    splits = args.splits or ops.decode_splits(B, H, G, C, hd)

    def run(i):
        ops.attention_decode(q, caches[i][0], caches[i][1], pos, seq, table, G, 1.0 / math.sqrt(hd), splits,
                             scratch={"auto": None, "cluster": False, "scratch": True}[args.merge])

    sec = _time(run, len(caches), 1 if args.once else args.iters, 0 if args.once else args.warmup)
    return {"kernel": "attention_decode", "batch": B, "ctx": C, "heads": H, "kv_heads": G, "head_dim": hd,
            "splits": splits, "us": round(sec * 1e6, 2), "GB/s": round(kv_bytes / sec / 1e9, 1)}


def bench_attention_prefill(args):
    from . import ops
    T, H, G, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
    caches, table = _paged_cache(1, T, G, hd, 2)
    q = torch.randn(T, H, hd, device="cuda").to(torch.bfloat16)
    start = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    kvlen = torch.tensor([T], dtype=torch.int32, device="cuda")

    fn = ops.attention_prefill_tc if (ops.attention_tc_supported(q) and not args.mma) else ops.attention_prefill
    if args.library:                                         # the library's causal attention on contiguous keys and values
        ql = q.transpose(0, 1).unsqueeze(0).contiguous()
        kl = [torch.randn(1, G, T, hd, device="cuda").to(torch.bfloat16) for _ in caches]
        vl = [torch.randn(1, G, T, hd, device="cuda").to(torch.bfloat16) for _ in caches]

    def run(i):
        if args.library:
            torch.nn.functional.scaled_dot_product_attention(ql, kl[i], vl[i], is_causal=True, enable_gqa=True)
        else:
            fn(q, caches[i][0], caches[i][1], start, kvlen, table, T, G, 1.0 / math.sqrt(hd))

    sec = _time(run, len(caches), 1 if args.once else args.iters, 0 if args.once else args.warmup)
    if args.stations and fn is ops.attention_prefill_tc and not args.library:
        _print_attention_stations(hd)
    flops = 2.0 * 2 * H * hd * T * (T + 1) / 2
    return {"kernel": "scaled_dot_product_attention (library)" if args.library else "attention_prefill", "tokens": T, "heads": H, "kv_heads": G, "head_dim": hd,
            "us": round(sec * 1e6, 2), "TFLOP/s": round(flops / sec / 1e12, 2)}


def bench_sample(args):
    from . import ops
    B, V = args.batch, args.vocab
    copies = max(2, math.ceil(2 * L2_BYTES / (B * V * 4)))
    copies = min(copies, 64)
    logits = [torch.randn(B, V, device="cuda") * 3 for _ in range(copies)]
    rng = torch.arange(1, B + 1, dtype=torch.int64, device="cuda") * 7919

    def run(i):
        if args.temperature <= 0:
            ops.argmax(logits[i])
        else:
            ops.sample(logits[i], rng, args.temperature, args.top_k, args.top_p, args.min_p)

    sec = _time(run, len(logits), 1 if args.once else args.iters, 0 if args.once else args.warmup)
    return {"kernel": "argmax" if args.temperature <= 0 else "sample", "batch": B, "vocab": V,
            "temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p, "min_p": args.min_p,
            "us": round(sec * 1e6, 2), "GB/s": round(B * V * 4 / sec / 1e9, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m picolm_b200.bench_kernels", description=__doc__.split("\n\n")[0])
    ap.add_argument("kernel", choices=["gemm", "attention_decode", "attention_prefill", "sample"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--out", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--merge", default="auto", choices=["auto", "cluster", "scratch"],
                    help="attention_decode: merge the key ranges inside a cluster or through scratch memory")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--swiglu", action="store_true", help="gemm: the product with the SwiGLU epilogue (n counts gate and up rows)")
    ap.add_argument("--pair", action="store_true", help="gemm (m > 64): the kernel of CTA pairs (tcgen05.mma.cta_group::2)")
    ap.add_argument("--residual", action="store_true",
                    help="gemm: the product in front of an RMSNorm; m <= 64: adds to the stream, norm weight, sums of squares; "
                         "m > 64: adds to the stream")
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--temperature", type=float, default=0.8, help="sample: 0 times the argmax kernel")
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--min-p", type=float, default=0.05)
    ap.add_argument("--mma", action="store_true", help="attention_prefill: the mma.sync kernel, not the tcgen05 one")
    ap.add_argument("--library", action="store_true",
                    help="gemm, attention_prefill: time the library's routine on the same sizes instead (a yardstick; "
                         "no model step uses it)")
    ap.add_argument("--copies", type=int, default=0,
                    help="gemm: weight copies to rotate through (default: enough to exceed L2; 1 keeps them in L2)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--once", action="store_true", help="one launch, no warm-up (for a profiler)")
    ap.add_argument("--graph", action="store_true", help="time the launches as one CUDA graph (for short kernels)")
    ap.add_argument("--stations", action="store_true",
                    help="gemm (m > 64), attention_prefill: run the kernel's trace build and print when its CTAs "
                         "(the attention: the threads of its first CTA) passed their stations in the last launch (stderr)")
    args = ap.parse_args(argv)
    if args.stations:
        from .ops import _lib
        _lib.VARIANT_OF["gemm_tc_wide"] = ("gemm_tc_wide@trace", ("-DPLM_WIDE_TRACE",))
        _lib.VARIANT_OF[f"attention_tc@hd{args.head_dim}"] = (f"attention_tc@hd{args.head_dim}_trace", ("-DPLM_ATTN_TRACE",))
    global USE_GRAPH
    USE_GRAPH = args.graph and not args.once
    fn = {"gemm": bench_gemm, "attention_decode": bench_attention_decode,
          "attention_prefill": bench_attention_prefill, "sample": bench_sample}[args.kernel]
    print(json.dumps(fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
