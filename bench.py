#!/usr/bin/env python3
"""Benchmark of picolm_b200 on one B200: decode tokens/s (the headline, batch 8)
with its HBM roofline, prefill of 2,048 tokens with its tensor-core fraction,
decode at batch 1 and 64, and the same decode measured end to end through the
Python entry point (host token ids in, host token ids out).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The model has the layer sizes
of BASELINE.json's configs[2] (Llama-3.2-1B shape) with random weights; every
timed step reads all weights (2.5 GB, far more than the 126 MB L2), so no L2
flush is needed between steps.  Prints one JSON line.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}     # an earlier measurement on this pool


def baseline_text(index=2):
    """The text of BASELINE.json's configs[index] ("" if it cannot be read)."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            return json.load(f)["configs"][index]
    except (OSError, KeyError, IndexError, ValueError):
        return ""


def bench_config(index=2):
    """The sizes of BASELINE.json's configs[index] (2, the Llama-3.2-1B shape, unless asked otherwise),
    read from its text."""
    text = baseline_text(index)

    def num(pattern, default):
        m = re.search(pattern, text)
        return int(m.group(1).replace(",", "")) if m else default

    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": num(r"(\d+) layers", 16), "hidden_size": num(r"hidden (\d+)", 2048),
        "num_attention_heads": num(r"(\d+) heads", 32), "num_key_value_heads": num(r"(\d+) KV heads", 8),
        "head_dim": num(r"head_dim (\d+)", 64), "intermediate_size": num(r"intermediate (\d+)", 8192),
        "vocab_size": num(r"vocab (\d+)", 128256), "rope_theta": float(num(r"rope_theta (\d+)", 500000)),
        "rope_scaling": {"rope_type": "llama3", "factor": float(num(r"factor (\d+)", 32)),
                         "low_freq_factor": float(num(r"low_freq (\d+)", 1)),
                         "high_freq_factor": float(num(r"high_freq (\d+)", 4)),
                         "original_max_position_embeddings": num(r"original (\d+)", 8192)},
        "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": "untied" not in text,
        "hidden_act": "silu", "bos_token_id": 128000, "eos_token_id": 128001,
    }
    m = re.search(r"rms_norm_eps ([0-9.e-]+)", text)
    if m:
        cfg["rms_norm_eps"] = float(m.group(1).rstrip("."))
    if "no rope scaling" in text:
        cfg["rope_scaling"] = None
    name = text.split(",")[0].strip() or "Llama-3.2-1B shape"
    prompt = num(r"prefill at ([\d,]+) tokens", 0) or num(r"([\d,]+)-token random-id prompts", 2048)
    return cfg, num(r"context (\d+)", 4096), prompt, num(r"seed (\d+)", 2), name


def peaks():
    p = dict(FALLBACK_PEAKS)
    src = "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if k in m:
                p[k] = float(m[k])
        src = "measured"
    except (OSError, ValueError):
        pass
    return p, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].startswith("Active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def reference_arm(args):
    """whoreson/picolm itself on this GPU: its stock CUDA command line, built by its own Makefile into
    baseline/_ref, on a GGUF file with random bfloat16 weights of the benchmark's shape (baseline/reference_arm.py).
    The reference serves one sequence at a time, so its decode rate is a batch-1 rate; `--steps` is the number of
    tokens it generates in the timed run, `--warmup` counts short runs before it."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as R
    cfg_dict, context, prompt_len, seed, model_name = bench_config(args.config)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    prefill_tokens = min(2048, context)
    new_tokens = max(args.steps, 16)
    try:
        binary = R.build()
        with tempfile.TemporaryDirectory() as tmp:
            gguf = os.path.join(tmp, "model.gguf")
            t0 = time.time()
            size = R.write_gguf(gguf, dict(cfg_dict, context=context), seed)
            print(f"[bench] wrote {size / 1e9:.2f} GB of GGUF in {time.time() - t0:.0f} s", file=sys.stderr)
            gpu = True
            try:
                small = R.run(binary, gguf, 16, 8, context, gpu=True, timeout=900)       # a small run first
                if small["backend"] != "cuda":
                    raise R.Unavailable("the reference's GPU backend did not initialise: " + "; ".join(small["stderr_head"]))
            except (R.Unavailable, subprocess.TimeoutExpired) as e:
                # its GPU path is not run again; the same binary without PICOLM_GPU is its CPU path
                print(f"[bench] the reference's GPU path failed ({e}); running its CPU path", file=sys.stderr)
                gpu = False
                small = R.run(binary, gguf, 16, 8, context, gpu=False, timeout=900)
            for _ in range(max(args.warmup - 1, 0)):
                R.run(binary, gguf, 16, 8, context, gpu=gpu, timeout=900)
            with ClockSampler() as sampler:
                res = R.run(binary, gguf, prefill_tokens, new_tokens, context, gpu=gpu, seed=seed, timeout=1800)
            clocks = sampler.summary()
    except R.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's command line did not finish in its time limit"}))
        return 0
    value = res["gen_tok_s"]
    out = {
        "metric": f"decode tokens/s ({model_name}, bf16, batch 1, 1 B200)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": res["gen_tokens"], "warmup": args.warmup,
        "ms_per_step": round(1e3 / value, 4) if value > 0 else None, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random letter prompts, random-init weights N(0, 0.02)",
        "impl": "reference",
        "config": {"model": model_name, "layers": cfg_dict["num_hidden_layers"], "layers_in_config": full_layers,
                   "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_attention_heads"],
                   "kv_heads": cfg_dict["num_key_value_heads"], "head_dim": cfg_dict["head_dim"],
                   "intermediate": cfg_dict["intermediate_size"], "vocab": cfg_dict["vocab_size"],
                   "tied": cfg_dict["tie_word_embeddings"], "global_batch": 1, "seq_len": context,
                   "prompt_len": res["prefill_tokens"], "prefill_tokens": res["prefill_tokens"],
                   "parallelism": "none (1 GPU)", "backend": res["backend"],
                   "how": "stock picolm CLI (make cuda), PICOLM_GPU=1, -t 0 -s 42; its own Prefill:/Generation: lines"},
        "clocks": clocks,
        # the command line's own timing is end to end: text in, text out, one process
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "prefill_tokens_per_s": res["prefill_tok_s"]},
        "prefill": {"value": res["prefill_tok_s"], "tokens": res["prefill_tokens"], "ms": round(res["prefill_s"] * 1e3, 1)},
        "points": {"decode_b1": value},
        "notes": res["stderr_head"],
    }
    print(json.dumps(out))
    return 0


def prefill_flops(cfg, T):
    d, F, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = 2 * T * d * (H + 2 * G) * hd + 2 * T * H * hd * d + 2 * T * d * 2 * F + 2 * T * F * d
    attn = 2 * 2 * H * hd * T * (T + 1) // 2                     # causal QK^T and PV
    return L * (per_layer + attn) + 2 * d * cfg["vocab_size"]    # LM head on the last row only


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0: all)")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4],
                    help="which of BASELINE.json's configs gives the layer sizes (default 2, the headline)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 decode points")
    ap.add_argument("--unequal", action="store_true",
                    help="also time one step of eight prompts of 128 to 2,048 tokens (always done for a configuration "
                         "that names an unequal batch)")
    ap.add_argument("--long-context", type=int, default=32768,
                    help="with the other points: one request's decode rate after a prompt of this many tokens (0: skip)")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch every kernel of a decode step by itself (for a profiler's launch list)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"picolm_b200 is a one-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    from picolm_b200 import ops
    from picolm_b200.api import generate
    from picolm_b200.config import config_from_dict
    from picolm_b200.engine import Engine
    from picolm_b200.engine.generate import greedy_steps_in_flight
    from picolm_b200.weights import write_random_model

    cfg_dict, context, prompt_len, seed, model_name = bench_config(args.config)
    prefill_tokens = min(2048, context)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_dict)
    pk, pk_src = peaks()
    torch.cuda.set_device(0)
    B = args.batch
    points_b = [] if args.skip_points else [1, 64]
    max_b = max([B] + points_b)

    with tempfile.TemporaryDirectory() as tmp:
        t0 = time.time()
        write_random_model(cfg, seed, tmp, norm_std=0.0)
        # the cache holds what the largest run needs (its prompts, warm-up and timed steps), not
        # max_b full contexts: at the 13B shape those would not fit the GPU
        need = max(prompt_len, prefill_tokens) + 2 * args.warmup + 3 * args.steps + 16
        per_seq = min(context, max((need + 63) // 64 * 64, prompt_len + 1536))
        kv_tok = 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2
        while max_b * per_seq * kv_tok > 70e9 and per_seq > (need + 63) // 64 * 64:   # leave room for the weights
            per_seq -= 64
        engine = Engine.from_folder(tmp, dtype="bfloat16", max_tokens=max_b * per_seq, max_seqs=max_b,
                                    max_seq_tokens=context, use_graphs=False if args.no_graphs else None)
    print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr)
    g = torch.Generator().manual_seed(seed)
    vocab = cfg.vocab_size

    def prompts(n, length=None):
        return [torch.randint(0, vocab, (length or prompt_len,), generator=g).tolist() for _ in range(n)]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------------------------------------------------------- prefill
    # Timed two ways, each against the peak that was measured the same way.  By itself: the device idle for
    # IDLE_S before every step, as one prompt arrives at a server that is not busy; its fraction is of the burst
    # GEMM rate (a kernel timed in isolation).  Back to back: the steps one after another without a pause, which
    # the power cap slows down; its fraction is of what a long library loop sustains.
    IDLE_S, reps = 0.02, 20
    flops = prefill_flops(cfg_dict, prefill_tokens)

    def prefill_times(idle_s):
        ps = [prompts(1, prefill_tokens)[0] for _ in range(args.warmup + reps)]
        times = []
        for i, p in enumerate(ps):
            s = engine.new_sequence()
            a, b = ev(), ev()
            torch.cuda.synchronize()
            if idle_s:
                time.sleep(idle_s)
            a.record()
            engine.step([(s, p)])
            b.record()
            torch.cuda.synchronize()
            engine.end_sequence(s)
            if i >= args.warmup:
                times.append(a.elapsed_time(b))
        return times

    times = prefill_times(IDLE_S)
    pf_ms = statistics.median(times)
    prefill = {"value": round(prefill_tokens / pf_ms * 1e3, 1), "tokens": prefill_tokens, "ms": round(pf_ms, 3),
               "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "ms_min_max": [round(min(times), 3), round(max(times), 3)], "from_graph": bool(engine._prompt_graphs),
               "idle_before_each_ms": IDLE_S * 1e3}
    times = prefill_times(0.0)
    bb_ms = statistics.median(times)
    prefill["back_to_back"] = {"value": round(prefill_tokens / bb_ms * 1e3, 1), "ms": round(bb_ms, 3),
                               "frac": round(flops / (bb_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                               "ms_min_max": [round(min(times), 3), round(max(times), 3)]}
    if "bf16_tflops_sustained" in pk:       # against what a long cuBLAS loop sustains under the power cap
        prefill["back_to_back"]["frac_of_sustained"] = round(flops / (bb_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    # ----------------------------------------------------------------- decode
    w_bytes = engine.model.weight_bytes_per_step()
    kv_per_token = engine.cache.kv_bytes_per_token()

    def decode_run(batch, steps, warmup, sample_clocks=False):
        """Decode at `batch` after prompts of `prompt_len`: `warmup` steps, then untimed steps for at least
        UNTIMED_S (the clocks dip after the prompts' step and come back), then R blocks of `steps` steps,
        each block between two events, the blocks back to back without the host waiting in between; R is
        chosen so that the blocks last at least TIMED_S together (as far as the context allows).  The median
        block gives the step's time whatever `steps` is.  The timed steps feed each sampled token to the next
        step on the device; the ids reach the host by a copy per step that nobody waits for until the end
        (`greedy_steps_in_flight`, which the tests compare with `generate`)."""
        UNTIMED_S, TIMED_S = 0.2, 0.5
        slots = [engine.new_sequence() for _ in range(batch)]
        ps = prompts(batch)
        toks = []
        for lo in range(0, batch, 8):                            # prompts in, eight sequences at a time
            logits = engine.step([(slots[i], ps[i]) for i in range(lo, min(lo + 8, batch))])
            toks += ops.argmax(logits).tolist()
        for _ in range(warmup):
            toks = ops.argmax(engine.step([(s, [t]) for s, t in zip(slots, toks)])).tolist()
        room = per_seq - prompt_len - warmup - 2                 # steps the cache still has room for
        tok_dev = torch.tensor(toks, dtype=torch.int32, device="cuda:0")
        # a first look at the step's time, to size what follows
        probe = max(1, min(8, room // 8))
        pinned = torch.empty((max(room, 1), batch), dtype=torch.int32).pin_memory()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        tok_dev = greedy_steps_in_flight(engine, slots, tok_dev, probe, pinned)
        b.record()
        torch.cuda.synchronize()
        est_ms = max(a.elapsed_time(b) / probe, 1e-3)
        room -= probe
        steps = max(1, min(steps, room // 2))
        untimed = max(0, min(int(UNTIMED_S * 1e3 / est_ms) + 1, room - steps))
        blocks = max(1, min(int(TIMED_S * 1e3 / (est_ms * steps)) + 1, (room - untimed) // steps))
        tok_dev = greedy_steps_in_flight(engine, slots, tok_dev, untimed, pinned)
        n0 = ops.launch_count()
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        marks = [ev() for _ in range(blocks + 1)]
        torch.cuda.synchronize()
        marks[0].record()
        for r in range(blocks):
            tok_dev = greedy_steps_in_flight(engine, slots, tok_dev, steps, pinned[r * steps:])
            marks[r + 1].record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        per_block = [marks[r].elapsed_time(marks[r + 1]) / steps for r in range(blocks)]
        ms = statistics.median(per_block)
        launches = (ops.launch_count() - n0) // blocks           # of one block of `steps` steps
        ctx_mean = prompt_len + warmup + probe + untimed + (blocks * steps + 1) / 2.0
        for s in slots:
            engine.end_sequence(s)
        achieved = (w_bytes + kv_per_token * ctx_mean * batch) / (ms * 1e-3) / 1e9
        return {"ms": ms, "launches": launches, "ctx_mean": ctx_mean, "achieved": achieved,
                "clocks": sampler.summary() if sampler else None, "steps": steps, "blocks": blocks,
                "untimed_steps": warmup + probe + untimed,
                "block_ms": [round(min(per_block), 4), round(ms, 4), round(max(per_block), 4)]}

    run = decode_run(B, args.steps, args.warmup, sample_clocks=True)
    ms, launches, clocks = run["ms"], run["launches"], run["clocks"]
    value = B / ms * 1e3
    roofline = {"bound": "hbm", "achieved": round(run["achieved"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(run["achieved"] / pk["hbm_gbs"], 4), "peaks": pk_src}
    points, points_frac = {}, {}
    for pb in points_b:
        pr = decode_run(pb, args.steps, args.warmup)
        points[f"decode_b{pb}"] = round(pb / pr["ms"] * 1e3, 1)
        points_frac[f"decode_b{pb}"] = round(pr["achieved"] / pk["hbm_gbs"], 4)

    # One request far into its context: the decode rate after a long prompt (an engine of its own, one sequence).
    n_long = args.long_context
    if n_long and not args.skip_points and n_long + 512 <= cfg.max_position_embeddings:
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(cfg, seed, tmp, norm_std=0.0)
            room = n_long + 512
            long_engine = Engine.from_folder(tmp, dtype="bfloat16", max_tokens=room, max_seqs=1, max_seq_tokens=room,
                                             use_graphs=False if args.no_graphs else None)
        long_prompt = prompts(1, n_long)[0]
        slot = long_engine.new_sequence()
        long_engine.step([(slot, long_prompt)])                    # untimed: the first step of this length
        long_engine.end_sequence(slot)
        slot = long_engine.new_sequence()                          # the same prompt again, as one timed step
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        long_logits = long_engine.step([(slot, long_prompt)])
        b.record()
        torch.cuda.synchronize()
        points[f"prefill_t{n_long}"] = round(n_long / a.elapsed_time(b) * 1e3, 1)
        points_frac[f"prefill_t{n_long}"] = round(
            prefill_flops(cfg_dict, n_long) / (a.elapsed_time(b) * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        tok = ops.argmax(long_logits).tolist()
        for _ in range(args.warmup):
            tok = ops.argmax(long_engine.step([(slot, tok)])).tolist()
        tok_dev = torch.tensor(tok, dtype=torch.int32, device="cuda:0")
        pinned = torch.empty((256, 1), dtype=torch.int32).pin_memory()
        tok_dev = greedy_steps_in_flight(long_engine, [slot], tok_dev, 64, pinned)      # the classes' graphs, the clocks
        per_block = []
        for r in range(4):
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            tok_dev = greedy_steps_in_flight(long_engine, [slot], tok_dev, 32, pinned)
            b.record()
            torch.cuda.synchronize()
            per_block.append(a.elapsed_time(b) / 32)
        lms = statistics.median(per_block)
        ctx_mean = n_long + args.warmup + 64 + 64
        long_engine.end_sequence(slot)
        points[f"decode_b1_ctx{n_long}"] = round(1e3 / lms, 1)
        points_frac[f"decode_b1_ctx{n_long}"] = round(
            (w_bytes + long_engine.cache.kv_bytes_per_token() * ctx_mean) / (lms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        del long_engine
        torch.cuda.empty_cache()

    # The unequal batch that the 8B configuration names: prompts of 128 to 2,048 tokens in one step.
    if "Unequal batch" in baseline_text(args.config) or args.unequal:
        lens = [128 + (2048 - 128) * i // 7 for i in range(8)]
        lens = [min(n, per_seq) for n in lens]
        times = []
        for i in range(3 + 10):
            slots = [engine.new_sequence() for _ in lens]
            ps = [prompts(1, n)[0] for n in lens]
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            engine.step(list(zip(slots, ps)))
            b.record()
            torch.cuda.synchronize()
            for sl in slots:
                engine.end_sequence(sl)
            if i >= 3:
                times.append(a.elapsed_time(b))
        ums = statistics.median(times)
        total = sum(lens)
        uflops = sum(prefill_flops(cfg_dict, n) for n in lens)
        points["prefill_unequal_128_2048"] = round(total / ums * 1e3, 1)
        points_frac["prefill_unequal_128_2048"] = round(uflops / (ums * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)

    # ------------------------------------------- end to end, host ids in and out
    # long enough to outlast the clock dip after the prompts' step: about a second of decoding, as far as the
    # cache has room
    gen_new = max(args.warmup + 2 * args.steps, int(1000.0 / ms))
    gen_new = max(8, min(gen_new, per_seq - prompt_len - 2))
    ps = prompts(B)
    # warm-up over the same lengths: decode steps are captured per length class, and a service has its classes captured
    generate(engine, ps, max_tokens=gen_new, temperature=0.0, stop_ids=[], max_batch=B)
    engine.reset_counters()
    outs, stats = generate(engine, ps, max_tokens=gen_new, temperature=0.0, stop_ids=[], max_batch=B,
                           return_stats=True)
    c = engine.counters
    e2e = {"value": round((stats.generated_tokens - B) / stats.generation_seconds, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(c["h2d_bytes"] / max(c["steps"], 1)),
           "d2h_bytes_per_step": int(c["d2h_bytes"] / max(c["steps"], 1)),
           "prefill_tokens_per_s": round(stats.prefill_tokens / stats.prefill_seconds, 1)}

    out = {
        "metric": f"decode tokens/s ({model_name}, bf16, batch {B}, 1 B200)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random token ids, random-init weights N(0, 0.02)", "impl": "ours",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_in_config": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": B, "seq_len": context, "prompt_len": prompt_len,
                   "prefill_tokens": prefill_tokens, "parallelism": "none (1 GPU)",
                   "l2": f"every step reads all weights ({w_bytes / 1e9:.1f} GB > 126 MB L2); no flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "points_roofline": points_frac,
        "window": {"blocks": run["blocks"], "steps_per_block": run["steps"], "untimed_steps_before": run["untimed_steps"],
                   "block_ms_min_median_max": run["block_ms"]},
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
