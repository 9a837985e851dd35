"""The command line, after the reference's (picolm/picolm.c:140-196, parsed at
picolm/picolm.c:820-940): a positional model path, `-p` prompt (or standard
input), `-n` max tokens, `-t` temperature, `-k` top-k, `--top-p`, `-s` seed, `-c`
context.  There is no tokenizer here, so a prompt is token ids separated by
commas or blanks; several prompts (one per line, or separated by ';' in `-p`)
run as batches.  Generated ids go to standard output, one line per prompt; the
reference's `Prefill:` / `Generation:` lines go to standard error
(picolm/picolm.c:1629-1636).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from typing import List


def parse_prompts(text: str) -> List[List[int]]:
    prompts = []
    for chunk in re.split(r"[;\n]", text):
        ids = [int(t) for t in re.split(r"[,\s]+", chunk.strip()) if t]
        if ids:
            prompts.append(ids)
    return prompts


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(
        prog="picolm_b200",
        description="picolm_b200 - Llama inference on one B200 (token ids in, token ids out)")
    ap.add_argument("model", nargs="?", help="model folder (config.json + model.safetensors)")
    g = ap.add_argument_group("Generation options")
    g.add_argument("-p", dest="prompt", help="input prompt as token ids, e.g. \"1,15,27\" (or pipe via stdin); "
                                             "';' or newlines separate several prompts")
    g.add_argument("-n", dest="max_tokens", type=int, default=256, help="max tokens to generate (default: 256)")
    g.add_argument("-t", dest="temperature", type=float, default=0.8, help="temperature (default: 0.8, 0=greedy)")
    g.add_argument("-k", dest="top_k", type=int, default=40, help="top-k sampling (default: 40, 0=off)")
    g.add_argument("--top-p", dest="top_p", type=float, default=0.9, help="top-p / nucleus sampling (default: 0.9)")
    g.add_argument("--min-p", dest="min_p", type=float, default=0.05,
                   help="drop tokens below min-p times the top probability (default: 0.05)")
    g.add_argument("-s", dest="seed", type=int, default=42, help="RNG seed (default: 42)")
    g.add_argument("-c", dest="context", type=int, default=0, help="context length override")
    g.add_argument("--stop-id", dest="stop_ids", type=int, action="append",
                   help="stop at this token id (default: the model's eos_token_id); may be repeated")
    e = ap.add_argument_group("Engine options")
    e.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="bfloat16 (serving kernels) or float32 (everything in true 32-bit)")
    e.add_argument("--max-batch", type=int, default=8, help="most sequences generated together (default: 8)")
    b = ap.add_argument_group("Benchmark options")
    b.add_argument("--benchmark", action="store_true",
                   help="benchmark mode: the prompt's step and -n decode steps with the time of every layer "
                        "(three iterations; per-layer ms and effective weight GB/s on standard error)")
    b.add_argument("--benchmark-ctx", action="store_true",
                   help="benchmark prefill+gen speed at growing context sizes: the prompt (-p) is prefilled again and "
                        "again behind what is already cached, -n tokens are generated after each, up to the context (-c)")
    i = ap.add_argument_group("Info options")
    i.add_argument("--list-tensors", action="store_true", help="list all tensors (name, shape, type) and exit")
    r = ap.add_argument_group("Random weights")
    r.add_argument("--random-weights", metavar="CONFIG_JSON",
                   help="write a model folder with random weights for this config.json and exit")
    r.add_argument("--out", help="folder to write with --random-weights")
    return ap


def benchmark_context_scaling(args, base: List[int]) -> int:
    """The reference's `--benchmark-ctx` (picolm/picolm.c:416-553): one sequence whose cache keeps growing;
    every round prefills the base prompt behind what is cached, then generates `-n` tokens greedily, and
    prints `ctx_size,prefill_tok/s,gen_tok/s` (the cached length before the round) to standard error."""
    import time

    from . import ops
    from .api import model_load
    engine = model_load(args.model, dtype=args.dtype, context=args.context or None, max_batch=1)
    limit = engine.cache.max_seq_tokens
    n_base, chunk = len(base), max(1, args.max_tokens)
    print(f"Base prompt: {n_base} tokens", file=sys.stderr)
    print("ctx_size,prefill_tok/s,gen_tok/s", file=sys.stderr)
    slot = engine.new_sequence()
    try:
        while engine.length(slot) + n_base + chunk <= limit:
            cached = engine.length(slot)
            engine.synchronize()
            t0 = time.perf_counter()
            tok = ops.argmax(engine.step([(slot, base)]))
            engine.synchronize()
            t1 = time.perf_counter()
            for _ in range(chunk):
                tok = ops.argmax(engine.step_device_tokens([slot], tok), out=engine.token_buffer(1))
            engine.synchronize()
            t2 = time.perf_counter()
            print(f"{cached},{n_base / (t1 - t0):.1f},{chunk / (t2 - t1):.1f}", file=sys.stderr)
    finally:
        engine.end_sequence(slot)
    return 0


def layer_times(marks, n_runs: int) -> List[float]:
    """Mean milliseconds of every run of the schedule from (run, elapsed ms) pairs of one or more steps."""
    total, count = [0.0] * n_runs, [0] * n_runs
    for run, ms in marks:
        total[run] += ms
        count[run] += 1
    return [t / c if c else 0.0 for t, c in zip(total, count)]


def benchmark_layers(args, base: List[int], iterations: int = 3) -> int:
    """The reference's `--benchmark` (picolm/picolm.c:1364-1475; its per-layer callback picolm/picolm.c:251-383):
    the prompt in one step, then `-n` tokens greedily, with the time of every layer taken by events around it
    (`Model.layer_hook`; the steps are launched kernel by kernel, not replayed from graphs).  Every iteration
    starts from an empty cache and prints, per layer, the milliseconds in the prompt's step, the mean
    milliseconds in a decode step and the rate at which the decode step reads the layer's weights; then the
    reference's `Prefill:` / `Generation:` lines.  (In a decode step a layer hands its last product to the norm that
    follows, so that product's time is counted with the next layer, the last layer's with none.)  The reference loops until it is interrupted; this runs
    `iterations` times (the first includes whatever is compiled or set up at first use)."""
    import time

    import torch

    from . import ops
    from .api import model_load
    engine = model_load(args.model, dtype=args.dtype, context=args.context or None, max_batch=1)
    model = engine.model
    n_runs = len(model.spec.schedule)
    n_new = max(0, min(args.max_tokens, engine.cache.max_seq_tokens - len(base)))
    weight_mb = [sum(part.weight_bytes() for _, part in model.blocks[i].parts()) / 1e6 for i in model.spec.schedule]
    events, started = [], {}

    def hook(run: int, layer: int, done: bool) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        if done:
            events.append((run, started.pop(run), e))
        else:
            started[run] = e

    def collect():
        engine.synchronize()
        out = [(run, a.elapsed_time(b)) for run, a, b in events]
        events.clear()
        return out

    try:
        model.layer_hook = hook
        for it in range(1, iterations + 1):
            slot = engine.new_sequence()
            try:
                engine.synchronize()
                t0 = time.perf_counter()
                tok = ops.argmax(engine.step([(slot, base)]))
                prefill = layer_times(collect(), n_runs)
                t1 = time.perf_counter()
                for _ in range(n_new):
                    tok = ops.argmax(engine.step_device_tokens([slot], tok), out=engine.token_buffer(1))
                decode = layer_times(collect(), n_runs)
                t2 = time.perf_counter()
            finally:
                engine.end_sequence(slot)
            print(f"=== iteration {it}: {len(base)} prompt tokens, {n_new} generated", file=sys.stderr)
            print("layer,prefill_ms,gen_ms,weight_MB,gen_weight_GB/s", file=sys.stderr)
            for run, i in enumerate(model.spec.schedule):
                rate = weight_mb[run] / decode[run] if decode[run] > 0 else 0.0          # MB / ms = GB/s
                print(f"{i},{prefill[run]:.3f},{decode[run]:.4f},{weight_mb[run]:.1f},{rate:.0f}", file=sys.stderr)
            print(f"layers: prefill {sum(prefill):.2f} ms, gen {sum(decode):.3f} ms a token", file=sys.stderr)
            pf, gn = t1 - t0, t2 - t1
            print(f"Prefill: {len(base)} tokens in {pf:.2f}s ({len(base) / pf if pf > 0 else 0:.1f} tok/s)", file=sys.stderr)
            print(f"Generation: {n_new} tokens in {gn:.2f}s ({n_new / gn if gn > 0 else 0:.1f} tok/s)", file=sys.stderr)
    finally:
        model.layer_hook = None
    return 0


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)

    if args.random_weights:
        if not args.out:
            ap.error("--random-weights needs --out DIR")
        from . import architectures  # noqa: F401
        from .config.registry import read_config
        from .weights import write_random_model
        write_random_model(read_config(args.random_weights), args.seed, args.out)
        print(f"wrote {args.out}", file=sys.stderr)
        return 0

    if not args.model:
        ap.print_usage(sys.stderr)
        return 1

    if args.list_tensors:
        from .weights import Checkpoint
        ck = Checkpoint(args.model)
        for name in sorted(ck.names()):
            ent = ck.entries[name]
            print(f"{name}\t{list(ent.shape)}\t{ent.dtype}")
        return 0

    text = args.prompt if args.prompt is not None else sys.stdin.read()
    try:
        prompts = parse_prompts(text)
    except ValueError as e:
        print(f"prompt must be token ids: {e}", file=sys.stderr)
        return 1
    if not prompts:
        print("no prompt given (-p \"1,2,3\" or token ids on stdin)", file=sys.stderr)
        return 1

    if args.benchmark_ctx:
        return benchmark_context_scaling(args, prompts[0])
    if args.benchmark:
        return benchmark_layers(args, prompts[0])

    from .api import generate, model_load
    engine = model_load(args.model, dtype=args.dtype, context=args.context or None,
                        max_batch=min(args.max_batch, len(prompts)))
    outputs, stats = generate(engine, prompts, max_tokens=args.max_tokens, temperature=args.temperature,
                              top_p=args.top_p, top_k=args.top_k, min_p=args.min_p, seed=args.seed,
                              stop_ids=args.stop_ids, return_stats=True)
    for out in outputs:
        print(" ".join(str(t) for t in out))
    sys.stdout.flush()
    pf, gn = stats.prefill_seconds, stats.generation_seconds
    print("---", file=sys.stderr)
    print(f"Prefill: {stats.prefill_tokens} tokens in {pf:.2f}s ({stats.prefill_tokens / pf if pf > 0 else 0:.1f} tok/s)",
          file=sys.stderr)
    print(f"Generation: {stats.generated_tokens} tokens in {gn:.2f}s "
          f"({stats.generated_tokens / gn if gn > 0 else 0:.1f} tok/s)", file=sys.stderr)
    print(f"Total: {pf + gn:.2f}s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
