"""Ways of cutting the same requests into steps, run through the engine."""
import torch


def run_whole(engine, tokens):
    """One request alone, all its tokens in one step, logits everywhere."""
    s = engine.new_sequence()
    try:
        return engine.step([(s, tokens)], [list(range(len(tokens)))]).float().cpu()
    finally:
        engine.end_sequence(s)


def run_tail(engine, tokens, tail=32):
    """All but the last `tail` tokens in one step, then the rest one by one.
    Returns logits [T, vocab] like run_whole."""
    s = engine.new_sequence()
    try:
        head = len(tokens) - tail
        out = []
        if head > 0:
            out.append(engine.step([(s, tokens[:head])], [list(range(head))]).float().cpu())
        for t in tokens[max(head, 0):]:
            out.append(engine.step([(s, [t])], [[0]]).float().cpu())
        return torch.cat(out, dim=0)
    finally:
        engine.end_sequence(s)


def run_batch(engine, requests, prompt_lens):
    """Requests that start together: prompts of `prompt_lens` tokens in one
    step, then one token each from the request's own continuation; a request
    leaves the batch when its tokens are used up.  Returns for each request its
    logits [T, vocab]."""
    slots = [engine.new_sequence() for _ in requests]
    outs = [[] for _ in requests]
    try:
        entries = [(slots[i], r[:n]) for i, (r, n) in enumerate(zip(requests, prompt_lens))]
        wants = [list(range(n)) for n in prompt_lens]
        logits = engine.step(entries, wants).float().cpu()
        o = 0
        for i, n in enumerate(prompt_lens):
            outs[i].append(logits[o:o + n])
            o += n
        pos = list(prompt_lens)
        live = [i for i, r in enumerate(requests) if pos[i] < len(r)]
        while live:
            logits = engine.step([(slots[i], [requests[i][pos[i]]]) for i in live], [[0]] * len(live)).float().cpu()
            for row, i in enumerate(live):
                outs[i].append(logits[row:row + 1])
                pos[i] += 1
            live = [i for i in live if pos[i] < len(requests[i])]
        return [torch.cat(o, dim=0) for o in outs]
    finally:
        for s in slots:
            engine.end_sequence(s)


def run_chunks(engine, tokens, sizes):
    """One request fed in pieces of `sizes` tokens (several tokens at a time after a cached prefix: the
    prompt kernels with a start position).  Returns logits [T, vocab] like run_whole."""
    assert sum(sizes) == len(tokens)
    s = engine.new_sequence()
    try:
        out, o = [], 0
        for n in sizes:
            out.append(engine.step([(s, tokens[o:o + n])], [list(range(n))]).float().cpu())
            o += n
        return torch.cat(out, dim=0)
    finally:
        engine.end_sequence(s)
